"""Small Nufetar configurations for the tests and model folders with seeded random weights."""
import copy
import os

import torch
from safetensors.torch import load_file, save_file


def attention(dim=32, heads=4, kv_heads=2, vdim=16, rot_dims=16, base=10000.0, scale=0.2, chunk=24, mlp=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim, "scale": scale,
                      "mask": {"size": chunk}, "rot": {"base": base, "dims": rot_dims}}}


def latent(dim=16, heads=4, kv_rank=24, rot_dim=8, vdim=24, base=10000.0, scale=0.25, window=20, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"dim": dim, "heads": heads, "kv_rank": kv_rank, "rot_dim": rot_dim, "vdim": vdim, "scale": scale,
                      "mask": {"size": window}, "rot": {"base": base, "dims": rot_dim}}}


def wkv(dim=32, heads=2, decay_rank=8, mlp=None):
    return {"type": "wkv", "mlp": mlp, "mixer": {"dim": dim, "heads": heads, "decay_rank": decay_rank}}


DENSE = lambda ff: {"ff": ff, "kind": "dense"}


def model(vocab, width, layers, eps=1e-5):
    return {"architecture": "Nufetar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# Different from one another in every size; what is equal or 1 in one is not in the others.
CONFIG_A = model(96, 64, [attention(mlp=DENSE(80)), latent(mlp=DENSE(48)), wkv(), attention(chunk=50, mlp=DENSE(80))])
# all heads with keys of their own and whole heads rotated; one latent head that sees itself and one token more;
# a state of 48 rows (three of four threads of a column have rows); a feed-forward wider than the model
CONFIG_B = model(200, 96, [wkv(dim=48, heads=3, decay_rank=5, mlp=DENSE(256)),
                           latent(dim=24, heads=1, kv_rank=40, rot_dim=16, vdim=40, base=500.0, scale=0.2, window=2),
                           attention(dim=48, heads=3, kv_heads=3, vdim=40, rot_dims=48, base=500.0, scale=0.15, chunk=100,
                                     mlp=DENSE(128)),
                           latent(dim=8, heads=6, kv_rank=64, rot_dim=32, vdim=16, base=1e6, scale=0.3, window=33)],
                 eps=1e-6)
# one key/value head for six query heads, runs of 7 positions (no multiple of a page), a latent row that is no
# multiple of 16 bytes, five small recurrent heads, a window longer than most prompts, no rotation in the first layer
CONFIG_C = model(130, 80, [attention(dim=16, heads=6, kv_heads=1, vdim=24, rot_dims=0, scale=0.25, chunk=7),
                           wkv(dim=16, heads=5, decay_rank=16, mlp=DENSE(96)),
                           latent(dim=32, heads=2, kv_rank=30, rot_dim=6, vdim=12, scale=0.18, window=300, mlp=DENSE(96)),
                           attention(dim=64, heads=2, kv_heads=2, vdim=8, rot_dims=32, base=250000.0, scale=0.125, chunk=64)])
# sizes of a larger model's heads: eight heads of 64, a latent row of 320, a state of 128 rows (eight threads a column)
CONFIG_W = model(128, 128, [attention(dim=64, heads=8, kv_heads=2, vdim=64, rot_dims=32, scale=0.125, chunk=128, mlp=DENSE(192)),
                            latent(dim=64, heads=4, kv_rank=256, rot_dim=64, vdim=64, scale=0.09, window=100),
                            wkv(dim=128, heads=2, decay_rank=32, mlp=DENSE(192))])
# nothing is a multiple of 8: every 16-byte path steps aside (products, pages, staging, the tensor-core attention)
CONFIG_ODD = model(77, 50, [attention(dim=12, heads=3, kv_heads=1, vdim=10, rot_dims=6, scale=0.3, chunk=9, mlp=DENSE(30)),
                            latent(dim=6, heads=3, kv_rank=20, rot_dim=4, vdim=10, scale=0.3, window=11),
                            wkv(dim=12, heads=3, decay_rank=3, mlp=DENSE(30))])
ONLY_ATTENTION = model(64, 48, [attention(dim=16, heads=4, kv_heads=2, vdim=16, rot_dims=8, scale=0.25, chunk=40)])
ONLY_LATENT = model(64, 48, [latent(dim=16, heads=3, kv_rank=16, rot_dim=8, vdim=16, scale=0.25, window=30)])
ONLY_WKV = model(64, 48, [wkv(dim=16, heads=3, decay_rank=4)])

BRANCH_GAIN = 0.3


def calm(w):
    """Every branch adds to the stream with a gain of BRANCH_GAIN instead of about 1: a random model of a few dozen
    columns otherwise turns the rounding of bfloat16 products into differences of a third of a logit, against
    which a fault would not stand out."""
    for k in w:
        if k.endswith((".mlp.down", ".mix.o")):
            w[k] *= BRANCH_GAIN


def make_dir(path, config, seed, edit=None, calmed=True):
    """A model folder with random weights; ``edit(tensors)`` may change them (float32 in, rounded to bfloat16 again)."""
    from mlx_lm_b200.weights import write_random_model

    write_random_model(str(path), copy.deepcopy(config), seed)
    file = os.path.join(str(path), "model.safetensors")
    w = {k: v.float() for k, v in load_file(file).items()}
    if calmed:
        calm(w)
    if edit is not None:
        edit(w)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, file)
    return load_file(file)


def sharpen(w, factor):
    """Queries scaled up so that single scores stand out: a key that is lost, or one too many, moves the logits."""
    for k in w:
        if k.endswith((".mix.q", ".mix.q.b")):
            w[k] *= factor


def with_mask(config, layer, size):
    c = copy.deepcopy(config)
    c["layers"][layer]["mixer"]["mask"]["size"] = size
    return c
