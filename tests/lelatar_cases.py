"""Small Lelatar configurations for the tests, model folders with seeded random weights, and a driver
that runs a schedule of steps through the engine in this process."""
import copy
import os

import numpy as np
import torch
from safetensors.torch import load_file, save_file

from helpers import Trace


def mamba(conv=4, groups=1, heads=4, norm_groups=1, state=16, vdim=16, mlp=None):
    return {"type": "mamba2", "mlp": mlp,
            "mixer": {"conv": conv, "groups": groups, "heads": heads, "norm_groups": norm_groups, "state": state, "vdim": vdim}}


def parallel(left, right, mlp=None):
    return {"type": "parallel", "mlp": mlp, "mixer": {"left": left, "right": right}}


def left(dim=32, heads=4, kv_heads=2, vdim=16, rot_dims=16, base=10000.0, scale=0.2):
    return {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim, "scale": scale, "rot": {"base": base, "dims": rot_dims}}


def right(conv=3, dim=16, heads=4, kv_heads=4, vdim=24):
    return {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim}


DENSE = lambda ff: {"ff": ff, "kind": "dense"}

# Different in every size from one another; sizes that are equal or 1 in one are not in the other.
CONFIG_P = {"architecture": "Lelatar", "vocab": 96, "width": 64, "norm": {"eps": 1e-5}, "token_side": {"dim": 8},
            "loop": {"start": 0, "stop": 2, "times": 2},
            "layers": [parallel(left(), right(), mlp=DENSE(80)), mamba()]}
CONFIG_Q = {"architecture": "Lelatar", "vocab": 200, "width": 96, "norm": {"eps": 1e-6},
            "loop": {"start": 1, "stop": 3, "times": 3},
            "layers": [mamba(conv=2, groups=2, heads=4, norm_groups=4, state=24, vdim=8, mlp=DENSE(128)),
                       mamba(conv=3, groups=4, heads=4, norm_groups=2, state=8, vdim=24),
                       parallel(left(dim=64, heads=2, kv_heads=1, vdim=64, rot_dims=64, base=500.0, scale=0.125),
                                right(conv=4, dim=32, heads=2, kv_heads=1, vdim=48)),
                       mamba(conv=4, groups=1, heads=2, norm_groups=1, state=40, vdim=32)]}
# no loop, a side input narrower than a 16-byte row, value heads wider than key heads, no rotation
CONFIG_R = {"architecture": "Lelatar", "vocab": 64, "width": 48, "norm": {"eps": 1e-5}, "token_side": {"dim": 4},
            "layers": [parallel(left(dim=16, heads=3, kv_heads=3, vdim=32, rot_dims=0, scale=0.3),
                                right(conv=2, dim=24, heads=3, kv_heads=1, vdim=16))]}
# heads of 48 (stored 48 wide), three groups, a span in the middle that runs twice, five layers
CONFIG_S = {"architecture": "Lelatar", "vocab": 300, "width": 192, "norm": {"eps": 1e-5}, "token_side": {"dim": 24},
            "loop": {"start": 1, "stop": 3, "times": 2},
            "layers": [mamba(conv=4, groups=3, heads=6, norm_groups=3, state=64, vdim=32),
                       parallel(left(dim=48, heads=6, kv_heads=3, vdim=48, rot_dims=24, base=500000.0, scale=0.15),
                                right(conv=3, dim=48, heads=6, kv_heads=2, vdim=16), mlp=DENSE(256)),
                       mamba(conv=4, groups=3, heads=6, norm_groups=3, state=64, vdim=32, mlp=DENSE(256)),
                       parallel(left(dim=48, heads=6, kv_heads=3, vdim=48, rot_dims=24, base=500000.0, scale=0.15),
                                right(conv=3, dim=48, heads=6, kv_heads=2, vdim=16)),
                       mamba(conv=4, groups=3, heads=6, norm_groups=3, state=64, vdim=32)]}
# wide heads and a large state: 128-wide attention heads, a state of 256 rows (sixteen threads a column)
CONFIG_T = {"architecture": "Lelatar", "vocab": 128, "width": 128, "norm": {"eps": 1e-5},
            "layers": [mamba(conv=4, groups=1, heads=2, norm_groups=2, state=256, vdim=16),
                       parallel(left(dim=128, heads=2, kv_heads=1, vdim=96, rot_dims=64, base=10000.0, scale=0.09),
                                right(conv=4, dim=128, heads=2, kv_heads=2, vdim=64), mlp=DENSE(192))]}
ONLY_MAMBA = {"architecture": "Lelatar", "vocab": 64, "width": 48, "norm": {"eps": 1e-5},
              "layers": [mamba(conv=4, groups=2, heads=6, norm_groups=3, state=20, vdim=8)]}


def vocab_of(config):
    return config["vocab"]


BRANCH_GAIN = 0.3


def calm(w):
    """Every branch adds to the stream with a gain of BRANCH_GAIN instead of about 1: a random model of a few dozen
    columns otherwise turns the rounding of bfloat16 products into differences of a third of a logit, against
    which a fault would not stand out.  (Gains of the normed branch outputs, and the last matrix of the others.)"""
    for k in w:
        if k.endswith((".left.out", ".right.out", ".side.norm", ".mlp.down")) or (k.endswith(".mix.o") and ".left" not in k and ".right" not in k):
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


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def run_engine(model, trace: Trace, page_size=16, n_pages=64, max_requests=4, max_len=1024, engine=None):
    """The trace's steps through ``Engine.step``: ``{(request, position): float32 row}``."""
    from mlx_lm_b200.engine import Engine, StepEntry

    eng = engine or Engine(model, page_size=page_size, n_pages=n_pages, max_requests=max_requests, max_len=max_len)
    got = {}
    for s, rows in zip(trace.steps, trace.rows):
        entries = []
        for e in s["entries"]:
            if not eng.has_request(e["id"]):
                eng.add_request(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        logits = eng.step(entries)
        if rows:
            a = logits.float().cpu().numpy()
            for key, row in zip(rows, a):
                got[key] = row
        eng.check_status()
        for rid in s["end"]:
            eng.finish(rid)
        eng.cache.check()
    return got


def worst(got, ref_by_request):
    """Largest |difference| over all rows, as a fraction of max(1, largest |reference logit| of the row).
    ``ref_by_request``: ``name -> [T, vocab]``; a request ``name:tag`` is compared with ``name``."""
    w = 0.0
    for (rid, pos), row in got.items():
        ref = ref_by_request[rid.split(":")[0]][pos].numpy()
        w = max(w, float(np.abs(row - ref).max() / max(1.0, np.abs(ref).max())))
    return w
