"""Nufetar, plainly: the whole sequence at once, dense masks, explicit loops, torch on the CPU.

One function per mechanism, written from the equations; nothing here is shared with the engine.  ``weights``
maps tensor names to tensors (any float dtype); everything is computed in ``dtype`` (float64 by default).

    rms(x)              x / sqrt(mean(x^2) + eps)
    turn_halves / turn_neighbours   rotation by position of pairs (i, i + n/2) / (2i, 2i + 1)
    talking_attention   grouped-query attention, value heads unit-RMS, scores mixed across heads, chunks, head gates
    latent_attention    keys and values expanded from a normed latent vector, a rotated key part shared by the heads
    wkv                 token shift, data-dependent decay, the recurrence with a bonus for the current token
    xielu               the feed-forward's activation with two learned numbers
"""
import math

import torch
import torch.nn.functional as F


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def angles(n_pairs, n_dims, base, positions, dtype):
    freq = torch.tensor([base ** (-2.0 * i / n_dims) for i in range(n_pairs)], dtype=dtype)
    a = positions.to(dtype)[:, None] * freq[None, :]            # [T, pairs]
    return torch.cos(a), torch.sin(a)


def turn_halves(x, n_dims, base, positions):
    """x [T, heads, d]: the first n_dims dimensions of every head turn, dimension i with i + n_dims/2."""
    if n_dims == 0:
        return x
    h = n_dims // 2
    cos, sin = angles(h, n_dims, base, positions, x.dtype)
    cos, sin = cos[:, None, :], sin[:, None, :]
    u, v = x[..., :h], x[..., h:n_dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., n_dims:]], dim=-1)


def turn_neighbours(x, n_dims, base, positions):
    """x [T, heads, d]: the first n_dims dimensions of every head turn, dimension 2i with 2i + 1."""
    if n_dims == 0:
        return x
    cos, sin = angles(n_dims // 2, n_dims, base, positions, x.dtype)
    cos, sin = cos[:, None, :], sin[:, None, :]
    out = x.clone()
    u, v = x[..., 0:n_dims:2], x[..., 1:n_dims:2]
    out[..., 0:n_dims:2] = u * cos - v * sin
    out[..., 1:n_dims:2] = v * cos + u * sin
    return out


def visible(T, window=None, chunk=None):
    """[T, T] bool: may query i read key j?"""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window:
        ok &= (i - j) < window
    if chunk:
        ok &= (i // chunk) == (j // chunk)
    return ok


def softmax_rows(scores, mask):
    return torch.softmax(scores.masked_fill(~mask, float("-inf")), dim=-1)


def talking_attention(w, p, m, x, eps):
    T = x.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (x @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (x @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (x @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    q = turn_halves(q, m["rot"]["dims"], m["rot"]["base"], pos)
    k = turn_halves(k, m["rot"]["dims"], m["rot"]["base"], pos)
    v = rms(v, eps)
    raw = torch.stack([q[:, h] @ k[:, h // (H // G)].T for h in range(H)]) * m["scale"]      # [H, T, T]
    mixed = torch.einsum("hg,gij->hij", w[p + "talk"], raw)
    mask = visible(T, chunk=m["mask"]["size"])
    gate = torch.sigmoid(x @ w[p + "g"].T)                                                   # [T, H]
    heads = []
    for h in range(H):
        a = softmax_rows(mixed[h], mask)
        heads.append((a @ v[:, h // (H // G)]) * gate[:, h:h + 1])
    return torch.cat(heads, dim=-1) @ w[p + "o"].T + w[p + "o.b"]


def latent_attention(w, p, m, x, eps):
    T = x.shape[0]
    H, d, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (x @ w[p + "q"].T).view(T, H, d + dr)
    down = x @ w[p + "dkv"].T
    c = rms(down[:, :R], eps) * w[p + "dkv.norm"]
    k_rot = turn_neighbours(down[:, None, R:], dr, m["rot"]["base"], pos)[:, 0]               # [T, dr], one for all heads
    q_rot = turn_neighbours(q[..., d:], dr, m["rot"]["base"], pos)
    k_up = (c @ w[p + "uk"].T).view(T, H, d)
    v_up = (c @ w[p + "uv"].T).view(T, H, dv)
    mask = visible(T, window=m["mask"]["size"])
    heads = []
    for h in range(H):
        s = (q[:, h, :d] @ k_up[:, h].T + q_rot[:, h] @ k_rot.T) * m["scale"]
        heads.append(softmax_rows(s, mask) @ v_up[:, h])
    return torch.cat(heads, dim=-1) @ w[p + "o"].T


def wkv(w, p, m, x, eps):
    T, D = x.shape
    H, d = m["heads"], m["dim"]
    before = torch.cat([torch.zeros(1, D, dtype=x.dtype), x[:-1]], dim=0)
    mixed = {s: x + (before - x) * w[p + "mu." + s] for s in "rkvgw"}
    r = (mixed["r"] @ w[p + "r"].T).view(T, H, d)
    k = (mixed["k"] @ w[p + "k"].T).view(T, H, d)
    v = (mixed["v"] @ w[p + "v"].T).view(T, H, d)
    gate = F.silu(mixed["g"] @ w[p + "g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mixed["w"] @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, d)
    u = w[p + "u"]
    out = torch.zeros(T, H, d, dtype=x.dtype)
    for h in range(H):
        S = torch.zeros(d, d, dtype=x.dtype)                    # [key channel, value channel]
        for t in range(T):
            kv = torch.outer(k[t, h], v[t, h])
            out[t, h] = (S + u[h][:, None] * kv).T @ r[t, h]
            S = decay[t, h][:, None] * S + kv
    return (rms(out, eps).reshape(T, H * d) * w[p + "norm"] * gate) @ w[p + "o"].T


def xielu(z, numbers):
    a, b = F.softplus(numbers[0]), F.softplus(numbers[1])
    return torch.where(z > 0, a * z * z + z / 2, (0.5 + b) * (torch.expm1(torch.clamp(z, max=0.0)) - z) + z / 2)


MIXERS = {"attention": talking_attention, "latent_attention": latent_attention, "wkv": wkv}


def forward(config, weights, tokens, dtype=torch.float64, layers_out=None):
    """Logits ``[T, vocab]`` of the whole sequence."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        x = x + MIXERS[layer["type"]](w, p + "mix.", layer["mixer"], rms(x, eps) * w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            h = rms(x, eps) * w[p + "norm2"]
            x = x + xielu(h @ w[p + "mlp.up"].T, w[p + "mlp.act"]) @ w[p + "mlp.down"].T
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * w["final.norm"]) @ w["embed"].T
