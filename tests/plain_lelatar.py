"""A plain, slow implementation of the Lelatar design: whole sequences on the CPU in one
float type, token by token where the design is recurrent, one function per mechanism.

It shares no code with the engine: it takes a config dictionary (the keys of config.json)
and a dictionary ``name -> tensor`` and uses torch only for array arithmetic.  The tests
compare the engine with it.

Notation: ``T`` tokens, width ``D``.  Linear weights are ``[out, in]`` and act as ``W x``.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def norm_around_zero(x, w, eps):
    """The model's norm: the weight is stored as its distance from one."""
    return unit_rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return unit_rms(x, eps) * w


def short_conv(u: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor]) -> torch.Tensor:
    """``u [T, C]``, ``w [C, taps]``: out[t, c] = sum_j w[c, taps-1-j] * u[t-j, c], zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    out = torch.zeros_like(u)
    for j in range(taps):
        if j < T:
            out[j:] += u[:T - j] * w[:, taps - 1 - j]
    if b is not None:
        out = out + b
    return out


def mamba2_mixer(h: torch.Tensor, P: Dict[str, torch.Tensor], pre: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * V
    proj = h @ P[pre + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, P[pre + "conv"], P[pre + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, V)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + P[pre + "dt_bias"])                     # [T, H]
    a = torch.exp(-torch.exp(P[pre + "A_log"]) * dt)           # [T, H]
    per = H // G
    grp = torch.arange(H) // per
    S = torch.zeros(H, N, V, dtype=h.dtype)
    y = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        Bt, Ct = B[t, grp], C[t, grp]                          # [H, N]
        S = a[t, :, None, None] * S + dt[t, :, None, None] * Bt[:, :, None] * x[t, :, None, :]
        y[t] = torch.einsum("hnv,hn->hv", S, Ct) + P[pre + "D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * P[pre + "norm"]
    return y @ P[pre + "o"].T


def rotate_heads(x: torch.Tensor, first: int, rot: dict) -> torch.Tensor:
    """``x [T, heads, dim]``; the first ``rot['dims']`` dimensions of every head turn by position."""
    T = x.shape[0]
    n = rot["dims"]
    half = n // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = float(rot["base"]) ** (-2.0 * i / n)
    ang = (torch.arange(first, first + T, dtype=torch.float64)[:, None] * freq[None, :])
    cos, sin = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:n]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., n:]], dim=-1)


def sink_attention(h, P, pre, m, eps):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = norm_plain(h @ P[pre + "q"].T, P[pre + "q.norm"], eps).reshape(T, H, dk)
    k = norm_plain(h @ P[pre + "k"].T, P[pre + "k.norm"], eps).reshape(T, G, dk)
    v = (h @ P[pre + "v"].T).reshape(T, G, dv)
    q, k = rotate_heads(q, 0, m["rot"]), rotate_heads(k, 0, m["rot"])
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~causal, -math.inf)
        sink = P[pre + "sink"][hd]
        top = torch.maximum(s.max(dim=-1, keepdim=True).values, sink)
        e = torch.exp(s - top)
        out[:, hd] = (e @ v[:, g]) / (e.sum(dim=-1, keepdim=True) + torch.exp(sink - top))
    return out.reshape(T, H * dv) @ P[pre + "o"].T


def gated_delta(h, P, pre, m, eps):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ P[pre + "q"].T, P[pre + "q.conv"], None)).reshape(T, G, dk)
    k = silu(short_conv(h @ P[pre + "k"].T, P[pre + "k.conv"], None)).reshape(T, G, dk)
    v = silu(short_conv(h @ P[pre + "v"].T, P[pre + "v.conv"], None)).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ P[pre + "b"].T)                                   # [T, H]
    decay = torch.exp(-torch.exp(P[pre + "A_log"]) * softplus(h @ P[pre + "a"].T + P[pre + "dt_bias"]))
    grp = torch.arange(H) // (H // G)
    S = torch.zeros(H, dk, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        kt, qt = k[t, grp], q[t, grp]                                          # [H, dk]
        S = decay[t, :, None, None] * S
        u = beta[t, :, None] * (v[t] - torch.einsum("hkv,hk->hv", S, kt))
        S = S + kt[:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, qt)
    o = unit_rms(o, eps) * P[pre + "norm"]
    o = o.reshape(T, H * dv) * silu(h @ P[pre + "g"].T)
    return o @ P[pre + "o"].T


def parallel_mixer(h, P, pre, m, eps):
    left = sink_attention(h, P, pre + "left.", m["left"], eps)
    right = gated_delta(h, P, pre + "right.", m["right"], eps)
    return 0.5 * (norm_plain(left, P[pre + "left.out"], eps) + norm_plain(right, P[pre + "right.out"], eps))


def dense_ff(h, P, pre):
    return (silu(h @ P[pre + "gate"].T) * (h @ P[pre + "up"].T)) @ P[pre + "down"].T


def token_side(x, tokens, P, i: int, dim: int, eps: float):
    e = P["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    g = gelu_tanh(x @ P[f"l{i}.side.gate"].T) * e
    y = g @ P[f"l{i}.side.proj"].T
    return x + norm_plain(y, P[f"l{i}.side.norm"], eps)


def layer(x, tokens, P, i: int, spec: dict, config: dict):
    eps = config["norm"]["eps"]
    h = norm_around_zero(x, P[f"l{i}.norm1"], eps)
    if spec["type"] == "mamba2":
        x = x + mamba2_mixer(h, P, f"l{i}.mix.", spec["mixer"], eps)
    elif spec["type"] == "parallel":
        x = x + parallel_mixer(h, P, f"l{i}.mix.", spec["mixer"], eps)
    else:
        raise ValueError(spec["type"])
    if spec.get("mlp") is not None:
        x = x + dense_ff(norm_around_zero(x, P[f"l{i}.norm2"], eps), P, f"l{i}.mlp.")
    side = config.get("token_side")
    if side:
        x = token_side(x, tokens, P, i, side["dim"], eps)
    return x


def run_order(config: dict) -> List[Tuple[int, Optional[int], bool]]:
    """``(layer, pass number or None, first of its pass)`` in the order the layers run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None, False) for i in range(a)]
    for t in range(times):
        order += [(i, t, i == a) for i in range(a, b)]
    order += [(i, None, False) for i in range(b, n)]
    return order


def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens, dtype=torch.float64, layers_out=None):
    """Logits ``[T, vocab]`` of a whole sequence; ``layers_out`` (a list) receives the stream after every layer run."""
    P = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x0 = P["embed"][tokens]
    x = x0
    for i, t, first in run_order(config):
        if first:
            x = torch.cat([x, x0], dim=-1) @ P["loop.in"].T + P["loop.step"][t]
        x = layer(x, tokens, P, i, config["layers"][i], config)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = norm_around_zero(x, P["final.norm"], config["norm"]["eps"])
    return x @ P["head"].T
