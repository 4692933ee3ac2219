"""Token mixers.  ``Attention``: multi-head (or grouped-query) causal
attention over a paged key/value cache.

One fused projection gives ``[q | k | v]`` per token (q = the first
``n_heads*head_dim`` columns, then k, then v, head j = columns
``[j*head_dim, (j+1)*head_dim)`` of each: mlx_lm/models/gpt2.py:52-58).  This
step's keys and values go into the request's pages first, then every token
attends keys ``max(0, p-window+1) .. p`` of its request through the block
table with scale ``head_dim**-0.5`` (mlx_lm/models/gpt2.py:39, 63-65), and
the output projection adds the residual in its epilogue.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import VECTOR, Init, Mixer, Normed, PagedKVSpec, ParamSpec, PositionEncoding, register_part
from .linear import FusedLinear, Linear


class Attention(Mixer):
    replayable = True
    kernel_libs = ("attention", "attention_prefill", "attention_prefill_tc")

    def __init__(self, name: str, width: int, n_heads: int, head_dim: int, n_kv_heads: Optional[int] = None,
                 window: Optional[int] = None, bias: bool = True, stored: str = "out_in",
                 qkv_name: str = "c_attn", out_name: str = "c_proj", scale: Optional[float] = None,
                 position: Optional[PositionEncoding] = None, init: Init = Init(), bias_init: Init = Init()):
        n_kv_heads = n_heads if n_kv_heads is None else n_kv_heads
        if n_heads % n_kv_heads:
            raise ValueError(f"{name}: {n_heads} query heads are not a multiple of {n_kv_heads} key/value heads")
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise ValueError(f"{name}: head size {head_dim} must be a multiple of 16 between 16 and 256")
        self.name, self.width = name, width
        self.n_heads, self.n_kv_heads, self.head_dim, self.window = n_heads, n_kv_heads, head_dim, window
        self.scale = head_dim ** -0.5 if scale is None else float(scale)
        self.position = position
        self.q_width, self.kv_width = n_heads * head_dim, n_kv_heads * head_dim
        self.qkv = Linear(f"{name}.{qkv_name}", width, self.q_width + 2 * self.kv_width, bias, stored,
                          init=init, bias_init=bias_init)
        self.out = Linear(f"{name}.{out_name}", self.q_width, width, bias, stored, init=init, bias_init=bias_init)

    def children(self):
        return (self.qkv, self.out)

    def cache_spec(self):
        return PagedKVSpec(self.n_kv_heads, self.head_dim, self.window)

    def fold_input_norm(self, norm) -> bool:
        return self.qkv.fold_norm(norm)

    def forward(self, ctx, x, residual, cache):
        T = x.shape[0]
        qkv = ctx.ws.get("qkv", T, self.q_width + 2 * self.kv_width, x.dtype)
        q = qkv[:, :self.q_width]
        src = x.source if isinstance(x, Normed) else x      # a Normed: the norm is folded into the projection
        if (cache.write and self.position is None and x.dtype == torch.bfloat16 and self.width % 8 == 0
                and src.stride(0) % 8 == 0 and src.data_ptr() % 16 == 0):
            # nothing to do to q and k before the cache: the projection's epilogue puts keys and values
            # into the pages itself
            fold = self.qkv.fold_of(ctx, x, few=T <= ops.SMALL_M) if isinstance(x, Normed) else None
            n_qkv = self.q_width + 2 * self.kv_width
            ops.label(self.qkv.name, 2.0 * T * self.width * n_qkv,
                      x.dtype.itemsize * (self.width * n_qkv + T * self.width + T * n_qkv))
            ops.linear_qkv_to_cache(src, self.qkv.weight, self.qkv.bias, qkv, ctx.positions, ctx.token_req,
                                    cache.block_table, cache.k, cache.v, self.q_width, ctx.status, ctx.stream,
                                    fold=fold)
        else:
            self.qkv.forward(ctx, x, qkv)
            k = qkv[:, self.q_width:self.q_width + self.kv_width]
            v = qkv[:, self.q_width + self.kv_width:]
            if self.position is not None:
                self.position.rotate(ctx, q, k)
            if cache.write:
                ops.kv_write(k, v, ctx.positions, ctx.token_req, cache.block_table, cache.k, cache.v, ctx.status,
                             ctx.stream)
        o = ctx.ws.get("attn_out", T, self.q_width, x.dtype)
        ops.label(self.name + ".attention")      # its cost depends on the requests' lengths: the caller knows them
        self.attend(ctx, q, cache, o)
        return self.out.forward(ctx, o, residual, residual=residual)

    def attend(self, ctx, q, cache, o) -> None:
        paged_attention(ctx, q, cache, o, self.n_heads, self.head_dim, self.scale, self.window)


def paged_attention(ctx, q, cache, o, n_heads: int, head_dim: int, scale: float, window: Optional[int],
                    sinks=None) -> None:
    """Causal attention of this step's queries over their requests' pages.  Rows of requests that bring one token
    go to a kernel for single queries (on tensor cores in bfloat16 for head sizes that are multiples of 16 up to
    128, else the split-key kernel on the CUDA cores), the rest to the kernel for portions; all write their rows
    of ``o``.  ``sinks``: float32 ``[n_heads]``, one more term of each head's softmax denominator, or None."""
    window = window or 0
    single_tiles = getattr(ctx, "single_tiles", None)
    if (ctx.n_single and single_tiles is not None
            and ops.attention_rows_supported(q.dtype, head_dim, ctx.n_single, n_heads, scale)):
        ops.attention_rows(q, single_tiles, ctx.n_single, cache.block_table, cache.k, cache.v, o, n_heads,
                           scale, window, ctx.status, ctx.stream, sinks=sinks)
    elif ctx.n_single:
        scratch = ctx.ws.flat("attn_partial", ops.attention_decode_scratch(
            ctx.n_single, n_heads, head_dim, ctx.max_len), torch.float32)
        counters = ctx.ws.flat("attn_tickets", ctx.n_single * n_heads, torch.int32)
        ops.attention_decode(q, ctx.positions, ctx.token_req, cache.block_table, cache.k, cache.v, o,
                             n_heads, scale, window, scratch, counters, ctx.max_len, ctx.status,
                             ctx.stream, rows=ctx.single_rows, sinks=sinks)
    if ctx.n_portion:
        if ops.attention_portions_supported(q.dtype, head_dim, scale) and ctx.portion_tiles is not None:
            ops.attention_portions(q, ctx.portion_tiles, ctx.n_portion_tiles, cache.block_table, cache.k,
                                   cache.v, o, n_heads, scale, window, ctx.status, ctx.stream, sinks=sinks,
                                   first_positions=ctx.req_first_position)
        else:
            ops.attention_generic(q, ctx.positions, ctx.token_req, cache.block_table, cache.k, cache.v, o,
                                  n_heads, scale, window, ctx.status, ctx.stream,
                                  rows=ctx.portion_rows, sinks=sinks)


register_part("mixer", "attention", Attention)


class SinkAttention(Mixer):
    """Grouped-query causal attention with the options of recent designs, each a parameter:

    * separate ``q``, ``k``, ``v`` tensors (run as one product), key/query size ``dim`` and value size ``vdim``
      that may differ (the pages hold heads ``head_dim`` wide, zero-filled beyond a head's own size);
    * ``qk_norm``: an RMS norm over a token's whole q projection, and whole k projection, before the heads are
      split, with plain weights ``<name>.q.norm`` / ``<name>.k.norm``;
    * ``rot_dims``: the first so many dimensions of every head turn with the position (dimension ``i`` paired
      with ``i + rot_dims/2``, angle ``p * rot_base**(-2i/rot_dims)``); 0 = no rotation;
    * ``scale`` of the scores as given; ``sink``: a learned number per head (``<name>.sink``) whose exponential
      is one more term of the softmax denominator, without a key or a value; ``window`` as in ``Attention``.

    ``mix`` returns the output projection in float32 (for a caller that combines it with something else);
    ``forward`` adds it to a float32 residual stream in that projection's epilogue."""
    replayable = True
    kernel_libs = ("attention", "attention_prefill", "attention_prefill_tc", "rotary")

    def __init__(self, name: str, width: int, n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float,
                 eps: float, rot_dims: int = 0, rot_base: float = 10000.0, qk_norm: bool = True, sink: bool = True,
                 window: Optional[int] = None, init: Init = Init()):
        if n_heads % n_kv_heads:
            raise ValueError(f"{name}: {n_heads} query heads are not a multiple of {n_kv_heads} key/value heads")
        if rot_dims % 2 or rot_dims > dim:
            raise ValueError(f"{name}: {rot_dims} rotated dimensions of {dim}")
        self.name, self.width = name, width
        self.n_heads, self.n_kv_heads, self.dim, self.vdim = n_heads, n_kv_heads, dim, vdim
        self.head_dim = (max(dim, vdim) + 15) // 16 * 16
        if self.head_dim > 256:
            raise ValueError(f"{name}: head size {max(dim, vdim)} is beyond 256")
        self.scale, self.eps, self.window = float(scale), float(eps), window
        self.rot_dims, self.rot_base, self.qk_norm, self.has_sink = rot_dims, float(rot_base), qk_norm, sink
        self.qkv = FusedLinear(f"{name}.qkv", width, [(f"{name}.q", n_heads * dim), (f"{name}.k", n_kv_heads * dim),
                                                      (f"{name}.v", n_kv_heads * vdim)], init=init)
        self.out = Linear(f"{name}.o", n_heads * vdim, width, bias=False, weight_suffix="", init=init)
        self.q_norm = self.k_norm = self.sinks = self.freq = None

    def children(self):
        return (self.qkv, self.out)

    def cache_spec(self):
        return PagedKVSpec(self.n_kv_heads, self.head_dim, self.window)

    def param_specs(self) -> List[ParamSpec]:
        specs = []
        if self.qk_norm:
            specs += [ParamSpec(f"{self.name}.q.norm", (self.n_heads * self.dim,), VECTOR, Init(1.0, 0.1)),
                      ParamSpec(f"{self.name}.k.norm", (self.n_kv_heads * self.dim,), VECTOR, Init(1.0, 0.1))]
        if self.has_sink:
            specs.append(ParamSpec(f"{self.name}.sink", (self.n_heads,), VECTOR, Init(0.0, 1.0)))
        return specs

    def bind(self, tensors, dtype, device) -> None:
        if self.qk_norm:
            self.q_norm, self.k_norm = tensors[f"{self.name}.q.norm"], tensors[f"{self.name}.k.norm"]
        if self.has_sink:
            self.sinks = tensors[f"{self.name}.sink"]
        if self.rot_dims:
            i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
            self.freq = (self.rot_base ** (-2.0 * i / self.rot_dims)).to(torch.float32).to(device)

    def bind_all(self, tensors, dtype, device) -> None:
        super().bind_all(tensors, dtype, device)
        if self.head_dim != self.vdim:
            # the attention kernels leave heads head_dim wide: give the output projection zero columns there
            w = self.out.weight.view(self.width, self.n_heads, self.vdim)
            wide = torch.zeros(self.width, self.n_heads, self.head_dim, dtype=w.dtype, device=w.device)
            wide[:, :, :self.vdim] = w
            self.out.use_weight(wide.view(self.width, self.n_heads * self.head_dim).contiguous())
            self.out.n_in = self.n_heads * self.head_dim

    def _heads_out(self, ctx, x, cache):
        T, H, G = x.shape[0], self.n_heads, self.n_kv_heads
        n = self.qkv.n_out
        proj = ctx.ws.get("attn_proj", T, (n + 7) // 8 * 8, x.dtype)[:, :n]
        self.qkv.forward(ctx, x, proj)
        q = ctx.ws.get("attn_q", T, H * self.head_dim, x.dtype)
        ops.label(self.name + ".prepare", 8.0 * T * n, 2.0 * x.element_size() * T * n)
        ops.qkv_prepare(proj, 0, H * self.dim, (H + G) * self.dim, H, G, self.dim, self.vdim, self.q_norm, self.k_norm,
                        self.eps, self.freq, ctx.positions, ctx.token_req, cache.block_table, cache.k, cache.v, q,
                        cache.write, ctx.status, ctx.stream)
        o = ctx.ws.get("attn_out", T, H * self.head_dim, x.dtype)
        ops.label(self.name + ".attention")
        paged_attention(ctx, q, cache, o, H, self.head_dim, self.scale, self.window, sinks=self.sinks)
        return o

    def mix(self, ctx, x, cache, tag: str = "mix_left"):
        o = self._heads_out(ctx, x, cache)
        return self.out.forward(ctx, o, ctx.ws.get(tag, x.shape[0], self.width, torch.float32))

    def forward(self, ctx, x, residual, cache):
        return self.out.forward(ctx, self._heads_out(ctx, x, cache), residual, residual=residual)


class ParallelMixer(Mixer):
    """Two mixers side by side on the same input: ``scale * (norm_l(left(x)) + norm_r(right(x)))`` added to the
    residual stream, each output RMS-normed over the model width with a plain weight (``<name>.left.out`` /
    ``<name>.right.out``) first.  Each side keeps its own cache (``cache_spec`` is a dictionary); the sides are
    any mixers that have ``mix(ctx, x, cache, tag) -> float32 [T, width]``."""
    replayable = True
    kernel_libs = ("rms",)

    def __init__(self, name: str, width: int, left: Mixer, right: Mixer, eps: float, scale: float = 0.5):
        self.name, self.width, self.left, self.right, self.eps, self.scale = name, width, left, right, float(eps), scale
        self.w_left = self.w_right = None

    def children(self):
        return (self.left, self.right)

    def cache_spec(self):
        out = {}
        for side, m in (("left", self.left), ("right", self.right)):
            spec = m.cache_spec()
            if isinstance(spec, dict):
                out.update({f"{side}.{k}": v for k, v in spec.items()})
            elif spec is not None:
                out[side] = spec
        return out

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec(f"{self.name}.left.out", (self.width,), VECTOR, Init(1.0, 0.1)),
                ParamSpec(f"{self.name}.right.out", (self.width,), VECTOR, Init(1.0, 0.1))]

    def bind(self, tensors, dtype, device) -> None:
        self.w_left, self.w_right = tensors[f"{self.name}.left.out"], tensors[f"{self.name}.right.out"]

    def forward(self, ctx, x, residual, cache):
        yl = self.left.mix(ctx, x, cache.side("left"), tag="mix_left")
        yr = self.right.mix(ctx, x, cache.side("right"), tag="mix_right")
        ops.label(self.name + ".combine", 8.0 * x.shape[0] * self.width, 16.0 * x.shape[0] * self.width)
        ops.residual_update(residual, yl, ctx.stream, w1=self.w_left, y2=yr, w2=self.w_right, scale=self.scale,
                            eps=self.eps)
        return residual


register_part("mixer", "sink_attention", SinkAttention)
register_part("mixer", "parallel", ParallelMixer)
