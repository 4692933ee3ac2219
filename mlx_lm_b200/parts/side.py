"""A per-layer input that depends on the token itself: a second, narrow embedding table whose row for the
token (the layer's own ``dim`` columns of it) is gated by the stream and added back to it,

    e = table[token][first : first + dim];  g = gelu_tanh(gate x) * e;  y = proj g;
    x <- x + y / sqrt(mean(y^2) + eps) * norm

A branch of a ``StreamBlock`` (``forward(ctx, x) -> x``).  The table belongs to the model, not to a layer:
every layer's part names the same tensor, and the model declares it once (``SideTable``).
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import MATRIX, VECTOR, Init, ParamSpec, Part
from .linear import Linear


class SideTable(Part):
    """The table ``[vocab, layers * dim]`` all ``TokenSideInput`` parts of a model read."""
    replayable = True

    def __init__(self, name: str, vocab_size: int, n_columns: int, init: Init = Init(0.0, 1.0)):
        self.name, self.vocab_size, self.n_columns, self.init = name, vocab_size, n_columns, init
        self.table: Optional[torch.Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec(self.name, (self.vocab_size, self.n_columns), MATRIX, self.init)]

    def bind(self, tensors, dtype, device) -> None:
        self.table = tensors[self.name]


class TokenSideInput(Part):
    replayable = True
    kernel_libs = ("elementwise", "rms")

    def __init__(self, name: str, width: int, dim: int, table: SideTable, first: int, eps: float, init: Init = Init()):
        self.name, self.width, self.dim, self.table, self.first, self.eps = name, width, dim, table, first, float(eps)
        self.gate = Linear(f"{name}.gate", width, dim, bias=False, weight_suffix="", init=init)
        self.proj = Linear(f"{name}.proj", dim, width, bias=False, weight_suffix="", init=init)
        self.norm_w: Optional[torch.Tensor] = None

    def children(self):
        return (self.gate, self.proj)

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec(f"{self.name}.norm", (self.width,), VECTOR, Init(1.0, 0.1))]

    def bind(self, tensors, dtype, device) -> None:
        self.norm_w = tensors[f"{self.name}.norm"]

    def forward(self, ctx, x):
        T = x.shape[0]
        if ctx.dtype == torch.float32:
            xa = x
        else:
            xa = ctx.ws.get("side_in", T, self.width, ctx.dtype)
            ops.label(self.name + ".cast", 0.0, (4.0 + xa.element_size()) * T * self.width)
            ops.join_rows(x, None, xa, ctx.stream)
        pad = (self.dim + 7) // 8 * 8      # rows of the narrow tensors start on 16-byte boundaries
        g = ctx.ws.get("side_gate", T, pad, ctx.dtype)[:, :self.dim]
        self.gate.forward(ctx, xa, g, activation="gelu_new")
        ge = ctx.ws.get("side_gated", T, pad, ctx.dtype)[:, :self.dim]
        ops.label(self.name + ".lookup", 1.0 * T * self.dim, 3.0 * g.element_size() * T * self.dim)
        ops.scale_by_rows(g, ctx.tokens, self.table.table, self.first, ge, ctx.status, ctx.stream)
        y = ctx.ws.get("side_y", T, self.width, torch.float32)
        self.proj.forward(ctx, ge, y)
        ops.label(self.name + ".add", 6.0 * T * self.width, 12.0 * T * self.width)
        ops.residual_update(x, y, ctx.stream, w1=self.norm_w, eps=self.eps)
        return x
