"""Feed-forward parts.  ``MLP``: ``down(act(up(x)))`` with biases, the dense
two-matrix form of mlx_lm/models/gpt2.py:71-80 with the inner width and the
activation as parameters; the activation runs in the first product's
epilogue and the residual add in the second's."""

from __future__ import annotations

from .base import VECTOR, FeedForward, Init, ParamSpec, register_part
import torch

from .. import ops
from .linear import ACTIVATIONS, FusedLinear, Linear


class MLP(FeedForward):
    replayable = True
    def __init__(self, name: str, width: int, inner: int, activation: str = "gelu_new", bias: bool = True,
                 stored: str = "out_in", up_name: str = "c_fc", down_name: str = "c_proj", init: Init = Init(),
                 bias_init: Init = Init()):
        if activation not in ACTIVATIONS:
            raise ValueError(f"{name}: activation {activation!r} is not one of {sorted(a for a in ACTIVATIONS if a)}")
        self.name, self.width, self.inner, self.activation = name, width, inner, activation
        self.up = Linear(f"{name}.{up_name}", width, inner, bias, stored, init=init, bias_init=bias_init)
        self.down = Linear(f"{name}.{down_name}", inner, width, bias, stored, init=init, bias_init=bias_init)

    def children(self):
        return (self.up, self.down)

    def fold_input_norm(self, norm) -> bool:
        return self.up.fold_norm(norm)

    def forward(self, ctx, x, residual):
        h = self.up.forward(ctx, x, ctx.ws.get("ffn_hidden", x.shape[0], self.inner, x.dtype),
                            activation=self.activation)
        return self.down.forward(ctx, h, residual, residual=residual)


register_part("feed_forward", "mlp", MLP)


class GatedMLP(FeedForward):
    """``down(silu(gate(x)) * up(x))`` without biases.  ``gate`` and ``up`` run as one product whose two halves
    a small kernel multiplies; the residual stream (float32) is added in the last product's epilogue."""
    replayable = True
    kernel_libs = ("elementwise",)

    def __init__(self, name: str, width: int, inner: int, gate_name: str = "gate", up_name: str = "up",
                 down_name: str = "down", init: Init = Init()):
        self.name, self.width, self.inner = name, width, inner
        self.gate_up = FusedLinear(f"{name}.gate_up", width, [(f"{name}.{gate_name}", inner), (f"{name}.{up_name}", inner)],
                                   init=init)
        self.down = Linear(f"{name}.{down_name}", inner, width, bias=False, weight_suffix="", init=init)

    def children(self):
        return (self.gate_up, self.down)

    def forward(self, ctx, x, residual):
        T = x.shape[0]
        both = ctx.ws.get("ffn_gate_up", T, 2 * self.inner, x.dtype)
        self.gate_up.forward(ctx, x, both)
        h = ctx.ws.get("ffn_hidden", T, self.inner, x.dtype)
        ops.label(self.name + ".act", 4.0 * T * self.inner, 3.0 * x.element_size() * T * self.inner)
        ops.gated_unit(both, h, ctx.stream)
        return self.down.forward(ctx, h, residual, residual=residual)


register_part("feed_forward", "gated_mlp", GatedMLP)


class LearnedActMLP(FeedForward):
    """``down(act(up(x)))`` without biases, where ``act`` has numbers of its own that the layer learns (a tensor
    ``<name>.act``).  ``xielu``: two numbers ``(a, b)``; ``z > 0: softplus(a) z^2 + z/2``,
    ``z <= 0: (1/2 + softplus(b)) (exp(z) - 1 - z) + z/2``.  The activation is a kernel of its own between the two
    products (float32 arithmetic, in place); the residual stream (float32) is added in the second product's epilogue."""
    replayable = True
    kernel_libs = ("elementwise",)
    ACTS = {"xielu": 2}      # name -> how many numbers

    def __init__(self, name: str, width: int, inner: int, activation: str = "xielu", up_name: str = "up",
                 down_name: str = "down", act_name: str = "act", init: Init = Init()):
        if activation not in self.ACTS:
            raise ValueError(f"{name}: activation {activation!r} is not one of {sorted(self.ACTS)}")
        self.name, self.width, self.inner, self.activation = name, width, inner, activation
        self.act_name = f"{name}.{act_name}"
        self.up = Linear(f"{name}.{up_name}", width, inner, bias=False, weight_suffix="", init=init)
        self.down = Linear(f"{name}.{down_name}", inner, width, bias=False, weight_suffix="", init=Init(0.0, inner ** -0.5))
        self.act = None

    def children(self):
        return (self.up, self.down)

    def param_specs(self):
        return [ParamSpec(self.act_name, (self.ACTS[self.activation],), VECTOR, Init(0.0, 0.5))]

    def bind(self, tensors, dtype, device) -> None:
        self.act = tensors[self.act_name].contiguous()

    def forward(self, ctx, x, residual):
        T = x.shape[0]
        h = self.up.forward(ctx, x, ctx.ws.get("ffn_hidden", T, self.inner, x.dtype))
        ops.label(self.name + ".act", 8.0 * T * self.inner, 2.0 * x.element_size() * T * self.inner)
        ops.xielu(h, h, self.act, ctx.stream)
        return self.down.forward(ctx, h, residual, residual=residual)


register_part("feed_forward", "learned_act_mlp", LearnedActMLP)
