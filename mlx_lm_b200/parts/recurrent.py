"""Mixers that keep a state of fixed size per request instead of keys and values: the selective
state-space layer of Mamba-2 and the gated delta rule.  Both read their inputs through short causal
convolutions whose last ``taps - 1`` inputs are part of the state.  State is float32 and lives in the
cache manager's slots; a step reads it at the start of each request's run of tokens and writes it back
at the end, so prompts may be cut into portions anywhere and decoding continues from it.

``mix`` returns the output projection in float32 (for a caller that combines it with something
else); ``forward`` adds it to a float32 residual stream in that projection's epilogue.
"""

from __future__ import annotations

from typing import List

import torch

from .. import ops
from .base import VECTOR, Init, Mixer, ParamSpec, StateSpec, register_part
from .linear import FusedLinear, Linear


class Mamba2Mixer(Mixer):
    """``in`` projects to ``[z | x | B | C | dt]`` (``inner = heads * vdim``, ``B`` and ``C`` of ``groups * state``);
    x, B, C pass one convolution (with bias) and silu; per head ``S <- exp(-exp(A_log) dt) S + dt B x^T``,
    ``y = S^T C + D x`` with ``dt = softplus(dt + dt_bias)``; ``y * silu(z)`` is RMS-normed in ``norm_groups``
    equal parts, times ``norm``, then ``o``."""
    replayable = True
    kernel_libs = ("recurrent", "rms")

    def __init__(self, name: str, width: int, n_heads: int, vdim: int, state: int, groups: int, norm_groups: int,
                 taps: int, eps: float, init: Init = Init()):
        if n_heads % groups or (n_heads * vdim) % norm_groups:
            raise ValueError(f"{name}: {n_heads} heads in {groups} groups, inner width in {norm_groups} parts")
        self.name, self.width = name, width
        self.n_heads, self.vdim, self.state, self.groups, self.norm_groups = n_heads, vdim, state, groups, norm_groups
        self.taps, self.eps = taps, float(eps)
        self.inner = n_heads * vdim
        self.conv_width = self.inner + 2 * groups * state
        self.n_proj = 2 * self.inner + 2 * groups * state + n_heads
        self.proj = Linear(f"{name}.in", width, self.n_proj, bias=False, weight_suffix="", init=init)
        self.out = Linear(f"{name}.o", self.inner, width, bias=False, weight_suffix="", init=init)

    def children(self):
        return (self.proj, self.out)

    def cache_spec(self):
        return {"conv": StateSpec((self.taps - 1, self.conv_width)),
                "ssm": StateSpec((self.n_heads, self.vdim, self.state))}     # column by column: the scan's layout

    def param_specs(self) -> List[ParamSpec]:
        n, H = self.name, self.n_heads
        return [ParamSpec(f"{n}.conv", (self.conv_width, self.taps), VECTOR, Init(0.0, 0.3)),
                ParamSpec(f"{n}.conv.b", (self.conv_width,), VECTOR, Init(0.0, 0.1)),
                ParamSpec(f"{n}.dt_bias", (H,), VECTOR, Init(0.0, 0.5)),
                ParamSpec(f"{n}.A_log", (H,), VECTOR, Init(0.0, 0.5)),
                ParamSpec(f"{n}.D", (H,), VECTOR, Init(1.0, 0.2)),
                ParamSpec(f"{n}.norm", (self.inner,), VECTOR, Init(1.0, 0.1))]

    def bind(self, tensors, dtype, device) -> None:
        n = self.name
        self.conv_w, self.conv_b = tensors[f"{n}.conv"], tensors[f"{n}.conv.b"]
        self.conv_wt = self.conv_w.t().contiguous()      # tap by tap, for the kernel that takes eight channels a thread
        self.dt_bias, self.a_log, self.d_skip = tensors[f"{n}.dt_bias"], tensors[f"{n}.A_log"], tensors[f"{n}.D"]
        self.norm_w = tensors[f"{n}.norm"]

    def _gated(self, ctx, x, cache):
        T, inner, GN = x.shape[0], self.inner, self.groups * self.state
        proj = ctx.ws.get("ssm_proj", T, (self.n_proj + 7) // 8 * 8, x.dtype)[:, :self.n_proj]
        self.proj.forward(ctx, x, proj)
        conv_state, ssm_state = cache.side("conv"), cache.side("ssm")
        xbc = ctx.ws.get("ssm_conv", T, self.conv_width, x.dtype)
        ops.label(self.name + ".conv", 2.0 * self.taps * T * self.conv_width, 2.0 * x.element_size() * T * self.conv_width)
        ops.conv_silu(proj[:, inner:inner + self.conv_width], self.conv_w, self.conv_b, conv_state.state,
                      conv_state.slots, ctx.positions, ctx.token_req, ctx.req_first_token, ctx.req_first_position, xbc,
                      ctx.stream, weight_by_tap=self.conv_wt)
        y = ctx.ws.get("ssm_y", T, inner, torch.float32)
        # what it has to move: its inputs and outputs, and every live request's state in and out
        ops.label(self.name + ".scan", 6.0 * T * inner * self.state, x.element_size() * T * self.conv_width + 4.0 * T * inner
                  + 8.0 * min(T, ctx.n_requests) * inner * self.state)
        ops.mamba2_scan(xbc, 0, inner, inner + GN, proj[:, inner + self.conv_width:], self.dt_bias, self.a_log,
                        self.d_skip, ssm_state.state, ssm_state.slots, ctx.token_req, ctx.req_first_token, y,
                        self.n_heads, self.groups, ctx.stream)
        g = ctx.ws.get("ssm_gated", T, inner, x.dtype)
        ops.label(self.name + ".norm", 8.0 * T * inner, (4.0 + 2 * x.element_size()) * T * inner)
        ops.rmsnorm(y, self.norm_w, g, self.eps, ctx.stream, groups=self.norm_groups, gate=proj[:, :inner],
                    gate_mode=ops.GATE_BEFORE)
        return g

    def mix(self, ctx, x, cache, tag: str = "mix_ssm"):
        g = self._gated(ctx, x, cache)
        return self.out.forward(ctx, g, ctx.ws.get(tag, x.shape[0], self.width, torch.float32))

    def forward(self, ctx, x, residual, cache):
        return self.out.forward(ctx, self._gated(ctx, x, cache), residual, residual=residual)


class GatedDeltaMixer(Mixer):
    """Linear attention with the gated delta rule.  ``q``, ``k`` (``kv_heads x dim``) and ``v`` (``heads x vdim``)
    each pass a convolution without bias and silu; q and k become unit vectors per head (q also divided by
    ``sqrt(dim)``); per head ``S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q`` with
    ``beta = sigmoid(b x)`` and ``g = exp(-exp(A_log) softplus(a x + dt_bias))``; every head's ``o`` is divided by
    its root mean square, times ``norm`` (shared by the heads), times ``silu(g x)``; then ``o``."""
    replayable = True
    kernel_libs = ("recurrent", "rms")

    def __init__(self, name: str, width: int, n_heads: int, n_kv_heads: int, dim: int, vdim: int, taps: int,
                 eps: float, init: Init = Init()):
        if n_heads % n_kv_heads:
            raise ValueError(f"{name}: {n_heads} heads over {n_kv_heads} query/key heads")
        self.name, self.width = name, width
        self.n_heads, self.n_kv_heads, self.dim, self.vdim, self.taps, self.eps = n_heads, n_kv_heads, dim, vdim, taps, float(eps)
        self.qk_width, self.v_width = n_kv_heads * dim, n_heads * vdim
        self.conv_width = 2 * self.qk_width + self.v_width
        self.proj = FusedLinear(f"{name}.in", width, [(f"{name}.q", self.qk_width), (f"{name}.k", self.qk_width),
                                                      (f"{name}.v", self.v_width), (f"{name}.g", self.v_width),
                                                      (f"{name}.b", n_heads), (f"{name}.a", n_heads)], init=init)
        self.out = Linear(f"{name}.o", self.v_width, width, bias=False, weight_suffix="", init=init)

    def children(self):
        return (self.proj, self.out)

    def cache_spec(self):
        return {"conv": StateSpec((self.taps - 1, self.conv_width)),
                "rule": StateSpec((self.n_heads, self.vdim, self.dim))}      # column by column: the scan's layout

    def param_specs(self) -> List[ParamSpec]:
        n, H = self.name, self.n_heads
        return [ParamSpec(f"{n}.q.conv", (self.qk_width, self.taps), VECTOR, Init(0.0, 0.3)),
                ParamSpec(f"{n}.k.conv", (self.qk_width, self.taps), VECTOR, Init(0.0, 0.3)),
                ParamSpec(f"{n}.v.conv", (self.v_width, self.taps), VECTOR, Init(0.0, 0.3)),
                ParamSpec(f"{n}.A_log", (H,), VECTOR, Init(0.0, 0.5)),
                ParamSpec(f"{n}.dt_bias", (H,), VECTOR, Init(0.0, 0.5)),
                ParamSpec(f"{n}.norm", (self.vdim,), VECTOR, Init(1.0, 0.1))]

    def bind(self, tensors, dtype, device) -> None:
        n = self.name
        self.conv_w = torch.cat([tensors[f"{n}.q.conv"], tensors[f"{n}.k.conv"], tensors[f"{n}.v.conv"]], dim=0).contiguous()
        self.conv_wt = self.conv_w.t().contiguous()
        self.a_log, self.dt_bias, self.norm_w = tensors[f"{n}.A_log"], tensors[f"{n}.dt_bias"], tensors[f"{n}.norm"]

    def _gated(self, ctx, x, cache):
        T, H = x.shape[0], self.n_heads
        n = self.proj.n_out
        proj = ctx.ws.get("delta_proj", T, (n + 7) // 8 * 8, x.dtype)[:, :n]
        self.proj.forward(ctx, x, proj)
        conv_state, rule_state = cache.side("conv"), cache.side("rule")
        qkv = ctx.ws.get("delta_conv", T, self.conv_width, x.dtype)
        ops.label(self.name + ".conv", 2.0 * self.taps * T * self.conv_width, 2.0 * x.element_size() * T * self.conv_width)
        ops.conv_silu(proj[:, :self.conv_width], self.conv_w, None, conv_state.state, conv_state.slots, ctx.positions,
                      ctx.token_req, ctx.req_first_token, ctx.req_first_position, qkv, ctx.stream,
                      weight_by_tap=self.conv_wt)
        g_off = self.conv_width
        b_off = g_off + self.v_width
        o = ctx.ws.get("delta_o", T, self.v_width, torch.float32)
        ops.label(self.name + ".scan", 8.0 * T * self.v_width * self.dim, x.element_size() * T * self.conv_width + 4.0 * T * self.v_width
                  + 8.0 * min(T, ctx.n_requests) * self.v_width * self.dim)
        ops.gated_delta_scan(qkv, 0, self.qk_width, 2 * self.qk_width, proj[:, b_off:b_off + H],
                             proj[:, b_off + H:b_off + 2 * H], self.dt_bias, self.a_log, rule_state.state,
                             rule_state.slots, ctx.token_req, ctx.req_first_token, o, H, self.n_kv_heads, ctx.stream)
        g = ctx.ws.get("delta_gated", T, self.v_width, x.dtype)
        ops.label(self.name + ".norm", 8.0 * T * self.v_width, (4.0 + 2 * x.element_size()) * T * self.v_width)
        ops.rmsnorm(o, self.norm_w, g, self.eps, ctx.stream, groups=H, period=self.vdim,
                    gate=proj[:, g_off:g_off + self.v_width], gate_mode=ops.GATE_AFTER)
        return g

    def mix(self, ctx, x, cache, tag: str = "mix_right"):
        g = self._gated(ctx, x, cache)
        return self.out.forward(ctx, g, ctx.ws.get(tag, x.shape[0], self.width, torch.float32))

    def forward(self, ctx, x, residual, cache):
        return self.out.forward(ctx, self._gated(ctx, x, cache), residual, residual=residual)


class WKVMixer(Mixer):
    """Time mixing in the manner of RWKV with a decay computed from the data.

    With ``x'`` the row of the token before (zeros before the first token; the last row of a step is part of the
    state), each of r, k, v, g, w reads its own mix ``x + (x' - x) mu_s`` (``<name>.mu.r`` ...).  ``r``, ``k``, ``v`` are
    products of their mixes (``heads x dim`` each), the gate is ``silu(W_g mix_g)``, the decay per head and key channel
    ``w = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0))``.  Per head, with a ``dim x dim`` state ``S``:
    ``o_t = (S + diag(u) k_t v_t^T)^T r_t`` (the bonus ``u`` for the current token only), then
    ``S <- diag(w_t) S + k_t v_t^T``.  Every head's ``o`` is divided by its root mean square, times ``<name>.norm``
    (one weight per column), times the gate; then ``<name>.o``.  Decay, exponentials, state and the norm are float32."""
    replayable = True
    kernel_libs = ("wkv", "rms")
    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, name: str, width: int, n_heads: int, dim: int, decay_rank: int, eps: float, init: Init = Init()):
        self.name, self.width, self.n_heads, self.dim, self.decay_rank, self.eps = name, width, n_heads, dim, decay_rank, float(eps)
        self.inner = n_heads * dim
        self.inner_p = (self.inner + 7) // 8 * 8      # sections of the shared buffers start on 16 bytes
        self.width_p = (width + 7) // 8 * 8
        lin = lambda s, n_in, n_out, i=init: Linear(f"{name}.{s}", n_in, n_out, bias=False, weight_suffix="", init=i)
        self.r, self.k, self.v, self.g = (lin(s, width, self.inner) for s in "rkvg")
        self.w1 = lin("w1", width, decay_rank)
        self.w2 = lin("w2", decay_rank, self.inner, Init(0.0, decay_rank ** -0.5))
        self.out = lin("o", self.inner, width, Init(0.0, self.inner ** -0.5))
        self.mu = self.bonus = self.norm_w = None

    def children(self):
        return (self.r, self.k, self.v, self.g, self.w1, self.w2, self.out)

    def cache_spec(self):
        return {"shift": StateSpec((self.width,)),
                "wkv": StateSpec((self.n_heads, self.dim, self.dim))}      # column by column: the scan's layout

    def param_specs(self) -> List[ParamSpec]:
        n = self.name
        return ([ParamSpec(f"{n}.mu.{s}", (self.width,), VECTOR, Init(0.5, 0.2)) for s in self.MIXES]
                + [ParamSpec(f"{n}.w0", (self.inner,), VECTOR, Init(-1.0, 1.0)),
                   ParamSpec(f"{n}.u", (self.n_heads, self.dim), VECTOR, Init(0.0, 0.5)),
                   ParamSpec(f"{n}.norm", (self.inner,), VECTOR, Init(1.0, 0.1))])

    def bind(self, tensors, dtype, device) -> None:
        n = self.name
        self.mu = torch.stack([tensors[f"{n}.mu.{s}"] for s in self.MIXES]).contiguous()
        self.bonus, self.norm_w = tensors[f"{n}.u"].contiguous(), tensors[f"{n}.norm"]

    def bind_all(self, tensors, dtype, device) -> None:
        super().bind_all(tensors, dtype, device)
        self.w2.bias = tensors[f"{self.name}.w0"]   # the decay's offset is the bias of its second product

    def _gated(self, ctx, x, cache):
        T, D, HD, HDp, Dp = x.shape[0], self.width, self.inner, self.inner_p, self.width_p
        shift, rule = cache.side("shift"), cache.side("wkv")
        mixes = ctx.ws.get("wkv_mixes", T, len(self.MIXES) * Dp, x.dtype)
        ops.label(self.name + ".shift", 2.0 * len(self.MIXES) * T * D, x.element_size() * (len(self.MIXES) + 1.0) * T * D)
        ops.token_shift_mix(x, self.mu, shift.state, shift.slots, ctx.positions, ctx.token_req, ctx.req_first_token,
                            mixes, ctx.stream)
        rkvg = ctx.ws.get("wkv_rkvg", T, 4 * HDp, x.dtype)
        for i, lin in enumerate((self.r, self.k, self.v, self.g)):
            lin.forward(ctx, mixes[:, i * Dp:i * Dp + D], rkvg[:, i * HDp:i * HDp + HD])
        L = self.decay_rank
        lora = ctx.ws.get("wkv_lora", T, (L + 7) // 8 * 8, x.dtype)[:, :L]
        self.w1.forward(ctx, mixes[:, 4 * Dp:4 * Dp + D], lora, activation="tanh")
        decay = ctx.ws.get("wkv_decay", T, HD, torch.float32)
        self.w2.forward(ctx, lora, decay)
        o = ctx.ws.get("wkv_o", T, HD, torch.float32)
        ops.label(self.name + ".scan", 6.0 * T * HD * self.dim, x.element_size() * 3.0 * T * HD + 8.0 * T * HD
                  + 8.0 * min(T, ctx.n_requests) * HD * self.dim)
        ops.wkv_scan(rkvg, 0, HDp, 2 * HDp, decay, self.bonus, rule.state, rule.slots, ctx.token_req, ctx.req_first_token,
                     o, self.n_heads, ctx.stream)
        gated = ctx.ws.get("wkv_gated", T, HD, x.dtype)
        ops.label(self.name + ".norm", 8.0 * T * HD, (4.0 + 2 * x.element_size()) * T * HD)
        ops.rmsnorm(o, self.norm_w, gated, self.eps, ctx.stream, groups=self.n_heads, gate=rkvg[:, 3 * HDp:3 * HDp + HD],
                    gate_mode=ops.GATE_AFTER)
        return gated

    def mix(self, ctx, x, cache, tag: str = "mix_wkv"):
        g = self._gated(ctx, x, cache)
        return self.out.forward(ctx, g, ctx.ws.get(tag, x.shape[0], self.width, torch.float32))

    def forward(self, ctx, x, residual, cache):
        return self.out.forward(ctx, self._gated(ctx, x, cache), residual, residual=residual)


register_part("mixer", "mamba2", Mamba2Mixer)
register_part("mixer", "wkv", WKVMixer)
register_part("mixer", "gated_delta", GatedDeltaMixer)
