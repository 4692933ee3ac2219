"""Lelatar: a decoder-only model whose config.json lists its layers one by one.

Every layer is a pre-norm block over a float32 residual stream (``parts.StreamBlock``): a mixer, an
optional gated feed-forward, and a per-layer token input.  Two kinds of layer: ``mamba2`` (a
selective state-space mixer) and ``parallel`` (softmax attention with sinks beside a gated delta
rule, their normed outputs averaged).  A span of layers may run several times with the same weights
(``loop``): every pass is entered through ``parts.LoopInput`` and keeps caches of its own.  The
norms store their weights around zero; the output head is a tensor of its own.

config.json keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``layers`` (``type``, ``mixer``,
``mlp``), ``loop`` (``start``, ``stop``, ``times``; optional), ``token_side.dim`` (optional).  Tensor names:
``embed``, ``loop.in``, ``loop.step``, ``side.embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.gate|up|down``,
``l<i>.side.gate|proj|norm``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from ..config.base import BaseModelArgs, ConfigError, _positive_int
from ..config.registry import register_architecture
from ..parts import (GatedDeltaMixer, GatedMLP, Init, LoopInput, Mamba2Mixer, ModelDescription, OutputHead,
                     ParallelMixer, Reentry, RMSNorm, RunEntry, SinkAttention, StreamBlock, TokenEmbedding,
                     TokenSideInput)
from ..parts.side import SideTable


def _need(d: dict, keys, what: str) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"{what} must be an object with the keys {', '.join(keys)}")
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"{what} lacks required key(s): {', '.join(missing)}")


@dataclass
class ModelArgs(BaseModelArgs):
    architecture: str
    vocab: int
    width: int
    layers: list
    norm: dict
    loop: Optional[dict] = None
    token_side: Optional[dict] = None

    def validate(self) -> None:
        _positive_int("vocab", self.vocab)
        _positive_int("width", self.width)
        _need(self.norm, ["eps"], "norm")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("layers must be a non-empty list")
        for i, spec in enumerate(self.layers):
            _need(spec, ["type", "mixer"], f"layers[{i}]")
            m = spec["mixer"]
            if spec["type"] == "mamba2":
                _need(m, ["conv", "groups", "heads", "norm_groups", "state", "vdim"], f"layers[{i}].mixer")
            elif spec["type"] == "parallel":
                _need(m, ["left", "right"], f"layers[{i}].mixer")
                _need(m["left"], ["dim", "heads", "kv_heads", "rot", "scale", "vdim"], f"layers[{i}].mixer.left")
                _need(m["left"]["rot"], ["base", "dims"], f"layers[{i}].mixer.left.rot")
                _need(m["right"], ["conv", "dim", "heads", "kv_heads", "vdim"], f"layers[{i}].mixer.right")
            else:
                raise ConfigError(f"layers[{i}].type {spec['type']!r}: 'mamba2' or 'parallel'")
            mlp = spec.get("mlp")
            if mlp is not None:
                _need(mlp, ["ff", "kind"], f"layers[{i}].mlp")
                if mlp["kind"] != "dense":
                    raise ConfigError(f"layers[{i}].mlp.kind {mlp['kind']!r}: 'dense'")
        if self.loop is not None:
            _need(self.loop, ["start", "stop", "times"], "loop")
            a, b, n = self.loop["start"], self.loop["stop"], self.loop["times"]
            if not (0 <= a < b <= len(self.layers)) or n < 1:
                raise ConfigError(f"loop {self.loop}: 0 <= start < stop <= {len(self.layers)} layers, times >= 1")
        if self.token_side is not None:
            _need(self.token_side, ["dim"], "token_side")

    @property
    def vocab_size(self) -> int:
        return self.vocab


def _mixer(name: str, D: int, spec: dict, eps: float):
    m = spec["mixer"]
    lin = Init(0.0, D ** -0.5)
    if spec["type"] == "mamba2":
        return Mamba2Mixer(name, D, m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"], m["conv"], eps,
                           init=lin)
    l, r = m["left"], m["right"]
    left = SinkAttention(f"{name}.left", D, l["heads"], l["kv_heads"], l["dim"], l["vdim"], l["scale"], eps,
                         rot_dims=l["rot"]["dims"], rot_base=l["rot"]["base"], qk_norm=True, sink=True, init=lin)
    right = GatedDeltaMixer(f"{name}.right", D, r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["conv"], eps, init=lin)
    return ParallelMixer(name, D, left, right, eps, scale=0.5)


def build(args: ModelArgs) -> ModelDescription:
    D, eps, n = args.width, float(args.norm["eps"]), len(args.layers)
    embed = TokenEmbedding("embed", args.vocab, D, weight_suffix="", stream_dtype=torch.float32, init=Init(0.0, 1.0))
    extras, side_dim, table = [], 0, None
    if args.token_side is not None:
        side_dim = int(args.token_side["dim"])
        table = SideTable("side.embed", args.vocab, n * side_dim)
        extras.append(table)
    blocks = []
    for i, spec in enumerate(args.layers):
        p = f"l{i}"
        norm_2 = ff = None
        if spec.get("mlp") is not None:
            norm_2 = RMSNorm(f"{p}.norm2", D, eps, offset=1.0)
            ff = GatedMLP(f"{p}.mlp", D, int(spec["mlp"]["ff"]), init=Init(0.0, D ** -0.5))
        branches = []
        if table is not None:
            branches.append(TokenSideInput(f"{p}.side", D, side_dim, table, i * side_dim, eps, init=Init(0.0, D ** -0.5)))
        blocks.append(StreamBlock(RMSNorm(f"{p}.norm1", D, eps, offset=1.0), _mixer(f"{p}.mix", D, spec, eps), norm_2, ff,
                                  branches))
    order: List[object] = []
    reentries = []
    if args.loop is None:
        order = [RunEntry(i) for i in range(n)]
    else:
        a, b, times = args.loop["start"], args.loop["stop"], args.loop["times"]
        reentries.append(LoopInput(D, times, init=Init(0.0, (2 * D) ** -0.5)))
        order += [RunEntry(i) for i in range(a)]
        for t in range(times):
            order.append(Reentry(0, t))
            # every pass keeps caches of its own: the first the blocks' own numbers, later ones numbers beyond them
            order += [RunEntry(i, cache=i if t == 0 else n + (t - 1) * (b - a) + (i - a)) for i in range(a, b)]
        order += [RunEntry(i) for i in range(b, n)]
    return ModelDescription(
        model_type="lelatar", width=D, vocab_size=args.vocab, embedding=embed, position=None, blocks=blocks,
        final_norm=RMSNorm("final.norm", D, eps, offset=1.0),
        head=OutputHead(args.vocab, D, name="head", weight_suffix="", init=Init(0.0, D ** -0.5)),
        order=order, args=args, reentries=reentries, extras=extras)


register_architecture("lelatar", ModelArgs, build)
