"""Nufetar: a decoder-only model whose config.json lists its layers one by one.

Every layer is a pre-norm block over a float32 residual stream (``parts.StreamBlock``) with plain RMS norms: a
mixer and an optional dense feed-forward whose activation has two learned numbers.  Three kinds of mixer:

``attention``         grouped-query attention with biases, a rotation of the first ``rot.dims`` dimensions (pairs
                      ``(i, i + dims/2)``), values divided by their root mean square, scores mixed across heads
                      before the softmax, keys visible inside runs of ``mask.size`` positions counted from the
                      sequence's start, and a sigmoid gate per head (``parts.TalkingHeadsAttention``);
``latent_attention``  attention over latent rows ``[c | rotated key part]`` shared by all heads, rotation pairs
                      ``(2i, 2i+1)``, a sliding window of ``mask.size`` positions (``parts.LatentAttention``);
``wkv``               a linear recurrence per head with a decay computed from the data (``parts.WKVMixer``).

The output head is the embedding table.

config.json keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``layers`` (``type``, ``mixer``, ``mlp``).  Tensor
names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.up|down|act``, ``final.norm``.  The inner size of the
decay's two products is not a key of the configuration: it is the first dimension of ``l<i>.mix.w1`` (a key
``decay_rank`` of the mixer, where present, says the same; the random-weights mode needs it or takes 32).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..config.base import BaseModelArgs, ConfigError, _positive_int
from ..config.registry import register_architecture
from ..parts import (Init, LatentAttention, LearnedActMLP, ModelDescription, OutputHead, RMSNorm, StreamBlock,
                     TalkingHeadsAttention, TokenEmbedding, WKVMixer)

DEFAULT_DECAY_RANK = 32


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

    def validate(self) -> None:
        _positive_int("vocab", self.vocab)
        _positive_int("width", self.width)
        _need(self.norm, ["eps"], "norm")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("layers must be a non-empty list")
        for i, spec in enumerate(self.layers):
            _need(spec, ["type", "mixer"], f"layers[{i}]")
            m, where = spec["mixer"], f"layers[{i}].mixer"
            if spec["type"] == "attention":
                _need(m, ["dim", "heads", "kv_heads", "mask", "rot", "scale", "vdim"], where)
                _need(m["rot"], ["base", "dims"], where + ".rot")
                _need(m["mask"], ["size"], where + ".mask")
            elif spec["type"] == "latent_attention":
                _need(m, ["dim", "heads", "kv_rank", "mask", "rot", "rot_dim", "scale", "vdim"], where)
                _need(m["rot"], ["base", "dims"], where + ".rot")
                _need(m["mask"], ["size"], where + ".mask")
                if m["rot"]["dims"] != m["rot_dim"]:
                    raise ConfigError(f"{where}: rot.dims {m['rot']['dims']} is not rot_dim {m['rot_dim']}")
            elif spec["type"] == "wkv":
                _need(m, ["dim", "heads"], where)
            else:
                raise ConfigError(f"layers[{i}].type {spec['type']!r}: 'attention', 'latent_attention' or 'wkv'")
            mlp = spec.get("mlp")
            if mlp is not None:
                _need(mlp, ["ff", "kind"], f"layers[{i}].mlp")
                if mlp["kind"] != "dense":
                    raise ConfigError(f"layers[{i}].mlp.kind {mlp['kind']!r}: 'dense'")

    def sizes_from_tensors(self, shapes: dict) -> None:
        """Sizes that only the weight files give (``shapes``: tensor name -> shape)."""
        for i, spec in enumerate(self.layers):
            w1 = shapes.get(f"l{i}.mix.w1")
            if spec["type"] == "wkv" and "decay_rank" not in spec["mixer"] and w1 is not None:
                spec["mixer"] = dict(spec["mixer"], decay_rank=int(w1[0]))

    @property
    def vocab_size(self) -> int:
        return self.vocab


def _mixer(name: str, D: int, spec: dict, eps: float):
    m = spec["mixer"]
    lin = Init(0.0, D ** -0.5)
    if spec["type"] == "attention":
        return TalkingHeadsAttention(name, D, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], eps,
                                     rot_dims=m["rot"]["dims"], rot_base=m["rot"]["base"], interleaved=False, bias=True,
                                     talk=True, value_norm=True, head_gate=True, chunk=int(m["mask"]["size"]), init=lin,
                                     bias_init=Init(0.0, 0.1))
    if spec["type"] == "latent_attention":
        return LatentAttention(name, D, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["scale"], eps,
                               rot_base=m["rot"]["base"], interleaved=True, window=int(m["mask"]["size"]), init=lin)
    return WKVMixer(name, D, m["heads"], m["dim"], int(m.get("decay_rank", DEFAULT_DECAY_RANK)), eps, init=lin)


def build(args: ModelArgs) -> ModelDescription:
    D, eps = args.width, float(args.norm["eps"])
    embed = TokenEmbedding("embed", args.vocab, D, weight_suffix="", stream_dtype=torch.float32, init=Init(0.0, 1.0))
    blocks = []
    for i, spec in enumerate(args.layers):
        p = f"l{i}"
        norm_2 = ff = None
        if spec.get("mlp") is not None:
            norm_2 = RMSNorm(f"{p}.norm2", D, eps)
            ff = LearnedActMLP(f"{p}.mlp", D, int(spec["mlp"]["ff"]), activation="xielu", init=Init(0.0, D ** -0.5))
        blocks.append(StreamBlock(RMSNorm(f"{p}.norm1", D, eps), _mixer(f"{p}.mix", D, spec, eps), norm_2, ff))
    return ModelDescription(
        model_type="nufetar", width=D, vocab_size=args.vocab, embedding=embed, position=None, blocks=blocks,
        final_norm=RMSNorm("final.norm", D, eps), head=OutputHead(args.vocab, D, tied_to=embed), args=args)


register_architecture("nufetar", ModelArgs, build)
