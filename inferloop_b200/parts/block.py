"""Pre-norm residual block: h += mixer(norm1(h)); h += ffn(norm2(h))
(crates/model/recipes/src/decoder.rs:112-120 and :474-480)."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..csrc import ops
from ..weights.decl import WeightDecl
from . import registry
from .base import Block, CacheNeeds


class PreNormBlock(Block):
    """spec: hidden_size, and the tensor-name pieces of this arrangement:
    mixer_prefix, ffn_prefix, mixer_norm, ffn_norm (names under the layer prefix)."""

    def __init__(self, spec, ctx, prefix: str = "", layer=None) -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        mixer_prefix = prefix + spec.get("mixer_prefix", "self_attn.")
        ffn_prefix = prefix + spec.get("ffn_prefix", "mlp.")
        norm_cls_args = dict(width=self.hidden)
        self.norm1 = registry.build_norm(layer.norm, ctx, prefix + spec.get("mixer_norm", "input_layernorm."), **norm_cls_args)
        self.norm2 = registry.build_norm(layer.norm, ctx, prefix + spec.get("ffn_norm", "post_attention_layernorm."), **norm_cls_args)
        self.mixer = registry.build("mixer", layer.mixer, ctx, mixer_prefix)
        self.ffn = registry.build("feed_forward", layer.feed_forward, ctx, ffn_prefix)

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in (self.norm1, self.mixer, self.norm2, self.ffn))

    def declare_weights(self) -> List[WeightDecl]:
        return (self.norm1.declare_weights() + self.mixer.declare_weights()
                + self.norm2.declare_weights() + self.ffn.declare_weights())

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for part in (self.norm1, self.mixer, self.norm2, self.ffn):
            part.bind(tensors)

    def cache_needs(self) -> CacheNeeds:
        return self.mixer.cache_needs()

    def scratch_bytes(self, tokens: int) -> int:
        size = torch.empty((), dtype=self.ctx.dtype).element_size()
        return tokens * self.hidden * size + self.mixer.scratch_bytes(tokens) + self.ffn.scratch_bytes(tokens)

    def forward(self, hidden: torch.Tensor, step, cache) -> None:
        ws = self.ctx.workspace
        normed = ws.buffer("block.normed", hidden.shape, self.ctx.dtype)
        ops.scope("norm")
        self.norm1.forward(hidden, normed)
        ops.scope("mixer")
        self.mixer.forward(normed, hidden, step, cache)
        ops.scope("norm")
        self.norm2.forward(hidden, normed)
        ops.scope("feed_forward")
        self.ffn.forward(normed, hidden, step)


registry.register("block", "pre_norm", PreNormBlock)
