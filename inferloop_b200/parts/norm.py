"""RMSNorm: x / sqrt(mean(x^2) + eps) * weight, computed in 32-bit
(crates/testing/cpu/reference-ops/src/kernels.rs:38-54; weight offset 0 for this family,
crates/model/package/src/providers/qwen/mod.rs:252)."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..csrc import ops
from ..weights.decl import WeightDecl
from .base import Norm
from .registry import register


class RMSNorm(Norm):
    graph_safe = True
    """spec: eps; width is given by the owner through `prefix`-named weight of `width`."""

    def __init__(self, spec, ctx, prefix: str = "", width: int = 0, name: str = "weight") -> None:
        super().__init__(spec, ctx, prefix)
        self.eps = float(spec["eps"])
        self.width = int(width or spec.get("width", 0))
        self.weight_name = prefix + name
        self.weight = None

    def declare_weights(self) -> List[WeightDecl]:
        return [WeightDecl(self.weight_name, (self.width,), role="vector", init="norm")]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        ops.rmsnorm(x, self.weight, self.eps, out)


register("norm", "rms", RMSNorm)
