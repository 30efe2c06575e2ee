"""Maps on the logits, chosen by a model description's `logits_post`.

`soft_cap`: logits = cap * tanh(logits * scale / cap) (cap 0: scale only), computed in 32-bit
in place.  The architecture this engine serves asks for none; the part exists so that an
architecture that does is a description, not an edit of the model runner.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import LogitsPost
from .registry import register


class SoftCap(LogitsPost):
    graph_safe = True

    def __init__(self, spec, ctx, prefix: str = "") -> None:
        super().__init__(spec, ctx, prefix)
        self.cap = float(spec.get("cap", 0.0))
        self.scale = float(spec.get("scale", 1.0))
        if self.cap < 0.0:
            raise ValueError("soft_cap: cap must not be negative")

    def forward(self, logits: torch.Tensor) -> None:
        ops.scale_cap_inplace(logits, self.scale, self.cap)


register("logits", "soft_cap", SoftCap)
