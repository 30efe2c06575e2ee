"""Rotary position encoding, half-split (NeoX) pairing.

For i in [0, rd/2): angle_i = pos / theta^(2i/rd); the pair (x[i], x[i + rd/2]) is
rotated by it; elements past rd pass through
(crates/testing/cpu/reference-ops/src/kernels.rs:217-241; rd = floor(d * factor),
crates/model/recipes/src/decoder.rs:516-522).  The inverse frequencies are made in
64-bit on the host, as the reference's loader does
(crates/backend/cuda/src/loading/head_padding.rs:170-180); the per-token cos/sin table is
evaluated in 64-bit on the device and rounded once, and is shared by every layer of a
step that has the same constants.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from .base import PositionEncoding
from .registry import register


class RopeNeox(PositionEncoding):
    graph_safe = True
    def __init__(self, spec, ctx, prefix: str = "") -> None:
        super().__init__(spec, ctx, prefix)
        self.theta = float(spec["theta"])
        self.rotary_dim = int(spec["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and positive")
        self._inv_freq: Optional[torch.Tensor] = None

    @property
    def key(self):
        return ("rope_neox", self.theta, self.rotary_dim)

    def inv_freq(self) -> torch.Tensor:
        if self._inv_freq is None:
            half = self.rotary_dim // 2
            host = [self.theta ** (-(2.0 * i) / self.rotary_dim) for i in range(half)]
            self._inv_freq = torch.tensor(host, dtype=torch.float64, device=self.ctx.device)
        return self._inv_freq

    def table(self, step) -> Optional[torch.Tensor]:
        cached = step.position_tables.get(self.key)
        if cached is None:
            half = self.rotary_dim // 2
            cached = self.ctx.workspace.buffer(
                f"rope_table/{self.theta}/{self.rotary_dim}", (step.n_tokens, half, 2), torch.float32)
            ops.rope_table(step.positions, self.inv_freq(), cached)
            step.position_tables[self.key] = cached
        return cached


class NoPosition(PositionEncoding):
    graph_safe = True
    """A mixer that wants no position signal."""

    def table(self, step):
        return None


register("position", "rope_neox", RopeNeox)
register("position", "none", NoPosition)
