"""SwiGLU feed-forward: residual += W_down (silu(W_gate x) * (W_up x)).

(crates/model/recipes/src/decoder.rs:467-502; silu(z) = z * sigmoid(z) with the
two-branch sigmoid of crates/testing/cpu/reference-ops/src/kernels.rs:12-22.)  The gate
and up matrices are concatenated at load into one [2 I, H] matrix so one GEMM produces
both.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..csrc import ops
from ..weights.decl import WeightDecl
from .base import FeedForward
from .linear import linear
from .registry import register


class SwiGLU(FeedForward):
    graph_safe = True
    def __init__(self, spec, ctx, prefix: str = "") -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.names = {"gate": prefix + "gate_proj.weight", "up": prefix + "up_proj.weight",
                      "down": prefix + "down_proj.weight"}
        self.w_gate_up = self.w_down = None

    def declare_weights(self) -> List[WeightDecl]:
        n = self.names
        return [WeightDecl(n["gate"], (self.inter, self.hidden)),
                WeightDecl(n["up"], (self.inter, self.hidden)),
                WeightDecl(n["down"], (self.hidden, self.inter))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.w_gate_up = torch.cat([tensors[n["gate"]], tensors[n["up"]]], dim=0).contiguous()
        self.w_down = tensors[n["down"]].contiguous()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, step) -> None:
        T = x.shape[0]
        ws, dt = self.ctx.workspace, self.ctx.dtype
        gate_up = ws.buffer("mlp.gate_up", (T, 2 * self.inter), dt)
        linear(x, self.w_gate_up, gate_up)
        act = ws.buffer("mlp.act", (T, self.inter), dt)
        ops.silu_mul(gate_up, act)
        linear(act, self.w_down, residual, accumulate=True)


register("feed_forward", "swiglu", SwiGLU)
