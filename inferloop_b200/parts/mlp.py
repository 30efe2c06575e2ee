"""SwiGLU feed-forward: residual += W_down (silu(W_gate x) * (W_up x)).

(crates/model/recipes/src/decoder.rs:467-502; silu(z) = z * sigmoid(z) with the
two-branch sigmoid of crates/testing/cpu/reference-ops/src/kernels.rs:12-22.)  The gate
and up matrices are concatenated at load into one [2 I, H] matrix so one GEMM produces
both.  On the bfloat16 path, when I is a multiple of 64, their rows are interleaved in
blocks of 64 (64 gate rows, then the 64 up rows of the same features) and the product
silu(gate) * up is taken in the GEMM's epilogue, so the [T, 2 I] intermediate is never
written (the reference pairs the two projections in one launch and multiplies in a second:
crates/backend/cuda-kernels/src/tile/projection/prefill_gemm_kernels.rs:11-69,
tile/mlp/mlp_kernels.rs:27-36); otherwise the product is a kernel of its own.
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
        self.fused = False

    def declare_weights(self) -> List[WeightDecl]:
        n = self.names
        return [WeightDecl(n["gate"], (self.inter, self.hidden)),
                WeightDecl(n["up"], (self.inter, self.hidden)),
                WeightDecl(n["down"], (self.hidden, self.inter))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        gate, up = tensors[n["gate"]], tensors[n["up"]]
        self.fused = (gate.dtype == torch.bfloat16 and self.inter % 64 == 0 and self.hidden % 8 == 0)
        if self.fused:
            blocks = self.inter // 64
            self.w_gate_up = torch.stack(
                [gate.view(blocks, 64, self.hidden), up.view(blocks, 64, self.hidden)], dim=1
            ).reshape(2 * self.inter, self.hidden).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors[n["down"]].contiguous()

    def scratch_bytes(self, tokens: int) -> int:
        size = torch.empty((), dtype=self.ctx.dtype).element_size()
        fused = self.ctx.dtype == torch.bfloat16 and self.inter % 64 == 0 and self.hidden % 8 == 0
        return tokens * self.inter * size * (1 if fused else 3)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, step) -> None:
        T = x.shape[0]
        ws, dt = self.ctx.workspace, self.ctx.dtype
        act = ws.buffer("mlp.act", (T, self.inter), dt)
        ops.scope("feed_forward.gate_up (SwiGLU inside)" if self.fused else "feed_forward.gate_up")
        if self.fused and ops.gemm_tc_eligible(x, self.w_gate_up, act):
            ops.gemm_tc(x, self.w_gate_up, act, swiglu=True)
        elif self.fused:
            raise ops.KernelError("SwiGLU: the interleaved weight needs the tensor-core GEMM, which refused this input")
        else:
            gate_up = ws.buffer("mlp.gate_up", (T, 2 * self.inter), dt)
            linear(x, self.w_gate_up, gate_up)
            ops.scope("feed_forward.swiglu")
            ops.silu_mul(gate_up, act)
        ops.scope("feed_forward.down")
        linear(act, self.w_down, residual, accumulate=True)


register("feed_forward", "swiglu", SwiGLU)
