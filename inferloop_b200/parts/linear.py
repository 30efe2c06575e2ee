"""y = x W^T (+ b): the one place that decides which matrix kernel runs.

Weights are stored [out, in] (crates/model/recipes/src/decoder.rs:55-64).  On the 32-bit
path every product is an exact 32-bit multiply-add in a fixed order (gemm_simt.cu).  On
the bfloat16 path the tensor-core kernel runs when the shape meets its alignment rules;
any other shape takes the same exact kernel with bfloat16 inputs.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
           bias: Optional[torch.Tensor] = None, accumulate: bool = False) -> None:
    """out (+)= x @ weight.T (+ bias).  `accumulate` adds into a 32-bit `out`."""
    if x.dtype == torch.bfloat16 and ops.gemm_tc_eligible(x, weight, out):
        ops.gemm_tc(x, weight, out, bias, accumulate)
    else:
        ops.gemm_simt(x, weight, out, bias, accumulate)
