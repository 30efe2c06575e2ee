"""Sampling options of a request: the reference's names, defaults and ranges
(crates/foundation/ir/src/request.rs:44-68 fields and defaults, :165-183 ranges)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0            # 0 selects the highest logit
    top_k: Optional[int] = None         # keep the k best; None disables
    top_p: float = 1.0                  # smallest sorted prefix with mass >= p
    min_p: float = 0.0                  # drop candidates whose weight relative to the best is below
    presence_penalty: float = 0.0       # subtracted from logits of generated tokens
    repetition_penalty: float = 1.0     # divides positive / multiplies negative logits of seen tokens
    eos_tokens: Tuple[int, ...] = ()
    seed: int = 0
    eos_token: Optional[int] = None

    def __post_init__(self) -> None:
        object.__setattr__(self, "eos_tokens", tuple(int(t) for t in self.eos_tokens))
        ok = (math.isfinite(self.temperature) and self.temperature >= 0.0
              and self.top_k != 0 and (self.top_k is None or self.top_k > 0)
              and math.isfinite(self.top_p) and 0.0 < self.top_p <= 1.0
              and math.isfinite(self.min_p) and 0.0 <= self.min_p <= 1.0
              and math.isfinite(self.presence_penalty) and -2.0 <= self.presence_penalty <= 2.0
              and math.isfinite(self.repetition_penalty) and self.repetition_penalty > 0.0
              and 0 <= int(self.seed) < (1 << 64))
        if not ok:
            raise ValueError("invalid sampling parameters")

    def uses_plain_greedy(self) -> bool:
        """Highest logit directly, no penalties (request.rs:154-160)."""
        return (self.temperature == 0.0 and self.presence_penalty == 0.0
                and self.repetition_penalty == 1.0)

    def uses_plain_temperature(self) -> bool:
        """A draw from softmax(logits / T) with no filter and no penalty."""
        return (self.temperature > 0.0 and self.top_k is None and self.top_p == 1.0
                and self.min_p == 0.0 and self.presence_penalty == 0.0
                and self.repetition_penalty == 1.0)

    def is_eos(self, token: int) -> bool:
        return token == self.eos_token or token in self.eos_tokens
