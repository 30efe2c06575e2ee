"""What a part says about each tensor it needs."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass(frozen=True)
class WeightDecl:
    """One tensor a part needs, by name.

    role:  "matrix" and "table" follow the engine's compute dtype (bfloat16, or float32
           on the 32-bit path); "vector" (norm weights, biases) is held in float32, which
           keeps a 32-bit tensor as stored and widens a 16-bit one without loss;
           "int" is an integer table held as int32.
    init:  distribution used by the random-weights mode: "normal" N(0, 0.02),
           "norm" 1 + N(0, 0.1), "bias" N(0, 0.02), "zeros".
    root:  True when the name is not under the model's weight prefix
           (`lm_head.weight`, crates/foundation/spi/src/model.rs:220-226).
    """

    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    root: bool = False

    def under(self, prefix: str) -> "WeightDecl":
        if self.root:
            return self
        return WeightDecl(prefix + self.name, self.shape, self.role, self.init, self.root)
