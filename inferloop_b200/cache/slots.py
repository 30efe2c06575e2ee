"""Slots for per-request state of fixed size.

A request takes one slot when it starts and keeps it until it ends; a mixer that
carries state of its own (a recurrent matrix, a convolution history) finds it at
`state[slot]`.  The reference gives a request one slot of its pool for life the same way
(crates/backend/cuda/src/resident/slot_batch.rs:364-403).  The attention-only
architecture built here declares no such state, but the slot is allocated all the same
so that a layer that needs it has it.
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional


class OutOfSlots(RuntimeError):
    pass


class SlotPool:
    def __init__(self, num_slots: int) -> None:
        if num_slots <= 0:
            raise ValueError("a slot pool needs at least one slot")
        self.num_slots = int(num_slots)
        self._free: List[int] = list(range(self.num_slots - 1, -1, -1))
        self._holder: List[Optional[Hashable]] = [None] * self.num_slots
        self._slot_of: Dict[Hashable, int] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    def slot_of(self, owner: Hashable) -> int:
        return self._slot_of[owner]

    def take(self, owner: Hashable) -> int:
        if owner in self._slot_of:
            raise ValueError(f"{owner!r} already holds slot {self._slot_of[owner]}")
        if not self._free:
            raise OutOfSlots(f"all {self.num_slots} state slots are in use")
        s = self._free.pop()
        self._holder[s] = owner
        self._slot_of[owner] = s
        return s

    def give_back(self, owner: Hashable) -> int:
        if owner not in self._slot_of:
            raise ValueError(f"{owner!r} holds no slot")
        s = self._slot_of.pop(owner)
        self._holder[s] = None
        self._free.append(s)
        return s

    def check(self) -> None:
        free = set(self._free)
        if len(free) != len(self._free):
            raise RuntimeError("a slot is on the free list twice")
        for s in range(self.num_slots):
            if (self._holder[s] is not None) == (s in free):
                raise RuntimeError(f"slot {s} is misaccounted")
        for owner, s in self._slot_of.items():
            if self._holder[s] != owner:
                raise RuntimeError(f"slot {s} of {owner!r} is recorded for {self._holder[s]!r}")
