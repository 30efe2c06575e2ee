"""Slots for per-request state of fixed size.

A request takes one slot when it starts and keeps it until it ends; a mixer that
carries state of its own (a recurrent matrix, a convolution history) finds it at
`state[slot]`.  The reference gives a request one slot of its pool for life the same way
(crates/backend/cuda/src/resident/slot_batch.rs:364-403).  The attention-only
architecture built here declares no such state, but the slot is allocated all the same
so that a layer that needs it has it.

The pool itself is C++ (`host/ilb_host.cpp`, `Slots`).
"""
from __future__ import annotations

import ctypes
from typing import Hashable, Optional

from .. import host
from .pages import OwnerIds, raise_for


class OutOfSlots(RuntimeError):
    pass


class SlotPool:
    def __init__(self, num_slots: int, _handle: Optional[int] = None, _ids: Optional[OwnerIds] = None) -> None:
        self._lib = host.lib()
        self._owned = _handle is None
        if _handle is None:
            if num_slots <= 0:
                raise ValueError("a slot pool needs at least one slot")
            h = ctypes.c_void_p()
            rc = self._lib.ilb_slots_new(int(num_slots), ctypes.byref(h))
            if rc:
                raise_for(rc)
            _handle = h.value
        self._h = ctypes.c_void_p(_handle)
        self.num_slots = int(num_slots)
        self._ids = _ids if _ids is not None else OwnerIds()

    def __del__(self) -> None:
        if getattr(self, "_owned", False) and getattr(self, "_h", None) is not None:
            self._lib.ilb_slots_free(self._h)
            self._h = None

    @property
    def num_free(self) -> int:
        return self._lib.ilb_slots_num_free(self._h)

    def slot_of(self, owner: Hashable) -> int:
        s = self._lib.ilb_slots_slot_of(self._h, self._ids.of(owner))
        if s < 0:
            raise KeyError(owner)
        return s

    def take(self, owner: Hashable) -> int:
        s = self._lib.ilb_slots_take(self._h, self._ids.of(owner))
        if s < 0:
            raise_for(s, self._ids)
        return s

    def give_back(self, owner: Hashable) -> int:
        s = self._lib.ilb_slots_give_back(self._h, self._ids.of(owner))
        if s < 0:
            raise_for(s, self._ids)
        return s

    def check(self) -> None:
        rc = self._lib.ilb_slots_check(self._h)
        if rc < 0:
            raise RuntimeError(host.last_error())
