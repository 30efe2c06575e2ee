"""Host ledger of cache pages: who holds which page.

A pool hands out page numbers and takes them back; it knows nothing of the memory
behind them.  Every page is either free or held by exactly one owner; freeing a page
that is free, or that another owner holds, is an error rather than a silent repair.
The reference keeps the same facts per page as `{generation, references}` with leases
that are checked on return (crates/engine/state/src/blocks.rs:8-28, :70-82, :208-225);
without prefix sharing one owner per page is enough.

The ledger itself is C++ (`host/ilb_host.cpp`, `Pool`); this class gives owners of any
hashable type a number and turns the library's codes into exceptions.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Hashable, List, Optional

from .. import host


class OutOfPages(RuntimeError):
    """The pool cannot cover the request; nothing was taken."""


class PageLedgerError(RuntimeError):
    """A page was freed twice, freed by a stranger, or is otherwise misaccounted."""


class OwnerIds:
    """Numbers for owners of any hashable type (the C++ side knows owners as integers)."""

    def __init__(self) -> None:
        self._id: Dict[Hashable, int] = {}
        self._name: Dict[int, Hashable] = {}
        self._pinned = set()
        self._next = 0

    def of(self, owner: Hashable) -> int:
        i = self._id.get(owner)
        if i is None:
            i = self._id[owner] = self._next
            self._name[i] = owner
            self._next += 1
        return i

    def name(self, i: int) -> Optional[Hashable]:
        return self._name.get(i)

    def pin(self, owner: Hashable) -> int:
        """Keep this owner's number until `unpin` (a scheduled request is known by it for its
        whole life, across preemptions)."""
        i = self.of(owner)
        self._pinned.add(owner)
        return i

    def unpin(self, owner: Hashable) -> None:
        self._pinned.discard(owner)

    def forget(self, owner: Hashable) -> None:
        if owner in self._pinned:
            return
        i = self._id.pop(owner, None)
        if i is not None:
            self._name.pop(i, None)

    def legend(self) -> str:
        if not self._id or len(self._id) > 8:
            return ""
        return " (owners: " + ", ".join(f"{i}={o!r}" for o, i in self._id.items()) + ")"


def raise_for(code: int, ids: Optional[OwnerIds] = None) -> None:
    """Turn a negative return code of the host library into the matching exception."""
    msg = host.last_error() + (ids.legend() if ids is not None else "")
    if code == host.OUT_OF_PAGES:
        raise OutOfPages(msg)
    if code == host.LEDGER:
        raise PageLedgerError(msg)
    if code == host.OUT_OF_SLOTS:
        from .slots import OutOfSlots
        raise OutOfSlots(msg)
    raise ValueError(msg)


class PagePool:
    def __init__(self, num_pages: int, _handle: Optional[int] = None, _ids: Optional[OwnerIds] = None) -> None:
        self._lib = host.lib()
        self._owned = _handle is None
        if _handle is None:
            if num_pages <= 0:
                raise ValueError("a page pool needs at least one page")
            h = ctypes.c_void_p()
            rc = self._lib.ilb_pool_new(int(num_pages), ctypes.byref(h))
            if rc:
                raise_for(rc)
            _handle = h.value
        self._h = ctypes.c_void_p(_handle)
        self.num_pages = int(num_pages)
        self._ids = _ids if _ids is not None else OwnerIds()

    def __del__(self) -> None:
        if getattr(self, "_owned", False) and getattr(self, "_h", None) is not None:
            self._lib.ilb_pool_free(self._h)
            self._h = None

    @property
    def num_free(self) -> int:
        return self._lib.ilb_pool_num_free(self._h)

    def _counters(self):
        out = (ctypes.c_longlong * 2)()
        self._lib.ilb_pool_counters(self._h, out)
        return out[0], out[1]

    @property
    def allocations(self) -> int:
        return self._counters()[0]

    @property
    def reuses(self) -> int:
        return self._counters()[1]

    def owner_of(self, page: int) -> Optional[Hashable]:
        i = self._lib.ilb_pool_owner_of(self._h, int(page))
        return None if i < 0 else self._ids.name(i)

    def take(self, owner: Hashable, count: int) -> List[int]:
        """`count` pages for `owner`, or OutOfPages with nothing taken."""
        if owner is None:
            raise ValueError("owner must not be None")
        if count < 0:
            raise ValueError("negative page count")
        out = (ctypes.c_int * max(1, count))()
        rc = self._lib.ilb_pool_take(self._h, self._ids.of(owner), int(count), out)
        if rc < 0:
            raise_for(rc, self._ids)
        return list(out[:count])

    def give_back(self, owner: Hashable, pages: List[int]) -> None:
        arr = (ctypes.c_int * max(1, len(pages)))(*[int(p) for p in pages])
        rc = self._lib.ilb_pool_give_back(self._h, self._ids.of(owner), arr, len(pages))
        if rc < 0:
            raise_for(rc, self._ids)

    def check(self) -> None:
        """Every page is free or owned, never both, never neither, none listed twice."""
        rc = self._lib.ilb_pool_check(self._h)
        if rc < 0:
            raise_for(rc, self._ids)

    def held_by(self, owner: Hashable) -> List[int]:
        i = self._ids.of(owner)
        return [p for p in range(self.num_pages) if self._lib.ilb_pool_owner_of(self._h, p) == i]
