"""Host ledger of cache pages: who holds which page.

A pool hands out page numbers and takes them back; it knows nothing of the memory
behind them.  Every page is either free or held by exactly one owner; freeing a page
that is free, or that another owner holds, is an error rather than a silent repair.
The reference keeps the same facts per page as `{generation, references}` with leases
that are checked on return (crates/engine/state/src/blocks.rs:8-28, :70-82, :208-225);
without prefix sharing one owner per page is enough.
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional


class OutOfPages(RuntimeError):
    """The pool cannot cover the request; nothing was taken."""


class PageLedgerError(RuntimeError):
    """A page was freed twice, freed by a stranger, or is otherwise misaccounted."""


class PagePool:
    def __init__(self, num_pages: int) -> None:
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        # Last freed, first reused: a page that comes back is handed out again at once,
        # which keeps the working set small and makes stale contents show up early.
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))
        self._owner: List[Optional[Hashable]] = [None] * self.num_pages
        self.allocations = 0
        self.reuses = 0
        self._ever_used = [False] * self.num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def owner_of(self, page: int) -> Optional[Hashable]:
        return self._owner[page]

    def take(self, owner: Hashable, count: int) -> List[int]:
        """`count` pages for `owner`, or OutOfPages with nothing taken."""
        if owner is None:
            raise ValueError("owner must not be None")
        if count < 0:
            raise ValueError("negative page count")
        if count > len(self._free):
            raise OutOfPages(f"need {count} pages, {len(self._free)} free of {self.num_pages}")
        out = []
        for _ in range(count):
            p = self._free.pop()
            if self._owner[p] is not None:
                raise PageLedgerError(f"free list held page {p}, which {self._owner[p]!r} owns")
            self._owner[p] = owner
            self.allocations += 1
            if self._ever_used[p]:
                self.reuses += 1
            self._ever_used[p] = True
            out.append(p)
        return out

    def give_back(self, owner: Hashable, pages: List[int]) -> None:
        for p in pages:
            if not (0 <= p < self.num_pages):
                raise PageLedgerError(f"page {p} is outside the pool of {self.num_pages}")
            if self._owner[p] is None:
                raise PageLedgerError(f"page {p} freed twice (by {owner!r})")
            if self._owner[p] != owner:
                raise PageLedgerError(f"page {p} belongs to {self._owner[p]!r}, not {owner!r}")
        if len(set(pages)) != len(pages):
            raise PageLedgerError(f"{owner!r} returns a page twice in one call: {pages}")
        for p in pages:
            self._owner[p] = None
            self._free.append(p)

    def check(self) -> None:
        """Every page is free or owned, never both, never neither, none listed twice."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise PageLedgerError("a page is on the free list twice")
        for p in range(self.num_pages):
            owned = self._owner[p] is not None
            if owned == (p in free):
                raise PageLedgerError(
                    f"page {p} is {'both owned and free' if owned else 'neither owned nor free'}")

    def held_by(self, owner: Hashable) -> List[int]:
        return [p for p, o in enumerate(self._owner) if o == owner]
