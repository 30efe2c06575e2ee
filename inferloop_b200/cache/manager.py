"""The cache manager: pages of keys and values with a block table per request, one page
group per distinct need, and a slot of fixed-size state per request.

Layers are sorted into *page groups* by what they need (`PagedKVNeed`: kv heads, head
size, window).  A group has its own pool, its own block tables and one device tensor
`[layers_in_group, 2, pages, kv_heads, page_size, head_dim]`; layer l's keys are
`storage[l, 0]`, its values `storage[l, 1]`.  Pages are taken when the step that first
touches them is prepared, all groups or none (the reference grows pages per step,
all-or-nothing: crates/engine/state/src/logical/reservation.rs:106-158), and given back
when the request ends (crates/engine/runtime/src/pipeline/lifecycle.rs:242-251) or, in a
group with a window, as soon as every position of a page is older than any key a future
token can read.  A released entry of a block table becomes -1; kernels never follow it.

Everything here is host bookkeeping; with `device=None` no memory is allocated, which
is how the ledger is tested without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from ..config.spec import RunEntry
from ..parts.base import CacheNeeds, PagedKVNeed, SlotStateNeed
from .pages import OutOfPages, PageLedgerError, PagePool
from .slots import OutOfSlots, SlotPool


@dataclass
class LayerCache:
    """What a mixer gets: its keys/values (or None), the group whose block table applies,
    whether this run-order entry may write them, and its slot-state tensors by name."""
    layer: int
    group: Optional[int]
    page_size: int
    k: Optional[torch.Tensor]
    v: Optional[torch.Tensor]
    writable: bool
    state: Dict[str, torch.Tensor] = field(default_factory=dict)


@dataclass
class PageGroup:
    index: int
    need: PagedKVNeed
    layers: List[int]
    pool: PagePool
    page_size: int
    storage: Optional[torch.Tensor] = None
    tables: Dict[Hashable, List[int]] = field(default_factory=dict)

    def page_bytes(self, element_size: int) -> int:
        return (len(self.layers) * 2 * self.need.kv_heads * self.page_size
                * self.need.head_dim * element_size)


class CacheManager:
    def __init__(self, layer_needs: Sequence[CacheNeeds], page_size: int, num_pages: int,
                 max_requests: int, dtype: torch.dtype = torch.float32,
                 device: Optional[torch.device] = None,
                 run_order: Optional[Sequence[RunEntry]] = None) -> None:
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = int(page_size)
        self.dtype = dtype
        self.device = device
        self.layer_needs = list(layer_needs)
        n_layers = len(self.layer_needs)
        order = list(run_order) if run_order is not None else [RunEntry(i, i) for i in range(n_layers)]
        # Only layers that some entry names as cache owner hold memory.
        owners = sorted({e.cache_of for e in order})
        self.groups: List[PageGroup] = []
        self._group_of_layer: Dict[int, int] = {}
        self._index_in_group: Dict[int, int] = {}
        for layer in owners:
            need = self.layer_needs[layer].paged
            if need is None:
                continue
            for g in self.groups:
                if g.need == need:
                    break
            else:
                g = PageGroup(len(self.groups), need, [], PagePool(num_pages), self.page_size)
                self.groups.append(g)
            self._group_of_layer[layer] = g.index
            self._index_in_group[layer] = len(g.layers)
            g.layers.append(layer)
        if device is not None:
            for g in self.groups:
                g.storage = torch.zeros(
                    (len(g.layers), 2, num_pages, g.need.kv_heads, self.page_size, g.need.head_dim),
                    dtype=dtype, device=device)
        # fixed-size state
        self.slots = SlotPool(max_requests)
        self._slot_state: Dict[Tuple[int, str], torch.Tensor] = {}
        self._slot_needs: Dict[int, Tuple[SlotStateNeed, ...]] = {}
        for layer in owners:
            needs = self.layer_needs[layer].slots
            if needs:
                self._slot_needs[layer] = tuple(needs)
                if device is not None:
                    for need in needs:
                        self._slot_state[(layer, need.name)] = torch.zeros(
                            (max_requests,) + tuple(need.shape), dtype=need.dtype, device=device)
        self._length: Dict[Hashable, int] = {}
        self.stats = {"begun": 0, "released": 0, "window_pages_released": 0}

    # ------------------------------------------------------------------ requests
    def has(self, request: Hashable) -> bool:
        return request in self._length

    def length(self, request: Hashable) -> int:
        """Tokens of `request` whose keys and values are in the cache."""
        return self._length[request]

    def live_requests(self) -> List[Hashable]:
        return list(self._length)

    def begin(self, request: Hashable) -> int:
        """Register a request: takes its state slot (zeroed), no pages yet."""
        if request in self._length:
            raise ValueError(f"request {request!r} is already live")
        slot = self.slots.take(request)
        for t in self._slot_state.values():
            t[slot].zero_()
        self._length[request] = 0
        for g in self.groups:
            g.tables[request] = []
        self.stats["begun"] += 1
        return slot

    def slot_of(self, request: Hashable) -> int:
        return self.slots.slot_of(request)

    def _first_needed_block(self, g: PageGroup, first_query_pos: int) -> int:
        """Blocks below this index hold only keys no present or future token reads."""
        if g.need.window is None:
            return 0
        oldest_key = max(0, first_query_pos - g.need.window + 1)
        return oldest_key // self.page_size

    def pages_needed(self, request: Hashable, new_length: int) -> Dict[int, int]:
        """Pages each group must still take to cover tokens [0, new_length), after the
        pages a window lets go are counted as returned."""
        cur = self._length[request]
        out = {}
        for g in self.groups:
            table = g.tables[request]
            want = -(-new_length // self.page_size)
            first = self._first_needed_block(g, cur)
            releasable = sum(1 for b in range(min(first, len(table))) if table[b] >= 0)
            out[g.index] = max(0, want - len(table)) - releasable
        return out

    def ensure(self, request: Hashable, new_length: int) -> None:
        """Make room for tokens [length, new_length) in every group, or raise OutOfPages
        and change nothing but pages a window had already let go."""
        cur = self._length[request]
        if new_length < cur:
            raise ValueError(f"request {request!r} cannot shrink from {cur} to {new_length}")
        for g in self.groups:   # first give back what a window has passed
            table = g.tables[request]
            first = self._first_needed_block(g, cur)
            gone = [table[b] for b in range(min(first, len(table))) if table[b] >= 0]
            if gone:
                g.pool.give_back(request, gone)
                for b in range(min(first, len(table))):
                    table[b] = -1
                self.stats["window_pages_released"] += len(gone)
        want = -(-new_length // self.page_size)
        for g in self.groups:
            extra = want - len(g.tables[request])
            if extra > g.pool.num_free:
                raise OutOfPages(
                    f"request {request!r} needs {extra} more pages in group {g.index}, "
                    f"{g.pool.num_free} free of {g.pool.num_pages}")
        for g in self.groups:
            extra = want - len(g.tables[request])
            if extra > 0:
                g.tables[request].extend(g.pool.take(request, extra))

    def commit(self, request: Hashable, new_length: int) -> None:
        """Record that tokens up to `new_length` are now in the cache."""
        want = -(-new_length // self.page_size)
        for g in self.groups:
            if len(g.tables[request]) < want:
                raise PageLedgerError(
                    f"request {request!r} commits {new_length} tokens but holds "
                    f"{len(g.tables[request])} blocks in group {g.index}")
        if new_length < self._length[request]:
            raise ValueError("commit cannot shrink a request")
        self._length[request] = new_length

    def release(self, request: Hashable) -> None:
        """The request ends (or is preempted): all its pages and its slot come back."""
        if request not in self._length:
            raise ValueError(f"request {request!r} is not live")
        for g in self.groups:
            table = g.tables.pop(request)
            g.pool.give_back(request, [p for p in table if p >= 0])
        self.slots.give_back(request)
        del self._length[request]
        self.stats["released"] += 1

    # ------------------------------------------------------------------ views
    def block_table(self, group: int, request: Hashable) -> List[int]:
        return self.groups[group].tables[request]

    def max_blocks(self, requests: Sequence[Hashable]) -> int:
        m = 1
        for g in self.groups:
            for r in requests:
                m = max(m, len(g.tables[r]))
        return m

    def layer_cache(self, entry: RunEntry) -> LayerCache:
        owner = entry.cache_of
        gi = self._group_of_layer.get(owner)
        k = v = None
        if gi is not None and self.groups[gi].storage is not None:
            s = self.groups[gi].storage[self._index_in_group[owner]]
            k, v = s[0], s[1]
        state = {need.name: self._slot_state[(owner, need.name)]
                 for need in self._slot_needs.get(owner, ()) if (owner, need.name) in self._slot_state}
        return LayerCache(owner, gi, self.page_size, k, v, entry.writes_cache, state)

    # ------------------------------------------------------------------ facts
    def free_pages(self) -> Dict[int, int]:
        return {g.index: g.pool.num_free for g in self.groups}

    def check(self) -> None:
        """Ledger invariants: every page free or held once; tables and pools agree."""
        for g in self.groups:
            g.pool.check()
            seen: Dict[int, Hashable] = {}
            for r, table in g.tables.items():
                for p in table:
                    if p < 0:
                        continue
                    if p in seen:
                        raise PageLedgerError(f"page {p} of group {g.index} is in the tables of {seen[p]!r} and {r!r}")
                    seen[p] = r
                    if g.pool.owner_of(p) != r:
                        raise PageLedgerError(f"page {p} is in {r!r}'s table but owned by {g.pool.owner_of(p)!r}")
            held = g.pool.num_pages - g.pool.num_free
            if held != len(seen):
                raise PageLedgerError(f"group {g.index}: {held} pages held, {len(seen)} in tables (a page is lost)")
        self.slots.check()

    def inspect(self) -> dict:
        """Counterpart of the reference's KvCacheInspection
        (crates/foundation/ir/src/diagnostics.rs:80-98)."""
        return {
            "block_size": self.page_size,
            "live_requests": len(self._length),
            "groups": [{
                "index": g.index, "layers": list(g.layers), "kv_heads": g.need.kv_heads,
                "head_dim": g.need.head_dim, "window": g.need.window,
                "total": g.pool.num_pages, "free": g.pool.num_free,
                "active": g.pool.num_pages - g.pool.num_free,
                "allocations": g.pool.allocations, "reuses": g.pool.reuses,
            } for g in self.groups],
            "slots": {"total": self.slots.num_slots, "free": self.slots.num_free},
            **self.stats,
        }
