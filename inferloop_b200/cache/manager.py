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

The bookkeeping (pools, block tables, lengths, slots) lives in the C++ host library
(`host/ilb_host.cpp`, `Ledger`); this class owns the device tensors, gives requests of any
hashable type a number, and turns the library's codes into exceptions.  With `device=None`
no memory is allocated, which is how the ledger is tested without a GPU.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from .. import host

from ..config.spec import RunEntry
from ..parts.base import CacheNeeds, PagedKVNeed, SlotStateNeed
from .pages import OutOfPages, OwnerIds, PageLedgerError, PagePool, raise_for
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

    def page_bytes(self, element_size: int) -> int:
        return (len(self.layers) * 2 * self.need.kv_heads * self.page_size
                * self.need.head_dim * element_size)


class CacheManager:
    def __init__(self, layer_needs: Sequence[CacheNeeds], page_size: int, num_pages,
                 max_requests: int, dtype: torch.dtype = torch.float32,
                 device: Optional[torch.device] = None,
                 run_order: Optional[Sequence[RunEntry]] = None) -> None:
        """`num_pages`: one number for every page group, or one number per group in the
        order of :meth:`group_needs` (a group that reads a window needs fewer)."""
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
        found: List[Tuple[PagedKVNeed, List[int]]] = []
        for layer in owners:
            need = self.layer_needs[layer].paged
            if need is None:
                continue
            for gi, (n, layers) in enumerate(found):
                if n == need:
                    break
            else:
                gi = len(found)
                found.append((need, []))
            self._group_of_layer[layer] = gi
            self._index_in_group[layer] = len(found[gi][1])
            found[gi][1].append(layer)
        if isinstance(num_pages, (list, tuple)):
            if len(num_pages) != len(found):
                raise ValueError(f"{len(num_pages)} pool sizes for {len(found)} page groups")
            pages_of = [int(n) for n in num_pages]
        else:
            pages_of = [int(num_pages)] * len(found)
        if any(n <= 0 for n in pages_of):
            raise ValueError("a page pool needs at least one page")
        if max_requests <= 0:
            raise ValueError("a slot pool needs at least one slot")
        self._lib = host.lib()
        self._ids = OwnerIds()
        windows = (ctypes.c_int * max(1, len(found)))(*[(-1 if n.window is None else int(n.window)) for n, _ in found])
        h = ctypes.c_void_p()
        sizes = (ctypes.c_int * max(1, len(found)))(*pages_of)
        rc = self._lib.ilb_ledger_new(len(found), windows, sizes, self.page_size, int(max_requests), ctypes.byref(h))
        if rc:
            raise_for(rc)
        self._h = h
        for gi, (need, layers) in enumerate(found):
            pool = PagePool(pages_of[gi], _handle=self._lib.ilb_ledger_pool(self._h, gi), _ids=self._ids)
            self.groups.append(PageGroup(gi, need, layers, pool, self.page_size))
        if device is not None:
            for g in self.groups:
                g.storage = torch.zeros(
                    (len(g.layers), 2, g.pool.num_pages, g.need.kv_heads, self.page_size, g.need.head_dim),
                    dtype=dtype, device=device)
        # fixed-size state
        self.slots = SlotPool(max_requests, _handle=self._lib.ilb_ledger_slots(self._h), _ids=self._ids)
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
        self._live: Dict[Hashable, int] = {}        # request -> its number in the ledger

    def __del__(self) -> None:
        h = getattr(self, "_h", None)
        if h is not None and h.value:
            self._lib.ilb_ledger_free(h)
            self._h = None

    @staticmethod
    def group_needs(layer_needs: Sequence[CacheNeeds], run_order: Optional[Sequence[RunEntry]] = None) -> List[Tuple[PagedKVNeed, List[int]]]:
        """The page groups a model gets, in group order: (need, layers of the group).  For
        callers that size every pool by itself before the manager exists."""
        needs = list(layer_needs)
        order = list(run_order) if run_order is not None else [RunEntry(i, i) for i in range(len(needs))]
        found: List[Tuple[PagedKVNeed, List[int]]] = []
        for layer in sorted({e.cache_of for e in order}):
            need = needs[layer].paged
            if need is None:
                continue
            for n, layers in found:
                if n == need:
                    layers.append(layer)
                    break
            else:
                found.append((need, [layer]))
        return found

    @property
    def stats(self) -> Dict[str, int]:
        out = (ctypes.c_longlong * 4)()
        self._lib.ilb_ledger_stats(self._h, out)
        return {"begun": out[0], "released": out[1], "window_pages_released": out[2]}

    @property
    def handle(self) -> ctypes.c_void_p:
        """The C++ ledger (for the step builder)."""
        return self._h

    def id_of(self, request: Hashable) -> int:
        """The number under which the ledger knows a live request."""
        return self._live[request]

    # ------------------------------------------------------------------ requests
    def has(self, request: Hashable) -> bool:
        return request in self._live

    def length(self, request: Hashable) -> int:
        """Tokens of `request` whose keys and values are in the cache."""
        return self._lib.ilb_ledger_length(self._h, self._live[request])

    def live_requests(self) -> List[Hashable]:
        return list(self._live)

    def begin(self, request: Hashable) -> int:
        """Register a request: takes its state slot (zeroed), no pages yet."""
        if request in self._live:
            raise ValueError(f"request {request!r} is already live")
        rid = self._ids.of(request)
        slot = self._lib.ilb_ledger_begin(self._h, rid)
        if slot < 0:
            self._ids.forget(request)
            raise_for(slot, self._ids)
        self._live[request] = rid
        for t in self._slot_state.values():
            t[slot].zero_()
        return slot

    def slot_of(self, request: Hashable) -> int:
        return self._lib.ilb_ledger_slot_of(self._h, self._live[request])

    def pages_needed(self, request: Hashable, new_length: int) -> Dict[int, int]:
        """Pages each group must still take to cover tokens [0, new_length), after the
        pages a window lets go are counted as returned."""
        out = (ctypes.c_int * max(1, len(self.groups)))()
        rc = self._lib.ilb_ledger_pages_needed(self._h, self._live[request], int(new_length), out)
        if rc < 0:
            raise_for(rc, self._ids)
        return {g.index: out[g.index] for g in self.groups}

    def ensure(self, request: Hashable, new_length: int) -> None:
        """Make room for tokens [length, new_length) in every group, or raise OutOfPages
        and change nothing but pages a window had already let go."""
        rc = self._lib.ilb_ledger_ensure(self._h, self._live[request], int(new_length))
        if rc < 0:
            raise_for(rc, self._ids)

    def commit(self, request: Hashable, new_length: int) -> None:
        """Record that tokens up to `new_length` are now in the cache."""
        rc = self._lib.ilb_ledger_commit(self._h, self._live[request], int(new_length))
        if rc < 0:
            raise_for(rc, self._ids)

    def release(self, request: Hashable) -> None:
        """The request ends (or is preempted): all its pages and its slot come back."""
        if request not in self._live:
            raise ValueError(f"request {request!r} is not live")
        rc = self._lib.ilb_ledger_release(self._h, self._live[request])
        if rc < 0:
            raise_for(rc, self._ids)
        del self._live[request]
        self._ids.forget(request)

    def released_in_ledger(self, request: Hashable) -> None:
        """The scheduler (C++) has already given back this request's pages and slot in the
        ledger; drop it from the table of live requests here too."""
        if self._live.pop(request, None) is not None:
            self._ids.forget(request)

    @property
    def ids(self) -> OwnerIds:
        """Numbers of the requests, shared with the scheduler."""
        return self._ids

    # ------------------------------------------------------------------ views
    def block_table(self, group: int, request: Hashable) -> List[int]:
        n = self._lib.ilb_ledger_table_len(self._h, int(group), self._live[request])
        if n < 0:
            raise_for(n, self._ids)
        out = (ctypes.c_int * max(1, n))()
        self._lib.ilb_ledger_table(self._h, int(group), self._live[request], out, n)
        return list(out[:n])

    def max_blocks(self, requests: Sequence[Hashable]) -> int:
        m = 1
        for g in self.groups:
            for r in requests:
                m = max(m, self._lib.ilb_ledger_table_len(self._h, g.index, self._live[r]))
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
        rc = self._lib.ilb_ledger_check(self._h)
        if rc < 0:
            raise_for(rc, self._ids)

    def inspect(self) -> dict:
        """Counterpart of the reference's KvCacheInspection
        (crates/foundation/ir/src/diagnostics.rs:80-98)."""
        return {
            "block_size": self.page_size,
            "live_requests": len(self._live),
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
