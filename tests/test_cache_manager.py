"""The cache manager's ledger (no GPU): no page lost, held twice or freed twice."""
import random

import pytest
from hypothesis import given, settings, strategies as st

from inferloop_b200.cache import CacheManager, OutOfPages, PageLedgerError, PagePool, SlotPool
from inferloop_b200.cache.slots import OutOfSlots
from inferloop_b200.config.spec import RunEntry
from inferloop_b200.parts.base import CacheNeeds, PagedKVNeed, SlotStateNeed

FULL = CacheNeeds(paged=PagedKVNeed(2, 16, None))
WIN = CacheNeeds(paged=PagedKVNeed(2, 16, 10))


def test_pool_take_and_give_back():
    pool = PagePool(4)
    a = pool.take("a", 3)
    assert len(set(a)) == 3 and pool.num_free == 1
    with pytest.raises(OutOfPages):
        pool.take("b", 2)
    assert pool.num_free == 1                      # nothing was taken
    with pytest.raises(PageLedgerError, match="belongs to"):
        pool.give_back("b", [a[0]])
    pool.give_back("a", [a[0]])
    with pytest.raises(PageLedgerError, match="freed twice"):
        pool.give_back("a", [a[0]])
    with pytest.raises(PageLedgerError, match="twice in one call"):
        pool.give_back("a", [a[1], a[1]])
    b = pool.take("b", 1)
    assert b == [a[0]] and pool.reuses == 1        # last freed, first reused
    pool.check()


def test_slots():
    s = SlotPool(2)
    assert {s.take("a"), s.take("b")} == {0, 1}
    with pytest.raises(OutOfSlots):
        s.take("c")
    with pytest.raises(ValueError):
        s.take("a")
    s.give_back("a")
    with pytest.raises(ValueError):
        s.give_back("a")
    assert s.take("c") in (0, 1)
    s.check()


def test_pages_are_taken_per_step_and_returned_at_the_end():
    m = CacheManager([FULL, FULL], page_size=4, num_pages=6, max_requests=4)
    assert len(m.groups) == 1 and m.groups[0].layers == [0, 1]
    m.begin("a")
    assert m.free_pages() == {0: 6}                # admission takes no page
    m.ensure("a", 5)
    assert m.free_pages() == {0: 4} and len(m.block_table(0, "a")) == 2
    m.commit("a", 5)
    m.ensure("a", 8)                               # still inside the second page
    assert m.free_pages() == {0: 4}
    m.commit("a", 8)
    m.begin("b")
    with pytest.raises(OutOfPages):
        m.ensure("b", 17)                          # 5 pages, 4 free: all or nothing
    assert m.free_pages() == {0: 4} and m.block_table(0, "b") == []
    m.ensure("b", 16)
    m.commit("b", 16)
    with pytest.raises(OutOfPages):
        m.ensure("a", 9)
    m.release("b")
    m.ensure("a", 9)
    m.commit("a", 9)
    m.check()
    m.release("a")
    assert m.free_pages() == {0: 6} and m.slots.num_free == 4
    with pytest.raises(ValueError):
        m.release("a")
    with pytest.raises(PageLedgerError):
        m.begin("c"); m.commit("c", 3)             # commit without pages


def test_groups_by_need_and_window_release():
    m = CacheManager([FULL, WIN, FULL, WIN], page_size=4, num_pages=8, max_requests=2)
    assert [g.layers for g in m.groups] == [[0, 2], [1, 3]]
    assert m.groups[1].need.window == 10
    m.begin("a")
    m.ensure("a", 16); m.commit("a", 16)
    assert m.free_pages() == {0: 4, 1: 4}
    # next query is position 16: oldest key it reads is 16 - 10 + 1 = 7 -> block 1; block 0 goes
    m.ensure("a", 17); m.commit("a", 17)
    assert m.block_table(1, "a")[0] == -1 and m.block_table(1, "a")[1] >= 0
    assert m.block_table(0, "a")[0] >= 0           # the full group keeps everything
    assert m.free_pages() == {0: 3, 1: 4}          # window group: +1 released, -1 taken
    for n in range(18, 33):
        m.ensure("a", n); m.commit("a", n)
        m.check()
    held = [p for p in m.block_table(1, "a") if p >= 0]
    assert len(held) <= 4                          # ceil((10 + 1) / 4) + 1
    assert m.inspect()["window_pages_released"] >= 4
    m.release("a")
    assert m.free_pages() == {0: 8, 1: 8}


def test_every_group_has_a_pool_of_its_own_size():
    """A group that reads a window can be given fewer pages than the group that keeps every
    key: a long request then fits although the small pool never holds more than the window."""
    needs = [FULL, WIN, FULL, WIN]
    assert [(n.window, layers) for n, layers in CacheManager.group_needs(needs)] == [(None, [0, 2]), (10, [1, 3])]
    m = CacheManager(needs, page_size=4, num_pages=[16, 5], max_requests=2)
    assert [g.pool.num_pages for g in m.groups] == [16, 5] and m.free_pages() == {0: 16, 1: 5}
    m.begin("a")
    for n in range(1, 61):                       # one token at a time: 15 pages of the full group in the end
        m.ensure("a", n); m.commit("a", n)
        m.check()
    assert m.free_pages()[0] == 1 and m.free_pages()[1] >= 1
    m.begin("b")
    with pytest.raises(OutOfPages):              # the full group is what runs out
        m.ensure("b", 8)
    m.release("a"); m.release("b")
    assert m.free_pages() == {0: 16, 1: 5}
    with pytest.raises(ValueError, match="pool sizes"):
        CacheManager(needs, page_size=4, num_pages=[16], max_requests=2)
    with pytest.raises(ValueError, match="at least one page"):
        CacheManager(needs, page_size=4, num_pages=[16, 0], max_requests=2)
    # a whole prompt at once needs the window's pages beside the step's own
    m = CacheManager(needs, page_size=4, num_pages=[16, 5], max_requests=2)
    m.begin("c")
    with pytest.raises(OutOfPages):
        m.ensure("c", 40)                        # 10 pages of the window group in one step


def test_borrowed_cache_allocates_nothing_and_slot_state_is_declared():
    needs = [CacheNeeds(paged=PagedKVNeed(1, 16, None)),
             CacheNeeds(paged=PagedKVNeed(4, 32, None)),
             CacheNeeds(slots=(SlotStateNeed("s", (3, 5)),))]
    order = [RunEntry(0, 0), RunEntry(1, 0, writes_cache=False), RunEntry(2, 2), RunEntry(0, 0)]
    m = CacheManager(needs, page_size=8, num_pages=4, max_requests=2, run_order=order)
    assert len(m.groups) == 1 and m.groups[0].layers == [0]   # layer 1 borrows layer 0's cache
    c = m.layer_cache(order[1])
    assert c.layer == 0 and c.group == 0 and not c.writable
    assert m.layer_cache(order[2]).group is None


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 2 ** 31), st.integers(1, 6), st.sampled_from([None, 5, 13]))
def test_random_orders_never_lose_or_duplicate_a_page(seed, page_size, window):
    rng = random.Random(seed)
    needs = [FULL, CacheNeeds(paged=PagedKVNeed(2, 16, window))]
    m = CacheManager(needs, page_size=page_size, num_pages=12, max_requests=4)
    live = {}
    counter = 0
    for _ in range(120):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            rid = f"r{counter}"; counter += 1
            m.begin(rid); live[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            new = live[rid] + rng.randint(1, 9)
            before = m.free_pages()
            try:
                m.ensure(rid, new)
                m.commit(rid, new)
                live[rid] = new
            except OutOfPages:
                after = m.free_pages()
                # nothing taken; a window may have let pages go, never the reverse
                assert all(after[g] >= before[g] for g in before)
        elif live:
            rid = rng.choice(list(live))
            m.release(rid); del live[rid]
        m.check()
        for rid, n in live.items():
            assert m.length(rid) == n
            for g in m.groups:
                table = m.block_table(g.index, rid)
                assert len(table) >= -(-n // page_size)
                # every position a future token can still read has a page
                oldest = 0 if g.need.window is None else max(0, n - g.need.window + 1)
                for pos in range(oldest, n):
                    assert table[pos // page_size] >= 0
    for rid in list(live):
        m.release(rid)
    assert all(v == 12 for v in m.free_pages().values()) and m.slots.num_free == 4
