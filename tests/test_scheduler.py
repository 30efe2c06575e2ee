"""The scheduler's decisions (no GPU), against a runner that executes nothing."""
import pytest

from fake_runner import FakeRunner
from helpers import random_tokens
from inferloop_b200.engine.engine import Engine
from inferloop_b200.engine.scheduler import CapacityError
from inferloop_b200.sampling import SamplingParams


def make(runner, **kw):
    kw.setdefault("max_num_seqs", 4)
    kw.setdefault("prefill_chunk_tokens", 8)
    kw.setdefault("max_num_batched_tokens", 12)
    return Engine(None, runner=runner, **kw)


PROMPTS = [random_tokens(n, 50, 100 + n) for n in (3, 12, 31, 20, 7, 26)]


def serial_tokens(params, max_new=10):
    out = []
    for i, p in enumerate(PROMPTS):
        e = make(FakeRunner(num_pages=64), max_num_seqs=1)
        e.submit(p, params, max_new, request_id=i)
        while not e.is_idle():
            e.step()
        out.append(e.result(i).generated)
    return out


@pytest.mark.parametrize("params", [SamplingParams(), SamplingParams(temperature=0.8, seed=3),
                                    SamplingParams(temperature=1.1, top_k=7, top_p=0.9, seed=5)])
def test_mixed_batches_give_the_tokens_of_serial_runs(params):
    want = serial_tokens(params)
    runner = FakeRunner(num_pages=64)
    e = make(runner)
    ids = [e.submit(p, params, 10, request_id=i) for i, p in enumerate(PROMPTS)]
    while not e.is_idle():
        e.step()
    assert [e.result(i).generated for i in ids] == want
    mixed = [s for s in runner.steps if any(n > 1 for _, n in s) and any(n == 1 for _, n in s)]
    assert mixed, "no step held a prompt portion beside a decode token"
    assert all(sum(n for _, n in s) <= 12 and len(s) <= 4 for s in runner.steps)
    assert all(n <= 8 for s in runner.steps for _, n in s)
    assert all(v == 64 for v in runner.cache.free_pages().values())      # nothing leaked
    assert runner.cache.slots.num_free == runner.cache.slots.num_slots


def test_first_come_first_served_and_sequence_cap():
    runner = FakeRunner(num_pages=64)
    e = make(runner, max_num_seqs=2, max_num_batched_tokens=64, prefill_chunk_tokens=64)
    for i, p in enumerate(PROMPTS[:4]):
        e.submit(p, None, 3, request_id=i)
    e.step()
    assert [r for r, _ in runner.steps[0]] == [0, 1]
    while not e.is_idle():
        e.step()
    first_seen = []
    for s in runner.steps:
        for r, _ in s:
            if r not in first_seen:
                first_seen.append(r)
    assert first_seen == [0, 1, 2, 3]
    assert all(len(s) <= 2 for s in runner.steps)


def test_pages_run_out_preempt_by_recompute_same_tokens():
    want = serial_tokens(SamplingParams(), max_new=12)
    # 9 pages of 4 tokens: the six requests cannot all be held at once
    runner = FakeRunner(num_pages=11)
    e = make(runner, max_num_seqs=4)
    ids = [e.submit(p, None, 12, request_id=i) for i, p in enumerate(PROMPTS)]
    guard = 0
    while not e.is_idle():
        e.step()
        guard += 1
        assert guard < 2000, "no progress"
    assert [e.result(i).generated for i in ids] == want
    assert e.scheduler.stats["preemptions"] > 0
    assert any(e.result(i).preemptions > 0 for i in ids)
    assert all(v == 11 for v in runner.cache.free_pages().values())
    assert runner.cache.groups[0].pool.reuses > 0


def test_window_group_lets_long_requests_through():
    runner = FakeRunner(num_pages=40, window=6)
    e = make(runner)
    ids = [e.submit(p, None, 8, request_id=i) for i, p in enumerate(PROMPTS[:3])]
    while not e.is_idle():
        e.step()
    assert runner.cache.inspect()["window_pages_released"] > 0
    assert all(v == 40 for v in runner.cache.free_pages().values())


def test_a_request_too_large_for_the_cache_is_refused():
    e = make(FakeRunner(num_pages=4))
    with pytest.raises(CapacityError):
        e.submit(random_tokens(30, 50, 1), None, 4)
    with pytest.raises(ValueError, match="max_model_len"):
        make(FakeRunner(max_positions=32)).submit(random_tokens(30, 50, 1), None, 4)
    with pytest.raises(ValueError, match="vocabulary"):
        make(FakeRunner()).submit([1, 2, 99], None, 4)
    with pytest.raises(ValueError, match="empty"):
        make(FakeRunner()).submit([], None, 4)
    dup = make(FakeRunner())
    dup.submit([1], None, 2, request_id="x")
    with pytest.raises(ValueError):
        dup.submit([2], None, 2, request_id="x")


def test_eos_and_length_finish():
    runner = FakeRunner(num_pages=64)
    e = make(runner)
    p = PROMPTS[1]
    e.submit(p, None, 6, request_id=0)
    while not e.is_idle():
        e.step()
    free_run = e.result(0).generated
    assert len(free_run) == 6 and e.result(0).finish_reason == "length"
    e2 = make(FakeRunner(num_pages=64))
    e2.submit(p, SamplingParams(eos_token=free_run[2]), 6, request_id=0)
    while not e2.is_idle():
        e2.step()
    stop = free_run.index(free_run[2])
    assert e2.result(0).generated == free_run[:stop + 1] and e2.result(0).finish_reason == "eos"
    e3 = make(FakeRunner(num_pages=64), max_output_tokens=2)
    e3.submit(p, None, 6, request_id=0)
    while not e3.is_idle():
        e3.step()
    assert e3.result(0).generated == free_run[:2]


def test_half_portion_rule():
    # 3 decoding requests leave 5 of 8 budget tokens: a portion of 8 gets the 5 (>= half)
    runner = FakeRunner(num_pages=64)
    e = make(runner, max_num_batched_tokens=11, prefill_chunk_tokens=8)   # floor: 8 + 4 - 1
    for i in range(3):
        e.submit([1, 2], None, 20, request_id=i)
    e.step()
    e.submit(random_tokens(30, 50, 9), None, 2, request_id="late")
    e.step()
    last = dict(runner.steps[-1])
    assert last["late"] == 8 and all(last[i] == 1 for i in range(3))
    e2 = make(FakeRunner(num_pages=64), max_num_batched_tokens=11, prefill_chunk_tokens=8, max_num_seqs=4)
    e2.scheduler.config.max_num_batched_tokens = 6       # decodes take 3, 3 left < half of 8
    for i in range(3):
        e2.submit([1, 2], None, 20, request_id=i)
    e2.step()
    e2.submit(random_tokens(30, 50, 9), None, 2, request_id="late")
    e2.step()
    assert "late" not in dict(e2.runner.steps[-1])
    e2.scheduler.config.max_num_batched_tokens = 7       # 4 left >= half of 8
    e2.step()
    assert dict(e2.runner.steps[-1])["late"] == 4


def test_finished_requests_are_handed_over_and_forgotten():
    """`take_completed` drains results; without it the engine keeps at most
    `max_finished_kept` finished requests, the newest ones."""
    e = make(FakeRunner(num_pages=64))
    ids = [e.submit(p, SamplingParams(), 3) for p in PROMPTS[:3]]
    while not e.is_idle():
        e.step()
    done = e.take_completed()
    assert sorted(r.id for r in done) == sorted(ids) and all(len(r.generated) == 3 for r in done)
    assert e.take_completed() == [] and not e.requests and not e.scheduler.finished
    e.max_finished_kept = 2
    for k in range(5):
        e.submit(PROMPTS[k], SamplingParams(), 2, request_id=f"k{k}")
        while not e.is_idle():
            e.step()
    assert len(e.scheduler.finished) <= 3 and "k4" in e.requests and "k0" not in e.requests
    assert e.result("k4").generated and e.inspect()["finished"] <= 3


def test_a_whole_portion_beside_decodes_is_trimmed_to_the_token_tile():
    """With `step_token_multiple` m, a step that holds decode tokens and a whole portion has a
    multiple of m tokens (the matrix kernels' tile), as long as half a portion stays; a
    prompt's tail and a portion alone in its step are left as they are; tokens do not change."""
    prompts = [random_tokens(n, 50, 700 + n) for n in (5, 6, 7, 100, 45)]

    def run(multiple):
        runner = FakeRunner(num_pages=128)
        e = make(runner, max_num_seqs=5, prefill_chunk_tokens=32, max_num_batched_tokens=40)
        e.scheduler.config.step_token_multiple = multiple
        ids = [e.submit(p, SamplingParams(), 12, request_id=i) for i, p in enumerate(prompts)]
        while not e.is_idle():
            e.step()
        return [e.result(i).generated for i in ids], runner.steps

    plain_tokens, plain_steps = run(1)
    tokens, steps = run(16)
    assert tokens == plain_tokens
    assert any(sum(n for _, n in s) == 35 for s in plain_steps)              # three decodes + a portion of 32
    sizes = [[n for _, n in s] for s in steps]
    assert [1, 1, 1, 32] in [[n for _, n in s] for s in plain_steps] and [1, 1, 1, 32] not in sizes
    assert sizes.count([1, 1, 1, 29]) == 2                                    # 3 + 29 = 32 tokens: two tiles of 16
    # the prompt's tail (20 tokens) is not trimmed, and the newcomer beside it gets what the
    # budget leaves (17 of its 32: more than half), not the 9 that would reach the tile's edge
    assert [1, 1, 1, 20, 17] in sizes
    e = make(FakeRunner(num_pages=128), max_num_seqs=2, prefill_chunk_tokens=32, max_num_batched_tokens=40)
    e.scheduler.config.step_token_multiple = 16
    e.submit(random_tokens(70, 50, 1), SamplingParams(), 2)
    e.step()
    assert e.runner.steps[0] == [(0, 32)]                                     # alone in its step: whole


# ------------------------------------------------------------------ random workloads
from hypothesis import HealthCheck, given, settings, strategies as st


@settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(st.data())
def test_random_workloads_keep_the_invariants(data):
    """Requests of random lengths arrive before and between steps, some are aborted, the pool
    is anywhere from one request's need to plenty, budgets and the token tile vary.  Whatever
    the schedule: every step fits its budgets and the pages (the runner asserts that), every
    request that is not aborted gets exactly the tokens of a run alone, stops at its stop
    token or its length, and every page and slot is back at the end."""
    draw = data.draw
    page = draw(st.sampled_from([2, 4, 8]))
    window = draw(st.sampled_from([None, None, 6, 16]))
    chunk = draw(st.sampled_from([2, 5, 8, 16]))
    max_seqs = draw(st.integers(1, 5))
    budget = chunk + draw(st.integers(0, 6))
    multiple = draw(st.sampled_from([1, 1, 4]))
    n_req = draw(st.integers(1, 9))
    lens = [draw(st.integers(1, 40)) for _ in range(n_req)]
    news = [draw(st.integers(1, 12)) for _ in range(n_req)]
    stop = tuple(draw(st.lists(st.integers(0, 49), max_size=6, unique=True)))
    arrive = [draw(st.integers(0, 6)) for _ in range(n_req)]          # the step before which a request is submitted
    abort_at = {i: draw(st.integers(1, 10)) for i in range(n_req) if draw(st.integers(0, 5)) == 0}
    longest = max(l + n for l, n in zip(lens, news))
    pages = -(-longest // page) + 1 + draw(st.sampled_from([0, 1, 3, 20, 200]))
    params = SamplingParams(eos_tokens=stop) if draw(st.booleans()) else SamplingParams(temperature=0.9, seed=7, eos_tokens=stop)
    prompts = [random_tokens(l, 50, 900 + 13 * i + l) for i, l in enumerate(lens)]

    def alone(i):
        e = make(FakeRunner(num_pages=400, page_size=page, window=window), max_num_seqs=1, prefill_chunk_tokens=chunk,
                 max_num_batched_tokens=chunk + 1)
        e.submit(prompts[i], params, news[i], request_id=i)
        while not e.is_idle():
            e.step()
        return e.result(i).generated

    runner = FakeRunner(num_pages=pages, page_size=page, window=window, max_requests=8)
    e = make(runner, max_num_seqs=max_seqs, prefill_chunk_tokens=chunk, max_num_batched_tokens=budget)
    e.scheduler.config.step_token_multiple = multiple
    submitted, aborted, step = set(), set(), 0
    while len(submitted) < n_req or not e.is_idle():
        for i in range(n_req):
            if i not in submitted and arrive[i] <= step:
                e.submit(prompts[i], params, news[i], request_id=i)
                submitted.add(i)
        for i, when in abort_at.items():
            if i in submitted and i not in aborted and when == step:
                e.abort(i)
                aborted.add(i)
        e.step()
        step += 1
        assert step < 2000, "the schedule does not end"
    budget = e.scheduler.config.max_num_batched_tokens       # (raised to a portion beside every other sequence's token, if below)
    for s in runner.steps:
        assert sum(n for _, n in s) <= budget and len(s) <= max_seqs and all(n <= chunk for _, n in s)
    for i in range(n_req):
        got = e.result(i).generated
        if i in aborted:
            want = alone(i)
            assert got == want[:len(got)]
            continue
        assert got == alone(i)
        hits = [k for k, t in enumerate(got) if t in stop]
        assert (hits and hits[0] == len(got) - 1) or (not hits and len(got) == news[i])
    assert all(v == pages for v in runner.cache.free_pages().values())
    assert runner.cache.slots.num_free == runner.cache.slots.num_slots
