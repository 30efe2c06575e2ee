"""The engine against the plain implementation, in every way of cutting the work, in
32-bit and in bfloat16 (GPU).  All cases go through ModelRunner.step, the step function
that generation uses; two of them go through the bin/trace_run program itself."""
import json
import os
import random

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import (BF16_REL_OF_MAX, CONFIGS, Trace, assert_close, check_trace, make_model_folder,
                     random_tokens, run_trace_inprocess, run_trace_program)

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [1, 7, 16, 33, 90, 120], "B": [3, 12, 31, 64, 100, 150], "C": [5, 40, 77, 130, 200, 64],
           "D": [5, 64, 130, 300, 520, 33], "E": [5, 64, 130, 300, 520, 33], "F": [5, 64, 130, 300, 520, 33]}
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (cfg, seed, _) in CONFIGS.items():
        out[name] = make_model_folder(str(tmp_path_factory.mktemp("model") / name), cfg, seed)
    return out


@pytest.fixture(scope="module")
def requests_of():
    return {name: {f"r{i}": random_tokens(n, CONFIGS[name][0]["vocab_size"], 1000 + 17 * i + n)
                   for i, n in enumerate(lens)} for name, lens in LENGTHS.items()}


_REF = {}


def reference(folders, requests_of, name, dtype):
    """Plain logits [len, vocab] of every request, whole, computed once."""
    key = (name, dtype)
    if key not in _REF:
        model = plain.PlainModel(folders[name], round_to_bf16=(dtype == "bfloat16"))
        _REF[key] = {rid: model.logits(toks) for rid, toks in requests_of[name].items()}
    return _REF[key]


_RUNNERS = {}


def runner_for(folders, name, dtype, num_pages=256):
    from inferloop_b200.engine import ModelRunner
    key = (name, dtype, num_pages)
    if key not in _RUNNERS:
        _RUNNERS[key] = ModelRunner.from_folder(folders[name], dtype=dtype, page_size=CONFIGS[name][2],
                                                num_pages=num_pages, max_requests=8)
    r = _RUNNERS[key]
    for rid in r.cache.live_requests():
        r.end(rid)
    return r


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_each_request_alone_and_whole(folders, requests_of, name, dtype):
    trace = Trace()
    for rid, toks in requests_of[name].items():
        trace.step([(rid, toks, list(range(len(toks))))], end=[rid])
    r = runner_for(folders, name, dtype)
    check_trace(run_trace_inprocess(r, trace), trace, reference(folders, requests_of, name, dtype), dtype, f"{name} whole")
    r.cache.check()
    assert all(v == 256 for v in r.cache.free_pages().values())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_most_in_one_step_then_the_last_32_one_by_one(folders, requests_of, name, dtype):
    trace = Trace()
    for rid, toks in requests_of[name].items():
        head = max(1, len(toks) - 32)
        trace.step([(rid, toks[:head], [head - 1])])
        for i in range(head, len(toks)):
            trace.step([(rid, [toks[i]], [0])], end=[rid] if i == len(toks) - 1 else [])
        if head == len(toks):
            trace.step([], end=[rid])
    r = runner_for(folders, name, dtype)
    check_trace(run_trace_inprocess(r, trace), trace, reference(folders, requests_of, name, dtype), dtype, f"{name} decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_portions_of_changing_size(folders, requests_of, name, dtype):
    sizes = [7, 2, 13, 3, 2, 21, 5, 2, 9, 1, 17]
    trace = Trace()
    for k, (rid, toks) in enumerate(requests_of[name].items()):
        i, j = 0, k
        while i < len(toks):
            n = min(sizes[j % len(sizes)], len(toks) - i)
            trace.step([(rid, toks[i:i + n], list(range(n)))], end=[rid] if i + n == len(toks) else [])
            i += n
            j += 1
    r = runner_for(folders, name, dtype)
    check_trace(run_trace_inprocess(r, trace), trace, reference(folders, requests_of, name, dtype), dtype, f"{name} portions")


def mixed_trace(reqs, seed=0, tail=12, sizes=(2, 3, 5, 8, 13, 17, 29), live_max=4):
    """Up to four live requests; each step holds portions of some beside single decoded
    tokens of others, some requests sit a step out; a finished request's place is taken
    by the next one.  Returns the trace and the most tokens held at any time (each
    request rounded up to 64)."""
    rng = random.Random(seed)
    sizes = list(sizes)
    # every request runs twice, so late arrivals land on pages others have given back
    queue = [(f"{rid}.{rep}", rid) for rep in range(2) for rid in reqs]
    rng.shuffle(queue)
    live, cursor = [], {}
    trace, peak = Trace(), 0
    alias = {}
    while queue or live:
        while queue and len(live) < live_max:
            tid, rid = queue.pop()
            live.append(tid); cursor[tid] = 0; alias[tid] = rid
        entries, ended = [], []
        for tid in list(live):
            toks = reqs[alias[tid]]
            if len(live) > 1 and rng.random() < 0.25:
                continue                                       # sits this step out
            left = len(toks) - cursor[tid]
            n = 1 if left <= tail else min(left - tail, rng.choice(sizes))
            want = list(range(n)) if rng.random() < 0.7 else [n - 1]
            entries.append((tid, toks[cursor[tid]:cursor[tid] + n], want))
            cursor[tid] += n
            if cursor[tid] == len(toks):
                ended.append(tid)
        held = sum(-(-cursor[t] // 64) * 64 for t in live)
        peak = max(peak, held)
        if entries:
            trace.step(entries, end=ended)
        for tid in ended:
            live.remove(tid)
    return trace, peak, alias


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_mixed_batches_on_few_pages(folders, requests_of, name, dtype):
    from inferloop_b200.engine import ModelRunner
    reqs = requests_of[name]
    trace, peak, alias = mixed_trace(reqs, seed=len(name) + ord(name))
    page = CONFIGS[name][2]
    r = ModelRunner.from_folder(folders[name], dtype=dtype, page_size=page, num_pages=peak // page, max_requests=8)
    out = run_trace_inprocess(r, trace)
    ref = reference(folders, requests_of, name, dtype)
    check_trace(out, trace, {tid: ref[rid] for tid, rid in alias.items()}, dtype, f"{name} mixed")
    info = r.cache.inspect()
    assert all(g["reuses"] > 0 for g in info["groups"]), "the pool was large enough that no page was used again"
    assert all(g["free"] == g["total"] for g in info["groups"])
    assert any(len(s["entries"]) >= 3 and any(len(e["tokens"]) > 1 for e in s["entries"])
               and any(len(e["tokens"]) == 1 for e in s["entries"]) for s in trace.steps)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", [("C", 0), ("D", 1), ("E", 2), ("F", 3), ("D", 4), ("F", 5)])
def test_random_mixed_traces(folders, requests_of, name, seed, dtype):
    """Schedules drawn at random beyond the fixed ones above: portions up to 260 tokens (the
    many-token kernels beside single tokens), up to six live requests, decoding tails from none
    to 33 tokens, pages two and four times the configuration's, pools with and without slack.
    (Thousands of such traces were run once while the kernels were written; these stay.)"""
    from inferloop_b200.engine import ModelRunner
    rng = random.Random(77 * seed + 5)
    sizes = rng.choice([[1, 2, 40, 70, 150], [16, 32, 64, 128, 129, 200], [3, 97, 260], [2, 3, 5, 8, 13, 17, 29]])
    tail, live_max = rng.choice([0, 1, 12, 33]), rng.choice([2, 4, 6])
    page = min(128, CONFIGS[name][2] * rng.choice([1, 2, 4]))
    reqs = requests_of[name]
    trace, peak, alias = mixed_trace(reqs, seed=seed, tail=tail, sizes=sizes, live_max=live_max)
    pages = -(-(peak + 64 * live_max) // page) if page > 64 else (peak + rng.choice([0, 64])) // page
    r = ModelRunner.from_folder(folders[name], dtype=dtype, page_size=page, num_pages=pages, max_requests=8)
    out = run_trace_inprocess(r, trace)
    ref = reference(folders, requests_of, name, dtype)
    check_trace(out, trace, {tid: ref[rid] for tid, rid in alias.items()}, dtype, f"{name} random trace {seed}")
    assert all(g["free"] == g["total"] for g in r.cache.inspect()["groups"])


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_trace_program_itself(folders, requests_of, dtype, tmp_path):
    """bin/trace_run as a separate process, on a mixed trace with few pages."""
    name = "B"
    reqs = requests_of[name]
    trace, peak, alias = mixed_trace(reqs, seed=99)
    out = run_trace_program(folders[name], dtype, trace, str(tmp_path / "out"), max_tokens=peak,
                            block_size=CONFIGS[name][2])
    ref = reference(folders, requests_of, name, dtype)
    check_trace(out, trace, {tid: ref[rid] for tid, rid in alias.items()}, dtype, "trace_run")
    written = sorted(int(f[:-4]) for f in os.listdir(tmp_path / "out"))
    assert written == sorted(trace.rows)           # a file exactly where something was wanted


def test_the_trace_program_says_what_is_wrong_with_a_step(folders, tmp_path):
    """A line that is no step, and a step that the step function refuses (a token outside the
    vocabulary), end the program with status 2 and one line that names the place; the steps
    before them were run and reported."""
    import subprocess
    import sys
    from helpers import ROOT
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders["A"], "--dtype", "float32",
           "--out", str(tmp_path / "out"), "--max-tokens", "128", "--block-size", str(CONFIGS["A"][2])]
    good = '{"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [2]}], "end": []}\n'
    for bad, needle in (('{"step": 1, "entries": [{"id": "a", "tokens": "x"}]}\n', "line 2 is not a step"),
                        ('not json\n', "line 2 is not a step"),
                        ('{"step": 1, "entries": [{"id": "a", "tokens": [999999], "want": [0]}], "end": []}\n', "step 1:")):
        proc = subprocess.run(cmd, input=good + bad, capture_output=True, text=True, timeout=600)
        assert proc.returncode == 2, (proc.returncode, proc.stderr)
        assert proc.stdout.splitlines() == ["done 0"]
        assert needle in proc.stderr and "Traceback" not in proc.stderr, proc.stderr


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(folders, dtype, tmp_path):
    """A short prompt, then 700 tokens one by one: every page edge is crossed many times."""
    cfg = dict(CONFIGS["A"][0], max_position_embeddings=1024)
    d = make_model_folder(str(tmp_path / "long"), cfg, 3)
    toks = random_tokens(740, cfg["vocab_size"], 5)
    ref = plain.PlainModel(d, round_to_bf16=(dtype == "bfloat16")).logits(toks)
    from inferloop_b200.engine import ModelRunner, StepEntry
    r = ModelRunner.from_folder(d, dtype=dtype, page_size=4, num_pages=190, max_requests=2)
    got = [r.step([StepEntry("x", toks[:40], list(range(40)))]).float().cpu().clone()]
    for i in range(40, len(toks)):
        got.append(r.step([StepEntry("x", [toks[i]], [0])]).float().cpu().clone())
    assert_close(torch.cat(got), ref, dtype, "long decoding")


def test_decoding_across_the_long_context_mark(folders, monkeypatch):
    """A sequence that grows past ops.DECODE_LONG_CONTEXT (lowered here) gets a second recorded
    graph whose attention launch is shaped for long sequences (narrower clusters, several per
    sequence and kv head when it is long enough); the logits stay those of the plain model on
    both sides of the mark, and a second request beside it changes nothing."""
    from inferloop_b200.csrc import ops
    from inferloop_b200.engine import ModelRunner, StepEntry
    monkeypatch.setattr(ops, "DECODE_LONG_CONTEXT", 600)
    cfg = CONFIGS["D"][0]
    toks = random_tokens(1400, cfg["vocab_size"], 77)
    other = random_tokens(40, cfg["vocab_size"], 78)
    ref = plain.PlainModel(folders["D"], round_to_bf16=True).logits(toks)
    r = ModelRunner.from_folder(folders["D"], dtype="bfloat16", page_size=16, num_pages=120, max_requests=2)
    got = [r.step([StepEntry("x", toks[:560], [559])]).float().cpu().clone()]
    keys_before = set(r.graphs._recorded)
    for i in range(560, 640):
        got.append(r.step([StepEntry("x", [toks[i]], [0])]).float().cpu().clone())
    assert {k[2] for k in r.graphs._recorded} == {False, True} and len(r.graphs._recorded) == len(keys_before) + 2
    got.append(r.step([StepEntry("x", toks[640:1300], [659])]).float().cpu().clone())
    r.step([StepEntry("y", other, [])])
    for i in range(1300, 1400):               # 41 tiles and more: two clusters share each kv head
        out = r.step([StepEntry("x", [toks[i]], [0]), StepEntry("y", [other[i % 40]], [0])])
        got.append(out[:1].float().cpu().clone())
    rows = [559] + list(range(560, 640)) + [1299] + list(range(1300, 1400))
    assert_close(torch.cat(got), ref[rows], "bfloat16", "across the long-context mark")
    ops.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_the_first_tokens_of_a_sequence(folders, requests_of, name, dtype):
    """Position 0 alone, then 1, then 2: the smallest caches there are."""
    toks = requests_of[name]["r3"]
    ref = reference(folders, requests_of, name, dtype)["r3"]
    trace = Trace()
    for i in range(6):
        trace.step([("r3", [toks[i]], [0])])
    trace.step([("r3", toks[6:8], [0, 1])], end=["r3"])
    r = runner_for(folders, name, dtype)
    check_trace(run_trace_inprocess(r, trace), trace, {"r3": ref}, dtype, f"{name} first tokens")


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_float32_logits_do_not_depend_on_the_cut_at_all(folders, requests_of, name):
    """On the 32-bit path the order of every sum is fixed per position, so two ways of
    cutting give the same bits."""
    toks = requests_of[name]["r4"]
    r = runner_for(folders, name, "float32")
    from inferloop_b200.engine import StepEntry
    whole = r.step([StepEntry("w", toks, list(range(len(toks))))]).cpu().clone()
    r.end("w")
    parts, i = [], 0
    other = requests_of[name]["r2"]
    for n in [5, 2, 30, 1, 1, 9, len(toks)]:          # the last portion takes what is left
        n = min(n, len(toks) - i)
        if n <= 0:
            break
        entries = [StepEntry("p", toks[i:i + n], list(range(n)))]
        if i == 0:
            entries.insert(0, StepEntry("other", other, []))      # company in the batch
        parts.append(r.step(entries).cpu().clone())
        i += n
    assert torch.equal(torch.cat(parts), whole)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    from inferloop_b200 import Engine, SamplingParams
    cfg, _, page = CONFIGS[name]
    lens = [1, 7, 16, 33] if name == "A" else [3, 12, 31, 64, 100, 150]
    new = 16 if name == "A" else 24
    prompts = [random_tokens(n, cfg["vocab_size"], 50 + n) for n in lens]
    engine = Engine(folders[name], dtype=dtype, block_size=page, num_gpu_blocks_override=96,
                    max_num_seqs=4, prefill_chunk_tokens=32, max_num_batched_tokens=40)
    got = engine.generate(prompts, SamplingParams(), max_new_tokens=new)
    model = plain.PlainModel(folders[name], round_to_bf16=(dtype == "bfloat16"))
    for p, g in zip(prompts, got):
        assert len(g) == new
        if dtype == "float32":
            assert g == plain.generate(model, p, new), "greedy tokens differ from the plain implementation"
        else:
            # teacher-forced: every token the engine chose is within the bfloat16 bound of the best
            ref = model.logits(p + g)[len(p) - 1:-1]
            bound = BF16_REL_OF_MAX * float(ref.abs().max())
            for i, t in enumerate(g):
                assert ref[i, t] >= ref[i].max() - 2 * bound
    info = engine.inspect()
    assert info["running"] == 0 and all(g["free"] == g["total"] for g in info["cache"]["groups"])
    assert info["scheduler"]["steps"] < sum(lens) // 8 + new * 3      # it batched, it did not serialise


def test_temperature_generation_matches_the_plain_sampler(folders):
    """Tiny B's workload: portions of 32 mixed with decode steps, 24 tokens at T = 0.8
    with a fixed seed; in 32-bit the trajectory equals the plain implementation's."""
    from inferloop_b200 import Engine, SamplingParams
    cfg, _, page = CONFIGS["B"]
    prompts = [random_tokens(n, cfg["vocab_size"], 70 + n) for n in (3, 12, 31, 64)]
    engine = Engine(folders["B"], dtype="float32", block_size=page, num_gpu_blocks_override=64,
                    max_num_seqs=4, prefill_chunk_tokens=32)
    params = SamplingParams(temperature=0.8, seed=1234)
    got = engine.generate(prompts, params, max_new_tokens=24)
    model = plain.PlainModel(folders["B"])
    for rid, (p, g) in enumerate(zip(prompts, got)):
        assert g == plain.generate(model, p, 24, temperature=0.8, seed=1234, request=rid)
    # filters are applied by the device kernel too (penalties alone go through the host sampler)
    engine2 = Engine(folders["B"], dtype="float32", block_size=page, num_gpu_blocks_override=64, max_num_seqs=4)
    g2 = engine2.generate(prompts[:2], SamplingParams(temperature=0.9, top_k=5, top_p=0.9, seed=7), 8)
    for rid, (p, g) in enumerate(zip(prompts[:2], g2)):
        seq = list(p)
        for n, t in enumerate(g):
            want = plain.sample(model.logits(seq)[-1].float().tolist(), 0.9, 7, rid, n, top_k=5, top_p=0.9)
            assert t == want
            seq.append(t)


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("D", "bfloat16")])
def test_steps_launched_ahead_give_the_same_tokens(folders, name, dtype):
    """The engine launches the next decode step before it has read the ids of the running
    one.  With stop tokens some requests end while their row of the next step is already
    being computed: that row is dropped, everybody else's tokens are what they are without
    the lookahead, and every page comes back."""
    from inferloop_b200 import Engine, SamplingParams
    cfg, _, page = CONFIGS[name]
    prompts = [random_tokens(n, cfg["vocab_size"], 300 + n) for n in (9, 40, 17, 33)]

    def run(lookahead, params, new=24):
        e = Engine(folders[name], dtype=dtype, block_size=page, num_gpu_blocks_override=96, max_num_seqs=4,
                   prefill_chunk_tokens=64)
        e.lookahead = lookahead
        out = e.generate(prompts, params, max_new_tokens=new)
        info = e.inspect()
        assert info["running"] == 0 and all(g["free"] == g["total"] for g in info["cache"]["groups"])
        return out, info

    free_run, _ = run(False, SamplingParams())
    # stop tokens taken from the middle of two of the free-running answers
    stops = (free_run[0][7], free_run[2][13])
    params = SamplingParams(eos_tokens=stops)
    want, info_off = run(False, params)
    got, info_on = run(True, params)
    assert got == want
    assert len(got[0]) <= 8 and len(got[2]) <= 14, "the requests whose own tokens are the stop tokens end there"
    assert info_off["steps_launched_ahead"] == 0 and info_on["steps_launched_ahead"] > 5
    if dtype == "float32":
        model = plain.PlainModel(folders[name])
        for p, g in zip(prompts, got):
            ref = plain.generate(model, p, 24)
            cut = next((i + 1 for i, t in enumerate(ref) if t in stops), 24)
            assert g == ref[:cut]


def test_page_pressure_in_the_engine_gives_the_same_tokens(folders):
    """So few pages that requests are preempted and recomputed: tokens do not change."""
    from inferloop_b200 import Engine, SamplingParams
    cfg, _, page = CONFIGS["B"]
    prompts = [random_tokens(n, cfg["vocab_size"], 90 + n) for n in (31, 64, 40, 12, 55)]
    roomy = Engine(folders["B"], dtype="float32", block_size=page, num_gpu_blocks_override=128, max_num_seqs=4,
                   prefill_chunk_tokens=32)
    want = roomy.generate(prompts, SamplingParams(), 20)
    tight = Engine(folders["B"], dtype="float32", block_size=page, num_gpu_blocks_override=21, max_num_seqs=4,
                   prefill_chunk_tokens=32)
    got = tight.generate(prompts, SamplingParams(), 20)
    assert got == want
    assert tight.inspect()["scheduler"]["preemptions"] > 0


def test_refusals(folders, tmp_path):
    from inferloop_b200.engine import ModelRunner, StepEntry
    from inferloop_b200.cache import OutOfPages
    with pytest.raises(RuntimeError, match="CUDA device only"):
        ModelRunner.from_folder(folders["A"], device="cpu")
    r = ModelRunner.from_folder(folders["A"], dtype="float32", page_size=4, num_pages=4, max_requests=2)
    with pytest.raises(OutOfPages):
        r.step([StepEntry("a", list(range(17)), [])])
    assert not r.is_live("a") and r.cache.free_pages() == {0: 4}
    with pytest.raises(ValueError, match="vocabulary"):
        r.step([StepEntry("a", [999], [])])
    with pytest.raises(ValueError, match="twice"):
        r.step([StepEntry("a", [1], []), StepEntry("a", [2], [])])
    with pytest.raises(ValueError, match="outside its"):
        r.step([StepEntry("a", [1], [1])])
