"""Schedules that only a busy engine reaches, against the plain implementation (GPU): decode
batches of 20 to 64 requests (the recorded-graph sizes 24, 48 and 64, with and without
padding rows), page pressure together with replayed graphs and steps launched ahead, the
back-to-back decode driver, the default sizing of the cache, and a request aborted while a
step is on the device."""
import pytest
import torch

import plain_qwen3 as plain
from helpers import BF16_REL_OF_MAX, CONFIGS, assert_close, make_model_folder, random_tokens

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: make_model_folder(str(tmp_path_factory.mktemp("model") / name), CONFIGS[name][0], CONFIGS[name][1])
            for name in ("B", "D", "E", "F")}


_PLAIN = {}


def plain_model(folders, name, dtype):
    key = (name, dtype)
    if key not in _PLAIN:
        _PLAIN[key] = plain.PlainModel(folders[name], round_to_bf16=(dtype == "bfloat16"))
    return _PLAIN[key]


def within_bound_of_the_best(model, prompt, generated, dtype):
    """Teacher-forced check of greedy tokens: in 32-bit every token is the plain model's
    arg-max; in bfloat16 every token's plain logit is within twice the engine bound of the
    best one (two roundings of neighbours may swap them, nothing more)."""
    ref = model.logits(list(prompt) + list(generated))[len(prompt) - 1:-1]
    if dtype == "float32":
        assert list(generated) == [int(r.argmax()) for r in ref]
        return
    bound = BF16_REL_OF_MAX * float(ref.abs().max())
    for i, t in enumerate(generated):
        assert ref[i, t] >= ref[i].max() - 2 * bound, (i, t, float(ref[i, t]), float(ref[i].max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_live", [20, 24, 41, 64])
def test_many_requests_decoding_together(folders, n_live, dtype):
    """`n_live` requests with prompts of unequal length decode side by side for 40 steps;
    every step's logits of every request against the plain model.  20 and 41 requests run in
    launch shapes made for 24 and 48 (padding rows), 24 and 64 fill theirs."""
    from inferloop_b200.engine import ModelRunner, StepEntry
    cfg, _, page = CONFIGS["D"]
    steps = 40
    seqs = {f"q{i}": random_tokens(3 + (i * 7) % 90 + steps, cfg["vocab_size"], 4000 + i) for i in range(n_live)}
    model = plain_model(folders, "D", dtype)
    ref = {rid: model.logits(toks) for rid, toks in seqs.items()}
    pages = sum(-(-len(t) // page) for t in seqs.values()) + 4
    r = ModelRunner.from_folder(folders["D"], dtype=dtype, page_size=page, num_pages=pages, max_requests=64)
    ids = list(seqs)
    for k in range(0, n_live, 7):                                   # prompts, seven requests a step
        part = ids[k:k + 7]
        out = r.step([StepEntry(rid, seqs[rid][:len(seqs[rid]) - steps], [len(seqs[rid]) - steps - 1]) for rid in part])
        assert_close(out, torch.stack([ref[rid][len(seqs[rid]) - steps - 1] for rid in part]), dtype, "prompts")
    for s in range(steps):
        entries = [StepEntry(rid, [seqs[rid][len(seqs[rid]) - steps + s]], [0]) for rid in ids]
        out = r.step(entries)
        assert_close(out, torch.stack([ref[rid][len(seqs[rid]) - steps + s] for rid in ids]), dtype,
                     f"decode step {s} of {n_live} requests")
    if r.graphs is not None:
        from inferloop_b200.engine.graphs import bucket_for
        assert r.graphs.replays >= steps - 1 and any(k[0] == bucket_for(n_live) for k in r.graphs._recorded)
    from inferloop_b200.csrc import ops
    ops.check_device_errors()
    for rid in ids:
        r.end(rid)
    r.cache.check()


@pytest.mark.parametrize("name,dtype", [("D", "bfloat16"), ("F", "bfloat16"), ("D", "float32")])
def test_page_pressure_with_graphs_and_steps_launched_ahead(folders, name, dtype):
    """So few pages that decoding requests are preempted and recomputed, with recorded decode
    graphs, steps launched ahead and the decode attention that writes the cache itself all
    active.  In 32-bit the tokens equal the roomy run's; in bfloat16 (where a recomputed
    prompt is rounded otherwise than the decode steps it replaces) every token is checked
    against the plain model."""
    from inferloop_b200 import Engine, SamplingParams
    cfg, _, page = CONFIGS[name]
    prompts = [random_tokens(n, cfg["vocab_size"], 700 + n) for n in (70, 33, 120, 18, 95, 51)]
    new = 60

    def run(pages):
        e = Engine(folders[name], dtype=dtype, block_size=page, num_gpu_blocks_override=pages, max_num_seqs=4,
                   prefill_chunk_tokens=64)
        out = e.generate(prompts, SamplingParams(), new)
        info = e.inspect()
        assert info["running"] == 0 and all(g["free"] == g["total"] for g in info["cache"]["groups"])
        e.runner.cache.check()
        return out, info

    roomy, info_roomy = run(256)
    tight, info_tight = run(30)                    # four requests of up to 180 tokens want 41 pages
    assert info_roomy["scheduler"]["preemptions"] == 0 and info_tight["scheduler"]["preemptions"] > 0
    assert info_tight["steps_launched_ahead"] > 5
    model = plain_model(folders, name, dtype)
    for p, g in zip(prompts, tight):
        assert len(g) == new
        within_bound_of_the_best(model, p, g, dtype)
    if dtype == "float32":
        assert tight == roomy


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_back_to_back_decoding_gives_the_tokens_of_generation(folders, dtype):
    """`DecodeGraphs.run_greedy` (many decode steps with no host round trip, the driver the
    throughput measurement times) against `Engine.generate` and the plain model."""
    from inferloop_b200 import Engine, SamplingParams
    from inferloop_b200.engine import StepEntry
    cfg, _, page = CONFIGS["D"]
    prompts = [random_tokens(n, cfg["vocab_size"], 900 + n) for n in (40, 7, 130, 64, 22)]
    new = 48
    e = Engine(folders["D"], dtype=dtype, block_size=page, num_gpu_blocks_override=128, max_num_seqs=8,
               prefill_chunk_tokens=256)
    generated = e.generate(prompts, SamplingParams(), new)
    r = e.runner
    if r.graphs is None:
        pytest.skip("decode graphs are off for this model")
    first = []
    for i, p in enumerate(prompts):
        _, drawn = r.step([StepEntry(f"g{i}", p, [len(p) - 1])], draw_greedy=True)
        first.append(int(drawn.ids[0].item()))
    out = r.graphs.run_greedy([StepEntry(f"g{i}", [first[i]], [0]) for i in range(len(prompts))], new - 1)
    got = [[first[i]] + out[:, i].tolist() for i in range(len(prompts))]
    model = plain_model(folders, "D", dtype)
    for p, g in zip(prompts, got):
        within_bound_of_the_best(model, p, g, dtype)
    if dtype == "float32":
        assert got == generated
    assert all(r.cache.length(f"g{i}") == len(p) + new - 1 for i, p in enumerate(prompts))
    for i in range(len(prompts)):
        r.end(f"g{i}")
    r.cache.check()


def test_default_cache_size_and_abort_with_a_step_in_flight(folders):
    """An engine that is not told how many pages to make sizes its cache from the device's
    memory (no more than every sequence at full length can use), generates what the plain
    model generates, and a request aborted while the next step is already on the device
    leaves the others' tokens and the pool untouched."""
    from inferloop_b200 import Engine, SamplingParams
    cfg, _, page = CONFIGS["D"]
    prompts = [random_tokens(n, cfg["vocab_size"], 1200 + n) for n in (30, 12, 55)]
    model = plain_model(folders, "D", "float32")
    e = Engine(folders["D"], dtype="float32", block_size=page, max_num_seqs=4, max_model_len=512, prefill_chunk_tokens=64)
    info = e.inspect()
    group = info["cache"]["groups"][0]
    assert group["total"] == (512 // page) * 4 and group["free"] == group["total"]
    assert e.activation_reserve > 0
    want = [plain.generate(model, p, 30) for p in prompts]
    assert e.generate(prompts, SamplingParams(), 30) == want
    # the same again; the middle request is aborted once a step has been launched ahead
    ids = [e.submit(p, SamplingParams(), 30, request_id=f"a{i}") for i, p in enumerate(prompts)]
    aborted = False
    while not e.is_idle():
        e.step()
        if not aborted and e._ahead is not None and len(e.result("a1").generated) >= 5:
            e.abort("a1")
            aborted = True
    assert aborted, "no step was ever launched ahead"
    assert e.result("a1").finish_reason == "abort" and 5 <= len(e.result("a1").generated) < 30
    assert e.result("a0").generated == want[0] and e.result("a2").generated == want[2]
    assert e.result("a1").generated == want[1][:len(e.result("a1").generated)]
    info = e.inspect()
    assert info["running"] == 0 and all(g["free"] == g["total"] for g in info["cache"]["groups"])
    e.runner.cache.check()


def test_default_sizes_give_a_windowed_group_a_smaller_pool(folders):
    """Layers that read a window of 40 keys share a page group whose pool the default sizing
    makes as large as the window, the largest step and a page of slack need, not as large as
    the pool of the layers that keep every key; generation is what the plain model generates."""
    from inferloop_b200 import Engine, SamplingParams
    cfg, _, page = CONFIGS["E"]
    e = Engine(folders["E"], dtype="float32", block_size=page, max_num_seqs=4, max_model_len=1024, prefill_chunk_tokens=64)
    groups = {g["window"]: g for g in e.inspect()["cache"]["groups"]}
    assert groups[None]["total"] == (1024 // page) * 4
    per_request = -(-(40 + (64 + 3) + page) // page) + 1
    assert groups[40]["total"] == per_request * 4 < groups[None]["total"]
    prompts = [random_tokens(n, cfg["vocab_size"], 1500 + n) for n in (150, 60, 33, 97)]
    model = plain_model(folders, "E", "float32")
    assert e.generate(prompts, SamplingParams(), 40) == [plain.generate(model, p, 40) for p in prompts]
    info = e.inspect()
    assert all(g["free"] == g["total"] for g in info["cache"]["groups"]) and info["cache"]["window_pages_released"] > 0
    e.runner.cache.check()


@pytest.mark.parametrize("M", [8, 64])
def test_output_matrix_at_the_serving_vocabulary(M):
    """The tensor-core GEMM at the shape of the serving model's output matrix, (M, 151936,
    4096), where it runs as a persistent grid with more tiles than CTAs: a few hundred
    columns against 64-bit sums.  One row through the exact 32-bit kernel at that width too."""
    from inferloop_b200.csrc import ops
    N, K = 151936, 4096
    g = torch.Generator().manual_seed(M)
    a = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    wd = w.cuda()
    ops.gemm_tc(a.cuda(), wd, out)
    plan = ops.gemm_tc_plan(M, N, K)
    assert plan["swap"] == 1 and plan["tiles"] > plan["grid"], plan       # the persistent form
    ops.check_device_errors()
    assert torch.isfinite(out).all()
    cols = torch.cat([torch.arange(0, 64), torch.randint(0, N, (300,), generator=g), torch.arange(N - 64, N)])
    ref = a.double() @ w[cols].double().T
    got = out[:, cols.cuda()].double().cpu()
    err = (got - ref).abs()
    # 32-bit accumulation of 4096 products of bfloat16 values: relative 2^-20 of the sum of magnitudes
    bound = 1e-5 * (a.double().abs() @ w[cols].double().abs().T) + 1e-6
    assert (err <= bound).all(), float((err / bound).max())
    if M == 8:
        a32, w32 = a[:1].float().cuda(), wd.float()
        out32 = torch.full((1, N), float("nan"), dtype=torch.float32, device="cuda")
        ops.gemm_simt(a32, w32, out32)
        err = (out32[:, cols.cuda()].double().cpu() - ref[:1]).abs()
        assert (err <= 1e-6 + 1e-5 * ref[:1].abs()).all(), float(err.max())
