"""Sampling: the host sampler against the plain rules (no GPU) and the device kernels
against the host sampler (GPU)."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from inferloop_b200.sampling import SamplingParams, host


def test_params_ranges():
    SamplingParams(temperature=0.7, top_k=5, top_p=0.9, min_p=0.1, presence_penalty=-2.0, repetition_penalty=1.3)
    for bad in (dict(temperature=-1), dict(top_k=0), dict(top_p=0.0), dict(top_p=1.5), dict(min_p=2.0),
                dict(presence_penalty=3.0), dict(repetition_penalty=0.0), dict(temperature=float("nan"))):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
    assert SamplingParams().uses_plain_greedy() and not SamplingParams(presence_penalty=0.5).uses_plain_greedy()
    assert SamplingParams(eos_token=3, eos_tokens=(5,)).is_eos(5) and SamplingParams(eos_token=3).is_eos(3)


def test_host_sampler_equals_the_plain_rules():
    rng = np.random.default_rng(0)
    for trial in range(60):
        logits = rng.standard_normal(97).astype(np.float32) * 3
        if trial % 5 == 0:
            logits[10] = logits[40] = logits.max() + 1       # equal maxima
        kw = [dict(temperature=0.0), dict(temperature=0.8), dict(temperature=1.3, top_k=9),
              dict(temperature=0.6, top_p=0.7), dict(temperature=1.0, min_p=0.2),
              dict(temperature=0.9, top_k=20, top_p=0.8, min_p=0.05)][trial % 6]
        p = SamplingParams(seed=trial, **kw)
        want = plain.sample(logits.tolist(), p.temperature, p.seed, request=7, position=trial,
                            top_k=p.top_k, top_p=p.top_p, min_p=p.min_p)
        assert host.sample(logits, p, 7, trial) == want
    assert host.uniform(5, 9, 2) == plain.uniform_for(5, 9, 2)


def test_penalties():
    logits = np.array([2.0, -1.0, 1.9, 0.5], dtype=np.float32)
    p = SamplingParams(repetition_penalty=2.0)
    assert host.sample(logits, p, 0, 0, prompt=[0]) == 2                 # 2.0 / 2 < 1.9
    p = SamplingParams(presence_penalty=0.2)
    assert host.sample(logits, p, 0, 0, prompt=[0], generated=[]) == 0  # presence counts generated only
    assert host.sample(logits, p, 0, 0, generated=[0]) == 2
    with pytest.raises(ValueError):
        host.sample(logits, SamplingParams(repetition_penalty=1.5), 0, 0, prompt=[9])
    with pytest.raises(ValueError):
        host.sample(np.array([0.0, np.inf], dtype=np.float32), SamplingParams(), 0, 0)


# ---------------------------------------------------------------- the reference's own expectations
# Literal inputs and answers of the reference's sampler tests
# (crates/engine/workloads/tests/unit/sampling.rs): these pin the samplers here to the
# reference's output, not to a reading of its source.
F32_MIN, F32_MAX = float(np.finfo(np.float32).min), float(np.finfo(np.float32).max)
REFERENCE_GREEDY = [([2.0, 2.0, 1.0], 0), ([-0.0, 0.0, 0.0], 1), ([F32_MIN, -5.0, -6.0], 1), ([F32_MAX, F32_MAX], 0)]   # :5-12


def test_reference_expectations_greedy():
    """sampling.rs (tests) :4-19 and :98-99: ties, signed zero (total order: -0 < +0), the
    extremes of the range, non-finite and empty input refused."""
    for logits, want in REFERENCE_GREEDY:
        assert plain.greedy(logits) == want
        assert host.greedy(np.array(logits, dtype=np.float32)) == want
        assert host.sample(np.array(logits, dtype=np.float32), SamplingParams(), 1, 0) == want
    for invalid in (float("nan"), float("inf"), float("-inf")):
        with pytest.raises(ValueError):
            plain.greedy([F32_MAX, invalid])
        with pytest.raises(ValueError):
            host.sample(np.array([F32_MAX, invalid], dtype=np.float32), SamplingParams(), 1, 0)
    with pytest.raises(ValueError):
        host.sample(np.array([], dtype=np.float32), SamplingParams(), 1, 0)
    with pytest.raises(ValueError):
        plain.greedy([])
    assert host.sample(np.ones(1024, dtype=np.float32), SamplingParams(), 1, 0) == 0
    assert plain.greedy([1.0] * 1024) == 0


def test_reference_expectations_filters_and_penalties():
    """sampling.rs (tests) :103-140: nucleus 0.5 over [3, 1, 0] keeps token 0 for seeds
    0..20; min-p 0.9 keeps token 0; presence 2.0 with generated [0, 0] turns [3, 2] to token
    1; repetition 2.0 with prompt [0] does too."""
    logits = np.array([3.0, 1.0, 0.0], dtype=np.float32)
    for seed in range(20):
        assert host.sample(logits, SamplingParams(temperature=1.0, top_p=0.5, seed=seed), 1, 0) == 0
        assert plain.sample(logits.tolist(), 1.0, seed, 1, 0, top_p=0.5) == 0
        assert host.sample(logits, SamplingParams(temperature=1.0, min_p=0.9, seed=seed), 1, 0) == 0
        assert plain.sample(logits.tolist(), 1.0, seed, 1, 0, min_p=0.9) == 0
    two = np.array([3.0, 2.0], dtype=np.float32)
    assert host.sample(two, SamplingParams(temperature=0.0, min_p=0.9, presence_penalty=2.0), 1, 0,
                       prompt=[1], generated=[0, 0]) == 1
    assert host.sample(two, SamplingParams(temperature=0.0, min_p=0.9, repetition_penalty=2.0), 1, 0,
                       prompt=[0], generated=[]) == 1


def test_reference_expectations_top_k_trajectory():
    """sampling.rs (tests) :49-77: logits (17 i + seed) mod 53 over 257 tokens, T = 0.7,
    top-k in {none, 1, 7, 256, 1024}, request seed + 1, positions 0..8: the selection with a
    partial top-k equals the full sort's.  Here: the host sampler equals the plain one."""
    for seed in range(0, 128, 9):
        logits = np.array([float((i * 17 + seed) % 53) for i in range(257)], dtype=np.float32)
        for top_k in (None, 1, 7, 256, 1024):
            p = SamplingParams(seed=seed, top_k=top_k, temperature=0.7)
            for position in range(8):
                assert host.sample(logits, p, seed + 1, position) == \
                    plain.sample(logits.tolist(), 0.7, seed, seed + 1, position, top_k=top_k)


def test_generation_defaults_from_the_folder(tmp_path):
    """generation_config.json and eos_token_id as the reference reads them
    (crates/model/package/src/generation/read.rs:9-100) and a request's overrides field by
    field (generation/mod.rs:68-128)."""
    import json
    from inferloop_b200.sampling import GenerationDefaults
    d = GenerationDefaults.from_configs({"eos_token_id": 7})
    assert d.base == SamplingParams(eos_tokens=(7,)) and d.sources["eos_tokens"] == "config.json"
    d = GenerationDefaults.from_configs({"text_config": {"eos_token_id": [3, 4]}, "eos_token_id": 9})
    assert d.base.eos_tokens == (3, 4)
    gen = {"do_sample": True, "temperature": 0.6, "top_k": 20, "top_p": 0.95, "eos_token_id": [151645, 151643]}
    d = GenerationDefaults.from_configs({"eos_token_id": 1}, gen)
    assert d.base == SamplingParams(temperature=0.6, top_k=20, top_p=0.95, eos_tokens=(151645, 151643))
    assert d.sources["eos_tokens"] == "generation_config.json" and d.sources["min_p"] == "runtime fallback"
    # do_sample false (or absent) forces greedy whatever temperature the file names
    assert GenerationDefaults.from_configs({}, {"do_sample": False, "temperature": 0.6}).base.temperature == 0.0
    assert GenerationDefaults.from_configs({}, {"temperature": 0.6}).base.temperature == 0.0
    assert GenerationDefaults.from_configs({}, {"do_sample": True}).base.temperature == 1.0
    assert GenerationDefaults.from_configs({}, {"do_sample": True, "top_k": 0}).base.top_k is None
    for bad in ({"do_sample": 1}, {"top_k": -1}, {"top_k": 1.5}, {"eos_token_id": -1}, {"eos_token_id": "x"}, {"temperature": "hot"}):
        with pytest.raises(ValueError):
            GenerationDefaults.from_configs({}, bad)
    # overrides
    assert d.resolve({}) == d.base
    assert d.resolve({"temperature": 0.0}).temperature == 0.0 and d.resolve({"top_k": 0}).top_k is None
    assert d.resolve({"do_sample": False}).temperature == 0.0
    g = GenerationDefaults.from_configs({"eos_token_id": 1})
    assert g.resolve({"do_sample": True}).temperature == 1.0 and g.resolve({"do_sample": True, "temperature": 0.3}).temperature == pytest.approx(0.3)
    r = d.resolve({"eos_token": 5})
    assert r.eos_token == 5 and r.eos_tokens == () and r.is_eos(5) and not r.is_eos(151645)
    r = d.resolve({"eos_tokens": [8, 9], "seed": 3})
    assert r.eos_tokens == (8, 9) and r.eos_token is None and r.seed == 3
    with pytest.raises(ValueError, match="unknown sampling fields"):
        d.resolve({"temperatur": 1.0})
    # an explicit SamplingParams that names no stop token inherits the folder's
    assert d.with_stop_tokens(SamplingParams(temperature=0.2)).eos_tokens == (151645, 151643)
    assert d.with_stop_tokens(SamplingParams(eos_token=2)).eos_tokens == ()
    # from a folder
    folder = tmp_path / "m"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps({"eos_token_id": 11}))
    assert GenerationDefaults.from_folder(str(folder)).base.eos_tokens == (11,)
    (folder / "generation_config.json").write_text(json.dumps({"eos_token_id": [12]}))
    assert GenerationDefaults.from_folder(str(folder)).base.eos_tokens == (12,)
    (folder / "generation_config.json").write_text("[1]")
    with pytest.raises(ValueError):
        GenerationDefaults.from_folder(str(folder))


@pytest.mark.gpu
def test_device_argmax_reference_expectations():
    """The reference's literal greedy cases on the device kernel, one row each, and one wide
    row where the only +0 sits among -0 in another CTA's part of the vocabulary."""
    from inferloop_b200.csrc import ops
    for logits, want in REFERENCE_GREEDY:
        dev = torch.tensor([logits], dtype=torch.float32, device="cuda")
        out = torch.empty(1, dtype=torch.int32, device="cuda")
        bad = torch.empty(1, dtype=torch.int32, device="cuda")
        ops.argmax(dev, out, bad)
        assert out.tolist() == [want] and bad.tolist() == [0]
    wide = torch.full((1, 151936), -0.0)
    wide[0, 100000] = 0.0
    wide[0, 140000] = 0.0
    out = torch.empty(1, dtype=torch.int32, device="cuda")
    ops.argmax(wide.cuda(), out, None)
    assert out.tolist() == [100000]


@pytest.mark.gpu
@pytest.mark.parametrize("vocab", [257, 1000, 151936])
def test_device_argmax(vocab):
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(vocab)
    logits = torch.randn(5, vocab, generator=g)
    logits[1, 7] = logits[1, vocab - 3] = 50.0          # equal maxima: the lower index wins
    logits[2, vocab - 1] = 60.0
    dev = logits.cuda()
    out = torch.empty(5, dtype=torch.int32, device="cuda")
    bad = torch.empty(5, dtype=torch.int32, device="cuda")
    ops.argmax(dev, out, bad)
    assert out.tolist() == [host.greedy(r.numpy()) for r in logits]
    assert out.tolist()[1] == 7 and out.tolist()[2] == vocab - 1 and bad.tolist() == [0] * 5
    dev[3, 11] = float("nan")
    ops.argmax(dev, out, bad)
    assert bad.tolist() == [0, 0, 0, 1, 0]


@pytest.mark.gpu
@pytest.mark.parametrize("vocab", [320, 5003, 9000, 151936, 200003])
def test_device_temperature_draw_equals_the_host_rule(vocab):
    from inferloop_b200.csrc import ops
    rows = 64
    g = torch.Generator().manual_seed(vocab + 1)
    logits = torch.randn(rows, vocab, generator=g) * 2
    logits[3, 5] = logits[3, 100] = logits[3].max() + 0.5      # equals at the top
    logits[4, :] = 0.25                                         # all equal
    temps = [0.5 + 0.02 * i for i in range(rows)]
    us = [host.uniform(11, 3, i) for i in range(rows)]
    us[5], us[6] = 0.0, 1.0 - 2 ** -53
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    bad = torch.empty(rows, dtype=torch.int32, device="cuda")
    ops.sample_temperature(logits.cuda(), torch.tensor(temps, dtype=torch.float32).cuda(),
                           torch.tensor(us, dtype=torch.float64).cuda(), out, bad)
    got = out.tolist()
    assert bad.tolist() == [0] * rows
    same = 0
    for i in range(rows):
        # the host rule with the same uniform number
        order = np.lexsort((np.arange(vocab), -logits[i].double().numpy()))
        w = np.exp((logits[i].double().numpy()[order] - logits[i].max().item()) / float(np.float32(temps[i])))
        c = np.cumsum(w / w.sum())
        want = int(order[min(int(np.searchsorted(c, us[i], side="right")), vocab - 1)])
        if got[i] == want:
            same += 1
        else:   # sums in another order may move the crossing by rounding: then u sits on a boundary
            k = list(order).index(got[i])
            assert abs(c[k] - us[i]) < 1e-9 or (k > 0 and abs(c[k - 1] - us[i]) < 1e-9), (i, got[i], want)
    assert same >= rows - 1


@pytest.mark.gpu
@pytest.mark.parametrize("vocab", [320, 9000, 151936])
def test_device_filtered_draw_equals_the_host_rule(vocab):
    """top-k, min-p and top-p on the device: the same token as the host sampler (the
    reference's rule step by step) for the same uniform number, row by row with different
    filters, with equal logits at the top, inside the kept prefix and everywhere."""
    from inferloop_b200.csrc import ops
    rows = 40
    g = torch.Generator().manual_seed(vocab + 7)
    logits = torch.randn(rows, vocab, generator=g) * 2.5
    logits[3, 5] = logits[3, 100] = logits[3, 17] = logits[3].max() + 0.5      # three equals at the top
    logits[4, :] = 0.25                                                         # all equal
    logits[6, 10:30] = 1.5                                                      # a run of equals inside
    ks = [None, 1, 5, 50, 1000, 3]
    ps = [1.0, 0.9, 0.5, 0.1, 0.999]
    ms = [0.0, 0.05, 0.5, 0.0]
    params = [SamplingParams(temperature=0.4 + 0.03 * i, top_k=ks[i % len(ks)], top_p=ps[i % len(ps)],
                             min_p=ms[i % len(ms)], seed=21) for i in range(rows)]
    us = [host.uniform(21, i, 0) for i in range(rows)]
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    bad = torch.empty(rows, dtype=torch.int32, device="cuda")
    ops.sample_temperature(
        logits.cuda(), torch.tensor([p.temperature for p in params], dtype=torch.float32).cuda(),
        torch.tensor(us, dtype=torch.float64).cuda(), out, bad,
        torch.tensor([p.top_k or 0 for p in params], dtype=torch.int32).cuda(),
        torch.tensor([p.top_p for p in params], dtype=torch.float32).cuda(),
        torch.tensor([p.min_p for p in params], dtype=torch.float32).cuda())
    got = out.tolist()
    assert bad.tolist() == [0] * rows
    same = 0
    for i in range(rows):
        want = host.sample(logits[i].numpy(), params[i], i, 0)
        if got[i] == want:
            same += 1
        else:   # sums in another order can move a boundary by rounding: then the two are neighbours in the order
            order = list(np.lexsort((np.arange(vocab), -logits[i].double().numpy())))
            assert abs(order.index(got[i]) - order.index(want)) == 1, (i, got[i], want, params[i])
    assert same >= rows - 2, same


@pytest.mark.gpu
@pytest.mark.parametrize("vocab", [515, 151936])
def test_device_penalties_equal_the_host_rule(vocab):
    """Repetition and presence penalties applied by the device kernel (token bitmaps made
    from each row's prompt and output) before the filters and the draw: the same token as
    the host sampler, also for a row without a temperature (the best penalised logit)."""
    import dataclasses
    from inferloop_b200.sampling.device import DeviceSampler
    rows = 24
    g = torch.Generator().manual_seed(vocab + 3)
    logits = torch.randn(rows, vocab, generator=g) * 2.0
    rng = np.random.default_rng(vocab)
    params, hist = [], []
    for i in range(rows):
        top = [int(t) for t in torch.topk(logits[i], 6).indices]          # penalise what would win
        prompt = top[:3] + [int(t) for t in rng.integers(0, vocab, 20)]
        generated = top[3:5] + [int(t) for t in rng.integers(0, vocab, 7)] + top[3:4]
        params.append(SamplingParams(temperature=0.0 if i % 6 == 0 else 0.5 + 0.05 * i,
                                     top_k=None if i % 3 else 40, top_p=1.0 if i % 2 else 0.8,
                                     presence_penalty=[0.0, 1.5, -0.7][i % 3], repetition_penalty=[1.3, 1.0, 2.5, 0.8][i % 4],
                                     seed=5))
        hist.append((prompt, generated))
    sampler = DeviceSampler(torch.device("cuda", 0), max_rows=8)           # grows on demand
    drawn_with = [p if p.temperature > 0 else dataclasses.replace(p, temperature=1.0, top_k=1, top_p=1.0) for p in params]
    us = [host.uniform(5, i, len(hist[i][1])) for i in range(rows)]
    sampler.temperature_launch(logits.cuda(), [p.temperature for p in drawn_with], us, drawn_with, hist)
    got = sampler.read(rows)
    same = 0
    for i in range(rows):
        want = host.sample(logits[i].numpy(), params[i], i, len(hist[i][1]), prompt=hist[i][0], generated=hist[i][1])
        same += int(got[i] == want)
    assert same >= rows - 1, (same, got)
