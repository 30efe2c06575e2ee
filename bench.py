#!/usr/bin/env python3
"""Measurement of the engine on one B200, random bf16 weights, synthetic token ids.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]
                    [--config 8b|14b-mixed|32b-long] [--breakdown] [--kernels [attention|products]] [--further]

One JSON line on stdout.  The default (`--config 8b`) is the headline: Qwen3-8B layer sizes,
36 layers, batch 8, 1,024-token prompts; a "step" is one decode step of the whole batch.
  value     decoded tokens per second of K steps run back to back on the device (each
            step's arg-max feeds the next step there), timed with CUDA events;
  e2e       the same through the Python entry point (`Engine.step`): host token ids in,
            host token ids out, every step with its host->device copy of the step's
            arrays from pinned memory and its device->host read of the drawn ids;
  prefill   one 2,048-token prompt to its last logits (median of several);
  roofline  bytes a decode step must read (every weight once + the cache of the live
            requests) / its time, against the measured copy bandwidth;
  points    decode at batch 1 and 64.
`--config 14b-mixed`: Qwen3-14B layer sizes, 32 requests with prompts of 128 to 3,072 tokens
through `Engine.generate` with prompt portions of 512 tokens mixed with decoding, 128 greedy
tokens each; a "step" is one engine step and `--steps` is ignored (the job is run whole, once
untimed and once timed).  `--config 32b-long`: Qwen3-32B layer sizes, 8,192-token prompts,
decode at batch 1 and 16.  `--breakdown` adds the share of every op class in a decode step
and in the prefill step, from a pair of CUDA events around every kernel (the engine's
`device_timing="node"` mode; every kernel's figure carries the few microseconds that a pair
of events around a lone launch costs).  `--kernels` times kernels alone instead, at the layer
sizes of `--config`: the prefill attention at several lengths, and the layer's matrix products
at several token counts beside `torch.matmul` on the same shapes (the library's plain product,
for comparison only; it has no epilogue).  `--further` measures further sizes at the 8B layer
sizes: decode at batches 16 to 256, a prompt of 32,768 tokens in portions, the 32-bit path.
Peaks come from MEASURED_PEAKS.json beside this file when present, else the fallback
figures 6.65 TB/s and 1.59 PFLOP/s.  Weights (15 GB and more) exceed L2 (126 MB), so every
step reads them from HBM: no L2 flush is needed between timed steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

_COMMON = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", head_dim=128, vocab_size=151936,
               rope_theta=1000000.0, rms_norm_eps=1e-6, attention_bias=False, tie_word_embeddings=False,
               hidden_act="silu")
# layer sizes of Qwen3-8B, Qwen3-14B and Qwen3-32B
QWEN3_8B = dict(_COMMON, num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                intermediate_size=12288, max_position_embeddings=4096)
QWEN3_14B = dict(_COMMON, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                 intermediate_size=17408, max_position_embeddings=4096)
QWEN3_32B = dict(_COMMON, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8,
                 intermediate_size=25600, max_position_embeddings=16384)
FULL_LAYERS = 36
SEED = 2
PROMPT_LEN = 1024
PREFILL_LEN = 2048
PREFILL_SAMPLES = 5
PAGE = 16

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(HERE, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as fh:
                raw = json.load(fh)
            found = {}

            def walk(node):                     # the numbers may sit at the top or one level down
                if isinstance(node, dict):
                    for k, v in node.items():
                        if k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained") and isinstance(v, (int, float)):
                            found.setdefault(k, float(v))
                        else:
                            walk(v)
            walk(raw)
            if "hbm_gbs" in found and "bf16_tflops" in found:
                return dict(found, source="measured")
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0) -> None:
        self.path = tempfile.mktemp(prefix="ilb-clocks-", suffix=".csv")
        self.proc = None
        self.index = index

    def __enter__(self):
        try:
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=self.fh, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.fh.close()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            with open(self.path) as fh:
                for line in fh:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) < 6:
                        continue
                    try:
                        sm.append(float(parts[0])); mx.append(float(parts[1]))
                    except ValueError:
                        continue
                    for name, v in zip(names, parts[2:6]):
                        if v.lower().startswith("active"):
                            reasons.add(name)
            os.remove(self.path)
        except OSError:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def model_numbers(cfg: dict):
    """Parameters the matrix products of one token touch, and bytes of cache per token."""
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nq + 2 * nkv) * d * H + nq * d * H + 3 * H * I
    return {"layer_params": per_layer, "head_params": V * H, "kv_bytes_per_token": 2 * nkv * d * 2 * L,
            "attn_flops_per_pair": 4 * nq * d * L, "layers": L}


def step_flops(nums: dict, tokens: int, logit_rows: int, pairs: int) -> float:
    return (2.0 * tokens * nums["layer_params"] * nums["layers"] + 2.0 * logit_rows * nums["head_params"]
            + nums["attn_flops_per_pair"] * pairs)


def flat_config(name: str, cfg: dict, **more) -> dict:
    out = {"model": name, "layers": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
           "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
           "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "kv_page": PAGE, "kv_dtype": "bf16",
           "sampling": "greedy", "parallelism": "1 GPU"}
    out.update(more)
    return out


class Bench:
    """An engine with random weights and the measurements made on it."""

    def __init__(self, cfg: dict, seed: int, pages: int, max_seqs: int, max_model_len: int, chunk: int) -> None:
        import torch
        from inferloop_b200.engine.engine import Engine
        self.torch = torch
        self.cfg, self.nums, self.pk = cfg, model_numbers(cfg), peaks()
        t0 = time.time()
        self.engine = Engine(cfg, dtype="bfloat16", device=0, block_size=PAGE, num_gpu_blocks_override=pages,
                             max_num_seqs=max_seqs, max_model_len=max_model_len, prefill_chunk_tokens=chunk,
                             max_num_batched_tokens=chunk + max_seqs, random_weights_seed=seed)
        self.runner = self.engine.runner
        self.chunk = chunk
        self.weight_bytes = self.runner.model.weight_bytes()
        print(f"[bench] model ready in {time.time() - t0:.1f} s, weights {self.weight_bytes / 1e9:.2f} GB",
              file=sys.stderr, flush=True)
        self.gen = torch.Generator().manual_seed(seed)

    def prompts(self, n, length):
        return self.torch.randint(0, self.cfg["vocab_size"], (n, length), generator=self.gen).tolist()

    def prefill(self, ids, toks):
        """Every prompt in portions of `chunk`; returns each request's first drawn token."""
        from inferloop_b200.engine import StepEntry
        last = {}
        for rid, t in zip(ids, toks):
            for i in range(0, len(t), self.chunk):
                part = t[i:i + self.chunk]
                _, drawn = self.runner.step([StepEntry(rid, part, [len(part) - 1])], draw_greedy=True)
            last[rid] = int(drawn.ids[0].item())
        return last

    def decode_device(self, batch, steps, warmup, tag, prompt_len):
        """K decode steps back to back on the device; returns (tokens/s, ms/step, kernels/step, mean context)."""
        from inferloop_b200.engine import StepEntry
        torch, runner = self.torch, self.runner
        ids = [f"{tag}{i}" for i in range(batch)]
        last = self.prefill(ids, self.prompts(batch, prompt_len))
        entries = [StepEntry(rid, [last[rid]], [0]) for rid in ids]
        out = runner.graphs.run_greedy(entries, warmup)
        entries = [StepEntry(rid, [int(t)], [0]) for rid, t in zip(ids, out[-1].tolist())]
        start_ctx = runner.cache.length(ids[0])
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        runner.graphs.run_greedy(entries, steps)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        kernels = runner.graphs.recorded(batch, True).kernels + 1
        for rid in ids:
            runner.end(rid)
        return batch * steps / (ms / 1e3), ms / steps, kernels, start_ctx + steps / 2

    def decode_roofline(self, batch, mean_ctx, ms_per_step) -> dict:
        step_bytes = self.weight_bytes + batch * mean_ctx * self.nums["kv_bytes_per_token"]
        achieved = step_bytes / (ms_per_step / 1e3) / 1e9
        return {"bound": "hbm", "achieved": round(achieved, 1), "peak": self.pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / self.pk["hbm_gbs"], 4)}

    def prefill_timed(self, length, warmup, samples) -> dict:
        """One prompt of `length` tokens (in portions of `chunk`) to its last logits: the
        median of `samples` runs after `warmup` untimed ones."""
        from inferloop_b200.engine import StepEntry
        torch, runner = self.torch, self.runner
        toks = self.prompts(warmup + samples, length)
        times = []
        for i, t in enumerate(toks):
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for k in range(0, length, self.chunk):
                part = t[k:k + self.chunk]
                runner.step([StepEntry("pf", part, [len(part) - 1] if k + self.chunk >= length else [])])
            b.record()
            torch.cuda.synchronize()
            runner.end("pf")
            if i >= warmup:
                times.append(a.elapsed_time(b))
        pms = statistics.median(times)
        flops = sum(step_flops(self.nums, min(self.chunk, length - k), 1 if k + self.chunk >= length else 0,
                               sum(range(k + 1, min(k + self.chunk, length) + 1)))
                    for k in range(0, length, self.chunk))
        return {"value": round(length / (pms / 1e3), 1), "tokens": length, "ms": round(pms, 3),
                "frac": round(flops / (pms / 1e3) / (self.pk["bf16_tflops"] * 1e12), 4),
                "peak_tflops": self.pk["bf16_tflops"],          # the burst figure: the stricter of the two measured peaks
                "samples": [round(t, 3) for t in times]}

    def breakdown(self, batch, prompt_len, prefill_len) -> dict:
        """Share of every op class in a decode step of `batch` sequences and in one prefill
        step, from a pair of events around each kernel (steps run kernel by kernel)."""
        from inferloop_b200.engine import StepEntry
        runner = self.runner
        ids = [f"bd{i}" for i in range(batch)]
        last = self.prefill(ids, self.prompts(batch, prompt_len))
        runner.set_device_timing("node")
        out = {}
        try:
            entries = [StepEntry(rid, [last[rid]], [0]) for rid in ids]
            for i in range(3 + 8):
                if i == 3:
                    runner.timer.reset()
                _, drawn = runner.step(entries, draw_greedy=True)
                entries = [StepEntry(rid, [int(t)], [0]) for rid, t in zip(ids, drawn.ids.tolist())]
            out["decode"] = _per_step(runner.timer.summary())
            for rid in ids:
                runner.end(rid)
            toks = self.prompts(3, prefill_len)
            for i, t in enumerate(toks):
                if i == 2:
                    runner.timer.reset()
                runner.step([StepEntry("bdp", t[:self.chunk], [min(len(t), self.chunk) - 1])], draw_greedy=True)
                runner.end("bdp")
            out["prefill"] = _per_step(runner.timer.summary())
        finally:
            runner.set_device_timing("off")
        return out


    def breakdown_mixed(self, singles, context, portion) -> dict:
        """Share of every op class in a mixed step: `singles` requests that decode at
        `context` keys beside a `portion` of one long prompt whose earlier part is in the cache."""
        from inferloop_b200.engine import StepEntry
        runner = self.runner
        ids = [f"bm{i}" for i in range(singles)]
        last = self.prefill(ids, self.prompts(singles, context))
        steps = 3 + 5
        done = 1024                                   # of the long prompt, before the measured portions
        long_prompt = self.prompts(1, done + steps * portion)[0]
        self.prefill(["bmp"], [long_prompt[:done]])
        runner.set_device_timing("node")
        try:
            entries = [StepEntry(rid, [last[rid]], [0]) for rid in ids]
            for i in range(steps):
                if i == 3:
                    runner.timer.reset()
                part = long_prompt[done + i * portion:done + (i + 1) * portion]
                _, drawn = runner.step(entries + [StepEntry("bmp", part, [])], draw_greedy=True)
                entries = [StepEntry(rid, [int(t)], [0]) for rid, t in zip(ids, drawn.ids.tolist())]
            out = _per_step(runner.timer.summary())
        finally:
            runner.set_device_timing("off")
        for rid in ids + ["bmp"]:
            runner.end(rid)
        out["step"] = {"single_token_seqs": singles, "context": context, "portion_tokens": portion,
                       "portion_starts_at": f"{done} to {done + (steps - 1) * portion}"}
        return out


def _per_step(summary: dict) -> dict:
    n = max(summary.get("steps", {}).get("count", 1), 1)
    return {"steps": n, "ms_per_step_events_around_step": round(summary["steps"]["ms_total"] / n, 4),
            "ms_per_step_sum_of_kernels": round(summary["ops_ms_total"] / n, 4),
            "ops": {k: {"us_per_step": round(1e3 * v["ms"] / n, 2), "launches_per_step": v["launches"] / n,
                        "share": v["share"],
                        **({"kernels_us_per_step": {name: round(1e3 * per["ms"] / n, 2) for name, per in v["kernels"].items()}}
                           if len(v["kernels"]) > 1 else {})}
                    for k, v in summary["ops"].items()}}


# ----------------------------------------------------------------------------- the three configurations
def run_8b(args) -> dict:
    import torch
    from inferloop_b200.sampling import SamplingParams
    cfg = dict(QWEN3_8B, num_hidden_layers=args.layers)
    max_batch = max(64, args.batch)
    tokens_per_seq = PROMPT_LEN + args.warmup + args.steps + 64 + -(-max_batch * PROMPT_LEN // PREFILL_LEN)
    pages = max_batch * (-(-tokens_per_seq // PAGE)) + 256
    bench = Bench(cfg, SEED, pages, max_batch, 4096, PREFILL_LEN)
    engine, runner = bench.engine, bench.runner

    # ---------------------------------------------------------------- headline: device-timed decode
    with ClockSampler() as clocks:
        value, ms_per_step, kernels, mean_ctx = bench.decode_device(args.batch, args.steps, args.warmup, "d", PROMPT_LEN)
    clock_info = clocks.summary()

    # ---------------------------------------------------------------- end to end through Engine.step
    # (requests admitted first decode while the later prompts are still being taken in: room for those tokens too)
    while_prompts = -(-args.batch * PROMPT_LEN // PREFILL_LEN)
    rids = [engine.submit(p, SamplingParams(), max_new_tokens=args.warmup + args.steps + 32 + while_prompts)
            for p in bench.prompts(args.batch, PROMPT_LEN)]
    while any(runner.cache.length(r.id) < PROMPT_LEN for r in engine.scheduler.running) or engine.scheduler.waiting:
        engine.step()
    for _ in range(args.warmup):
        engine.step()
    torch.cuda.synchronize()
    h2d = d2h = 0
    made = lambda: sum(len(engine.result(r).generated) for r in rids)      # tokens handed to the host so far
    before = made()
    t_start = time.perf_counter()
    for _ in range(args.steps):
        engine.step()
        h2d += runner.stager.bytes_last
        d2h += engine.sampler.d2h_bytes_last
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t_start
    e2e_value = (made() - before) / e2e_s
    while not engine.is_idle():
        engine.step()
    engine.take_completed()

    result = {
        "metric": "Qwen3-8B bf16 decode tok/s", "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random-init weights (seed 2), token ids uniform in [0, vocab)",
        "config": flat_config("Qwen3-8B sizes", cfg, global_batch=args.batch, seq_len=4096, prompt_len=PROMPT_LEN,
                              layers_full=FULL_LAYERS, l2="inputs larger than L2 (weights 15 GB)",
                              peaks=bench.pk["source"]),
        "e2e": {"value": round(e2e_value, 2), "unit": "tokens/s", "h2d_bytes_per_step": h2d // args.steps,
                "d2h_bytes_per_step": d2h // args.steps},
        "gpu_launches": kernels * args.steps,
        "clocks": clock_info,
        "roofline": bench.decode_roofline(args.batch, mean_ctx, ms_per_step),
    }
    if not args.no_points:
        result["prefill"] = bench.prefill_timed(PREFILL_LEN, min(args.warmup, 3), PREFILL_SAMPLES)
        points = {}
        for b_, steps in ((1, min(args.steps, 64)), (64, min(args.steps, 64))):
            v, _, _, _ = bench.decode_device(b_, steps, args.warmup, f"p{b_}_", PROMPT_LEN)
            points[f"decode_b{b_}"] = round(v, 2)
        result["points"] = points
    if args.breakdown:
        result["breakdown"] = bench.breakdown(args.batch, PROMPT_LEN, PREFILL_LEN)
    return result


def run_14b_mixed(args) -> dict:
    """32 requests, prompts of 128 to 3,072 tokens, portions of 512 mixed with decoding, 128
    greedy tokens each, through Engine.generate: the scheduler and the mixed step, timed."""
    import torch
    from inferloop_b200.sampling import SamplingParams
    cfg = dict(QWEN3_14B)
    n_req, new, chunk, seed = 32, 128, 512, 3
    pages = n_req * (-(-(3072 + new) // PAGE)) + 64
    bench = Bench(cfg, seed, pages, n_req, 4096, chunk)
    engine = bench.engine
    lens = torch.randint(128, 3073, (n_req,), generator=bench.gen).tolist()

    def job():
        prompts = [bench.prompts(1, n)[0] for n in lens]
        engine.step_log = []
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = engine.generate(prompts, SamplingParams(), new)
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        log, engine.step_log = engine.step_log, None
        engine.take_completed()
        assert all(len(g) == new for g in out)
        return seconds, log

    job()                                           # untimed: records the decode graphs, sizes every buffer
    before = engine.inspect()["scheduler"]
    ahead_before = engine.steps_launched_ahead
    engine.runner.set_device_timing("graph")        # two events around every step: device time beside wall time
    with ClockSampler() as clocks:
        seconds, log = job()
    after = engine.inspect()["scheduler"]
    torch.cuda.synchronize()
    step_ms = [a.elapsed_time(b) for _, a, b in engine.runner.timer._steps]
    engine.runner.set_device_timing("off")
    kinds = {"mixed": [0, 0.0, 0], "decode_only": [0, 0.0, 0], "prompt_only": [0, 0.0, 0]}
    if len(step_ms) == len(log):
        for s, ms in zip(log, step_ms):
            k = "decode_only" if s["single_token_seqs"] == s["seqs"] else "mixed" if s["single_token_seqs"] else "prompt_only"
            kinds[k][0] += 1; kinds[k][1] += ms; kinds[k][2] += s["tokens"]
    nums, pk = bench.nums, bench.pk
    roof_s = 0.0
    for s in log:
        t_flop = step_flops(nums, s["tokens"], s["logit_rows"], s["pairs"]) / (pk["bf16_tflops"] * 1e12)
        t_byte = (bench.weight_bytes + s["keys"] * nums["kv_bytes_per_token"]) / (pk["hbm_gbs"] * 1e9)
        roof_s += max(t_flop, t_byte)
    steps = len(log)
    mixed = sum(1 for s in log if 0 < s["single_token_seqs"] < s["seqs"])
    decode_only = sum(1 for s in log if s["single_token_seqs"] == s["seqs"])
    generated, prompt_tokens = n_req * new, sum(lens)
    return {
        "metric": "Qwen3-14B-sized bf16 mixed batch: generated tok/s through Engine.generate",
        "value": round(generated / seconds, 2), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": 1,
        "ms_per_step": round(1e3 * seconds / steps, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random-init weights (seed 3), prompt lengths uniform in [128, 3072], token ids uniform in [0, vocab)",
        "config": flat_config("Qwen3-14B sizes", cfg, requests=n_req, prefill_chunk_tokens=chunk, max_new_tokens=new,
                              seq_len=4096, prompt_tokens=prompt_tokens, peaks=pk["source"]),
        "e2e": {"value": round(generated / seconds, 2), "unit": "tokens/s", "seconds": round(seconds, 4),
                "all_tokens_per_s": round((generated + prompt_tokens) / seconds, 1)},
        "composition": {"steps": steps, "mixed_steps": mixed, "decode_only_steps": decode_only,
                        "prompt_only_steps": steps - mixed - decode_only,
                        "mean_tokens_per_step": round(sum(s["tokens"] for s in log) / steps, 1),
                        "mean_seqs_per_step": round(sum(s["seqs"] for s in log) / steps, 1),
                        "preemptions": after["preemptions"] - before["preemptions"],
                        "steps_launched_ahead": engine.steps_launched_ahead - ahead_before},
        "device_time": {"seconds_on_device": round(sum(step_ms) / 1e3, 4), "seconds_wall": round(seconds, 4),
                        "by_step_kind": {k: {"steps": v[0], "ms_mean": round(v[1] / max(v[0], 1), 3), "tokens_mean": round(v[2] / max(v[0], 1), 1)}
                                         for k, v in kinds.items()}},
        "roofline": {"bound": "per step: the slower of flops / bf16 peak and bytes / HBM", "seconds": round(roof_s, 4),
                     "frac": round(roof_s / seconds, 4), "peak_tflops": pk["bf16_tflops"], "peak_gbs": pk["hbm_gbs"]},
        "clocks": clocks.summary(),
        **({"breakdown": {"mixed": bench.breakdown_mixed(24, 1536, 384)}} if args.breakdown else {}),
    }


def run_32b_long(args) -> dict:
    """Decode at batch 1 and 16 after 8,192-token prompts: long paged decode attention."""
    cfg = dict(QWEN3_32B, num_hidden_layers=args.layers if args.layers != FULL_LAYERS else 64)
    prompt_len, chunk, seed = 8192, 2048, 4
    steps = min(args.steps, 64)
    tokens_per_seq = prompt_len + args.warmup + steps + 64
    pages = 16 * (-(-tokens_per_seq // PAGE)) + 256
    bench = Bench(cfg, seed, pages, 16, 16384, chunk)
    points, rooflines = {}, {}
    with ClockSampler() as clocks:
        for b_ in (16, 1):
            v, ms, kernels, ctx = bench.decode_device(b_, steps, args.warmup, f"l{b_}_", prompt_len)
            points[f"decode_b{b_}"] = {"value": round(v, 2), "ms_per_step": round(ms, 4), "kernels_per_step": kernels}
            rooflines[f"decode_b{b_}"] = bench.decode_roofline(b_, ctx, ms)
    result = {
        "metric": "Qwen3-32B-sized bf16 decode tok/s after 8,192-token prompts", "value": points["decode_b16"]["value"],
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
        "ms_per_step": points["decode_b16"]["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random-init weights (seed 4), token ids uniform in [0, vocab)",
        "config": flat_config("Qwen3-32B sizes", cfg, global_batch=16, seq_len=16384, prompt_len=prompt_len,
                              layers_full=64, prefill_chunk_tokens=chunk, peaks=bench.pk["source"]),
        "points": points, "roofline": rooflines["decode_b16"], "rooflines": rooflines, "clocks": clocks.summary(),
    }
    if not args.no_points:
        result["prefill"] = bench.prefill_timed(prompt_len, 1, 3)
    if args.breakdown:
        result["breakdown"] = bench.breakdown(16, prompt_len, chunk)
    return result


def run_kernels(args) -> dict:
    """Kernels alone (CUDA events around 20 launches after 3; weights rotate over four copies
    so that nothing stays in L2)."""
    import math
    import torch
    from inferloop_b200.csrc import ops
    from inferloop_b200.parts import Workspace
    cfg = {"8b": QWEN3_8B, "14b-mixed": QWEN3_14B, "32b-long": QWEN3_32B}[args.config]
    nq, nkv, d, H, I = (cfg[k] for k in ("num_attention_heads", "num_key_value_heads", "head_dim", "hidden_size", "intermediate_size"))
    bf = torch.bfloat16

    def timed(f, n=20):
        for _ in range(3):
            f()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            f()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n * 1e3            # microseconds

    class Step:
        pass
    ws = Workspace(torch.device("cuda:0"))
    attention = {}
    # whole prompts, then a portion of 512 tokens behind 3,584 cached ones, its pages in order and scattered over the pool
    cases = [(f"prefill_{T}", T, 0, False) for T in (512, 1024, 2048, 4096, 8192)]
    cases += [("portion_512_after_3584", 512, 3584, False), ("portion_512_after_3584_pages_scattered", 512, 3584, True)]
    for name, T, start, scattered in cases if args.kernels in ("all", "attention") else ():
        n_pages = (start + T) // PAGE
        q = torch.randn(T, nq * d, device="cuda").to(bf)
        out = torch.empty_like(q)
        kc = torch.randn(n_pages + 4, nkv, PAGE, d, device="cuda").to(bf)
        vc = torch.randn_like(kc)
        st = Step()
        st.positions = torch.arange(start, start + T, dtype=torch.int32, device="cuda")
        st.seq_of_token = torch.zeros(T, dtype=torch.int32, device="cuda")
        st.cu_q = torch.tensor([0, T], dtype=torch.int32, device="cuda")
        st.h_q_len, st.h_kv_len, st.n_seqs, st.decode_only = [T], [start + T], 1, False
        order = torch.randperm(n_pages) if scattered else torch.arange(n_pages)
        table = order.to(torch.int32).cuda().view(1, -1).contiguous()
        us = timed(lambda: ops.attention(q, out, kc, vc, st, table, 0, 1 / math.sqrt(d), nq, nkv, d, workspace=ws))
        flops = 4.0 * nq * d * (T * start + T * (T + 1) / 2)
        attention[name] = {"us": round(us, 1), "tflops": round(flops / us / 1e6, 1)}
    products = {}
    shapes = [("qkv", (nq + 2 * nkv) * d, H, {}), ("o", H, nq * d, {"accumulate": True}),
              ("gate_up", 2 * I, H, {"swiglu": True}), ("down", H, I, {"accumulate": True})]
    for M in (8, 64, 128, 256, 512, 2048) if args.kernels in ("all", "products") else ():
        for name, N, K, kw in shapes:
            a = torch.randn(M, K, device="cuda").to(bf)
            weights = [torch.randn(N, K, device="cuda").to(bf) * 0.02 for _ in range(4)]
            n_out = N // 2 if kw.get("swiglu") else N
            out = torch.zeros(M, n_out, device="cuda", dtype=torch.float32 if kw.get("accumulate") else bf)
            plain = torch.empty(M, N, device="cuda", dtype=bf)
            turn = [0]

            def ours():
                ops.gemm_tc(a, weights[turn[0] % 4], out, None, **kw)
                turn[0] += 1

            def library():
                torch.matmul(a, weights[turn[0] % 4].T, out=plain)
                turn[0] += 1
            t_ours, t_lib = timed(ours), timed(library)
            products[f"{name}_m{M}"] = {"us": round(t_ours, 1), "tflops": round(2.0 * M * N * K / t_ours / 1e6, 1),
                                        "weights_gbs": round(2.0 * N * K / t_ours / 1e3, 1),
                                        "torch_matmul_us": round(t_lib, 1)}
            del weights
    ops.check_device_errors()
    return {"metric": "kernels alone", "config": flat_config(args.config, cfg), "attention": attention, "products": products,
            "peaks": peaks()}


def run_further(args) -> dict:
    """Further sizes at the 8B layer sizes: decode at batches 16 to 256 (1,024-token prompts),
    a prompt of 32,768 tokens in portions of 2,048 and of 8,192, and the 32-bit path (four
    layers: 512-token prompts and decode at batch 8)."""
    import torch
    from inferloop_b200.engine import StepEntry
    from inferloop_b200.engine.engine import Engine
    out = {"metric": "further sizes, Qwen3-8B layer sizes", "decode": {}, "prefill_32768": {}, "float32_4_layers": {}, "peaks": peaks()}
    cfg = dict(QWEN3_8B, num_hidden_layers=args.layers)
    max_batch = 256
    bench = Bench(cfg, SEED, max_batch * (-(-(PROMPT_LEN + 128) // PAGE)) + 256, max_batch, 4096, PREFILL_LEN)
    for batch in (16, 32, 128, 256):
        value, ms, kernels, ctx = bench.decode_device(batch, 32, 4, f"f{batch}_", PROMPT_LEN)
        out["decode"][f"b{batch}"] = {"value": round(value, 1), "ms_per_step": round(ms, 3),
                                      "roofline_frac": bench.decode_roofline(batch, ctx, ms)["frac"]}
    del bench
    torch.cuda.empty_cache()
    length = 32768
    long_cfg = dict(cfg, max_position_embeddings=length + 4096)
    for chunk in (2048, 8192):
        bench = Bench(long_cfg, SEED, (length + 4096) // PAGE + 64, 2, length + 1024, chunk)
        r = bench.prefill_timed(length, 1, 3)
        out["prefill_32768"][f"portions_of_{chunk}"] = {k: r[k] for k in ("value", "ms", "frac")}
        del bench
        torch.cuda.empty_cache()
    cfg4 = dict(QWEN3_8B, num_hidden_layers=4)
    engine = Engine(cfg4, dtype="float32", device=0, block_size=PAGE, num_gpu_blocks_override=8 * 40 + 64, max_num_seqs=8,
                    max_model_len=2048, prefill_chunk_tokens=512, max_num_batched_tokens=520, random_weights_seed=SEED)
    runner = engine.runner
    ids = [f"x{i}" for i in range(8)]
    toks = torch.randint(0, cfg4["vocab_size"], (8, 512), generator=torch.Generator().manual_seed(1)).tolist()
    runner.step([StepEntry("warm", toks[0], [511])], draw_greedy=True)
    runner.end("warm")
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for rid, t in zip(ids, toks):
        runner.step([StepEntry(rid, t, [511])], draw_greedy=True)
    b.record()
    torch.cuda.synchronize()
    out["float32_4_layers"]["prefill_512_ms"] = round(a.elapsed_time(b) / 8, 2)
    entries = [StepEntry(rid, [1], [0]) for rid in ids]
    for _ in range(3):
        runner.step(entries, draw_greedy=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(20):
        runner.step(entries, draw_greedy=True)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / 20
    out["float32_4_layers"]["decode_b8_ms_per_step"] = round(ms, 3)
    out["float32_4_layers"]["weights_gbs"] = round(runner.model.weight_bytes() / (ms / 1e3) / 1e9, 1)
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="8b", choices=["8b", "14b-mixed", "32b-long"])
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers (named in config) to save time")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 / prefill side measurements")
    ap.add_argument("--breakdown", action="store_true", help="add the per-op-class share of device time")
    ap.add_argument("--further", action="store_true", help="further sizes: batches to 256, a 32,768-token prompt, the 32-bit path")
    ap.add_argument("--kernels", nargs="?", const="all", default=None, choices=["all", "attention", "products"],
                    help="time kernels alone at the layer sizes of --config")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "pip: the reference checkout 'is not installable: neither setup.py nor pyproject.toml found' (a Rust workspace; no cargo/rustc "
                          "on this machine; it has no Python API)"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.kernels:
        print(json.dumps(run_kernels(args)))
        return 0
    if args.further:
        print(json.dumps(run_further(args)))
        return 0
    result = {"8b": run_8b, "14b-mixed": run_14b_mixed, "32b-long": run_32b_long}[args.config](args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
