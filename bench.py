#!/usr/bin/env python3
"""Headline measurement: Qwen3-8B-sized random bf16 model, decode tokens per second.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]

One JSON line on stdout.  A "step" is one decode step of the whole batch.
  value     decoded tokens per second of K steps run back to back on the device (each
            step's arg-max feeds the next step there), timed with CUDA events;
  e2e       the same through the Python entry point (`Engine.step`): host token ids in,
            host token ids out, every step with its host->device copy of the step's
            arrays from pinned memory and its device->host read of the drawn ids;
  prefill   one 2,048-token prompt to its last logits;
  roofline  bytes a decode step must read (every weight once + the cache of the live
            requests) / its time, against the measured copy bandwidth;
  points    decode at batch 1 and 64.
Peaks come from MEASURED_PEAKS.json beside this file when present, else the fallback
figures 6.65 TB/s and 1.59 PFLOP/s.  Weights (15 GB) exceed L2 (126 MB), so every step
reads them from HBM: no L2 flush is needed between timed steps.
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

# BASELINE.json configs[2]: Qwen3-8B layer sizes
QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
    vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, attention_bias=False,
    tie_word_embeddings=False, max_position_embeddings=4096, hidden_act="silu")
FULL_LAYERS = 36
SEED = 2
PROMPT_LEN = 1024
PREFILL_LEN = 2048
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
            "attn_flops_per_pair": 4 * nq * d * L}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers (named in config) to save time")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 / prefill side measurements")
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

    import torch
    from inferloop_b200.csrc import ops
    from inferloop_b200.engine import StepEntry
    from inferloop_b200.engine.engine import Engine
    from inferloop_b200.sampling import SamplingParams

    dev = torch.device("cuda:0")
    cfg = dict(QWEN3_8B, num_hidden_layers=args.layers)
    nums = model_numbers(cfg)
    pk = peaks()
    max_batch = max(64, args.batch)
    tokens_per_seq = PROMPT_LEN + args.warmup + args.steps + 64
    pages = max_batch * (-(-tokens_per_seq // PAGE)) + 256
    t0 = time.time()
    engine = Engine(cfg, dtype="bfloat16", device=0, block_size=PAGE, num_gpu_blocks_override=pages,
                    max_num_seqs=max_batch, max_model_len=4096, prefill_chunk_tokens=PREFILL_LEN,
                    max_num_batched_tokens=PREFILL_LEN + max_batch, random_weights_seed=SEED)
    runner = engine.runner
    print(f"[bench] model ready in {time.time() - t0:.1f} s, weights {runner.model.weight_bytes() / 1e9:.2f} GB",
          file=sys.stderr, flush=True)
    gen = torch.Generator().manual_seed(SEED)

    def prompts(n, length):
        return torch.randint(0, cfg["vocab_size"], (n, length), generator=gen).tolist()

    def prefill(ids, toks, chunk=PREFILL_LEN):
        last = {}
        for rid, t in zip(ids, toks):
            for i in range(0, len(t), chunk):
                part = t[i:i + chunk]
                logits, drawn = runner.step([StepEntry(rid, part, [len(part) - 1])], draw_greedy=True)
            last[rid] = int(drawn.ids[0].item())
        return last

    def decode_device(batch, steps, warmup, tag):
        """K decode steps back to back on the device; returns (tokens/s, ms/step, kernels/step, mean ctx)."""
        ids = [f"{tag}{i}" for i in range(batch)]
        last = prefill(ids, prompts(batch, PROMPT_LEN))
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

    # ---------------------------------------------------------------- headline: device-timed decode
    with ClockSampler() as clocks:
        value, ms_per_step, kernels, mean_ctx = decode_device(args.batch, args.steps, args.warmup, "d")
    clock_info = clocks.summary()
    weight_bytes = runner.model.weight_bytes()
    step_bytes = weight_bytes + args.batch * mean_ctx * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9

    # ---------------------------------------------------------------- end to end through Engine.step
    e2e_prompts = prompts(args.batch, PROMPT_LEN)
    for p in e2e_prompts:
        engine.submit(p, SamplingParams(), max_new_tokens=args.warmup + args.steps + 32)
    while any(engine.runner.cache.length(r.id) < PROMPT_LEN for r in engine.scheduler.running) \
            or engine.scheduler.waiting:
        engine.step()
    for _ in range(args.warmup):
        engine.step()
    torch.cuda.synchronize()
    h2d = d2h = 0
    t_start = time.perf_counter()
    for _ in range(args.steps):
        outs = engine.step()
        h2d += runner.stager.bytes_last
        d2h += 4 * len(outs)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t_start
    e2e_value = args.batch * args.steps / e2e_s
    while not engine.is_idle():
        engine.step()

    result = {
        "metric": "Qwen3-8B bf16 decode tok/s", "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random-init weights (seed 2), token ids uniform in [0, vocab)",
        "config": {"model": "Qwen3-8B sizes", "global_batch": args.batch, "seq_len": 4096,
                   "prompt_len": PROMPT_LEN, "parallelism": "1 GPU", "layers": args.layers,
                   "layers_full": FULL_LAYERS, "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "kv_page": PAGE,
                   "kv_dtype": "bf16", "sampling": "greedy", "l2": "inputs larger than L2 (weights 15 GB)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(e2e_value, 2), "unit": "tokens/s", "h2d_bytes_per_step": h2d // args.steps,
                "d2h_bytes_per_step": d2h // args.steps},
        "gpu_launches": kernels * args.steps,
        "clocks": clock_info,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }

    if not args.no_points:
        # ------------------------------------------------------------ prefill of 2,048 tokens
        toks = prompts(args.warmup + 1, PREFILL_LEN)
        for i in range(min(args.warmup, 3)):
            runner.step([StepEntry(f"pw{i}", toks[i], [PREFILL_LEN - 1])])
            runner.end(f"pw{i}")
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        runner.step([StepEntry("pf", toks[-1], [PREFILL_LEN - 1])])
        b.record()
        torch.cuda.synchronize()
        runner.end("pf")
        pms = a.elapsed_time(b)
        T = PREFILL_LEN
        flops = 2 * T * nums["layer_params"] * args.layers + 2 * nums["head_params"] \
            + nums["attn_flops_per_pair"] * T * (T + 1) / 2
        result["prefill"] = {"value": round(T / (pms / 1e3), 1), "tokens": T, "ms": round(pms, 3),
                             "frac": round(flops / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                             "peak_tflops": pk["bf16_tflops"]}      # the burst figure: the stricter of the two measured peaks
        # ------------------------------------------------------------ decode at batch 1 and 64
        points = {}
        for b_, steps in ((1, min(args.steps, 64)), (64, min(args.steps, 64))):
            v, _, _, _ = decode_device(b_, steps, args.warmup, f"p{b_}_")
            points[f"decode_b{b_}"] = round(v, 2)
        result["points"] = points
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
