"""Shared pieces of the tests: the tiny configurations, model folders, the comparison."""
from __future__ import annotations

import json
import os
import random
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Tiny A: every size small and a power of two, tied head, no bias.
CONFIG_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=64,
    num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128,
    vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6, attention_bias=False,
    tie_word_embeddings=True, max_position_embeddings=128, hidden_act="silu")
SEED_A, PAGE_A = 0, 4

# Tiny B: differs from A in every size and option; sizes that are no power of two,
# head_dim decoupled from hidden/heads, group of 3, biases, separate output matrix.
CONFIG_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=96,
    num_attention_heads=6, num_key_value_heads=2, head_dim=32, intermediate_size=224,
    vocab_size=320, rope_theta=1000000.0, rms_norm_eps=1e-5, attention_bias=True,
    tie_word_embeddings=False, max_position_embeddings=256, hidden_act="silu")
SEED_B, PAGE_B = 1, 8

# Tiny C: a window on some layers (two page groups), partial rotation, an odd
# vocabulary, head size 48, one kv head per query head.
CONFIG_C = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=4, hidden_size=80,
    num_attention_heads=5, num_key_value_heads=5, head_dim=48, intermediate_size=176,
    vocab_size=515, rope_theta=50000.0, rms_norm_eps=3e-6, attention_bias=False,
    tie_word_embeddings=True, max_position_embeddings=256, hidden_act="silu",
    partial_rotary_factor=0.5,
    layer_types=["full_attention", "sliding_attention", "full_attention", "sliding_attention"],
    sliding_window=20)
SEED_C, PAGE_C = 5, 16

# Small D: the geometry the serving kernels are built for (head size 128, groups of four,
# 16-token pages, widths that are multiples of 64), so that the engine-level cases also run
# through the tcgen05 prefill attention, the TMA decode attention, the cluster-reduced GEMM
# and the SwiGLU epilogue, not only through their general-purpose fallbacks.
CONFIG_D = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=256,
    num_attention_heads=8, num_key_value_heads=2, head_dim=128, intermediate_size=384,
    vocab_size=1000, rope_theta=1000000.0, rms_norm_eps=1e-6, attention_bias=False,
    tie_word_embeddings=False, max_position_embeddings=2048, hidden_act="silu")
SEED_D, PAGE_D = 7, 16

# Small E: D's geometry with a window of 40 on every second layer, so that block tables whose
# leading entries were given back (-1) reach the serving kernels (tcgen05 prefill attention,
# TMA decode attention with its fused input stage) through the real ledger.
CONFIG_E = dict(CONFIG_D, num_hidden_layers=3, layer_types=["full_attention", "sliding_attention", "sliding_attention"],
                sliding_window=40, vocab_size=600, rms_norm_eps=2e-6)
SEED_E, PAGE_E = 8, 16

# Small F: groups of five query heads per kv head at head size 128 (the geometry of the
# 14B-sized serving configuration): five does not divide the 128 rows of an attention tile.
CONFIG_F = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=320,
    num_attention_heads=10, num_key_value_heads=2, head_dim=128, intermediate_size=448,
    vocab_size=777, rope_theta=500000.0, rms_norm_eps=1e-5, attention_bias=False,
    tie_word_embeddings=True, max_position_embeddings=1024, hidden_act="silu")
SEED_F, PAGE_F = 9, 16

CONFIGS = {"A": (CONFIG_A, SEED_A, PAGE_A), "B": (CONFIG_B, SEED_B, PAGE_B),
           "C": (CONFIG_C, SEED_C, PAGE_C), "D": (CONFIG_D, SEED_D, PAGE_D),
           "E": (CONFIG_E, SEED_E, PAGE_E), "F": (CONFIG_F, SEED_F, PAGE_F)}

# |x - ref| <= atol + rtol * |ref| per element, the reference's own rule and defaults
# (crates/diagnostics/quality/src/verification.rs:22-67; crates/service/cli/src/constants.rs:19-22).
F32_RTOL = 1e-5
F32_ATOL = 1e-5
# bfloat16 keeps 8 significant bits (unit roundoff 2^-9).  The plain implementation rounds
# the weights only; the engine also rounds activations wherever a matrix product reads or
# writes them, which leaves noise on the logits: measured over whole prompts of the small
# configurations, root-mean-square 0.3e-3 to 0.9e-3 of the largest reference logit and at
# most 4.3e-3 for any element.  The bounds: every element within 1e-2 of the largest
# reference logit, and the root-mean-square error of a comparison within a quarter of that.
BF16_REL_OF_MAX = 1e-2


def make_model_folder(folder: str, config: dict, seed: int, dtype=torch.float32) -> str:
    from inferloop_b200.weights import write_random_model
    return write_random_model(folder, config, seed, dtype)


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def assert_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str = "",
                 bf16_rel_of_max: float = BF16_REL_OF_MAX) -> None:
    got = got.to(torch.float64).cpu()
    ref = ref.to(torch.float64).cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err = (got - ref).abs()
    if dtype == "float32":
        bound = F32_ATOL + F32_RTOL * ref.abs()
    else:
        bound = torch.full_like(ref, bf16_rel_of_max * float(ref.abs().max()))
        rms = float(err.pow(2).mean().sqrt())
        assert rms <= 0.25 * float(bound.flatten()[0]) or err.numel() < 64, \
            f"{what}: root-mean-square error {rms:.3e} exceeds {0.25 * float(bound.flatten()[0]):.3e}"
    bad = err > bound
    if bad.any():
        idx = torch.nonzero(bad)[0].tolist()
        raise AssertionError(
            f"{what}: {int(bad.sum())} of {bad.numel()} elements differ; first at {idx}: "
            f"got {got[tuple(idx)].item():.8g}, want {ref[tuple(idx)].item():.8g}; "
            f"max error {err.max().item():.3e}, max |ref| {ref.abs().max().item():.3e}")


class Trace:
    """Builds the JSON steps of a trace and remembers which (request, position) each
    written logits row belongs to."""

    def __init__(self) -> None:
        self.steps: List[dict] = []
        self.rows: Dict[int, List[Tuple[str, int]]] = {}
        self._cursor: Dict[str, int] = {}

    def step(self, entries: Sequence[Tuple[str, Sequence[int], Sequence[int]]], end: Sequence[str] = ()) -> int:
        n = len(self.steps)
        recs, rows = [], []
        for rid, tokens, want in entries:
            cur = self._cursor.get(rid, 0)
            recs.append({"id": rid, "tokens": list(tokens), "want": list(want)})
            rows += [(rid, cur + w) for w in want]
            self._cursor[rid] = cur + len(tokens)
        self.steps.append({"step": n, "entries": recs, "end": list(end)})
        if rows:
            self.rows[n] = rows
        for rid in end:
            self._cursor.pop(rid, None)
        return n

    def lines(self) -> str:
        return "".join(json.dumps(s) + "\n" for s in self.steps)


def run_trace_program(model_dir: str, dtype: str, trace: Trace, out_dir: str, max_tokens: int,
                      block_size: int | None = None, env: dict | None = None) -> Dict[int, np.ndarray]:
    """Run bin/trace_run as a separate program; returns {step: logits [wanted, vocab]}."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    if block_size:
        cmd += ["--block-size", str(block_size)]
    proc = subprocess.run(cmd, input=trace.lines(), capture_output=True, text=True, timeout=900, env=env)
    assert proc.returncode == 0, f"trace_run failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}"
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in trace.steps], proc.stdout
    with open(os.path.join(model_dir, "config.json")) as fh:
        vocab = json.load(fh)["vocab_size"]
    out = {}
    for step, rows in trace.rows.items():
        a = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4")
        assert a.size == len(rows) * vocab, f"step {step}: {a.size} floats for {len(rows)} rows"
        out[step] = a.reshape(len(rows), vocab)
    return out


def run_trace_inprocess(runner, trace: Trace) -> Dict[int, np.ndarray]:
    """The same steps through ModelRunner.step in this process."""
    from inferloop_b200.engine import StepEntry
    out = {}
    for s in trace.steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]
        if entries:
            logits = runner.step(entries)
            if logits.shape[0]:
                out[s["step"]] = logits.float().cpu().numpy().copy()
        for rid in s["end"]:
            if runner.is_live(rid):
                runner.end(rid)
    return out


def check_trace(outputs: Dict[int, np.ndarray], trace: Trace, ref_logits: Dict[str, torch.Tensor],
                dtype: str, what: str, bf16_rel_of_max: float = BF16_REL_OF_MAX) -> None:
    """Every written row against the plain implementation's logits of that request at
    that position."""
    for step, rows in trace.rows.items():
        got = torch.from_numpy(outputs[step])
        ref = torch.stack([ref_logits[rid][pos] for rid, pos in rows])
        assert_close(got, ref, dtype, f"{what} step {step} rows {rows[:4]}...", bf16_rel_of_max)
