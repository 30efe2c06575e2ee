"""Trace replay: feed given token ids through a model step by step and write logits.

It samples nothing and owns nothing: it drives the same :class:`ModelRunner` (model,
step function, cache manager, kernels) that generation uses.  The reference's nearest
tools are `infer verify`, which feeds growing prefixes straight to the backend and
compares logits (crates/service/cli/src/host_quality.rs:129-223), and `infer replay`,
which re-executes recorded engine actions (crates/service/cli/src/commands/replay.rs:6-53).

Input, one JSON object per line on standard input:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, `<out>/<step>.f32` holds the logits at the
wanted places, in the order of the entries and of `want`, little-endian 32-bit floats
[wanted, vocab].  After every step a line `done <step>` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List

PAGE_TOKENS = 16


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder that receives <step>.f32")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time (each rounded up to 64)")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--block-size", type=int, default=PAGE_TOKENS, help="tokens per cache page")
    return p


def main(argv: List[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    if args.max_tokens <= 0:
        print("trace_run: --max-tokens must be positive", file=sys.stderr)
        return 2
    if args.block_size <= 0 or 64 % args.block_size != 0:
        print("trace_run: --block-size must divide 64", file=sys.stderr)
        return 2
    import numpy as np
    import torch
    from .batch import StepEntry
    from .runner import ModelRunner

    os.makedirs(args.out, exist_ok=True)
    num_pages = -(-args.max_tokens // args.block_size)
    runner = ModelRunner.from_folder(
        args.model, dtype=args.dtype, device=args.device, page_size=args.block_size,
        num_pages=num_pages, max_requests=16,
        progress=lambda m: print(f"[trace_run] {m}", file=sys.stderr, flush=True))
    for line_no, line in enumerate(sys.stdin, 1):
        line = line.strip()
        if not line:
            continue
        try:
            rec = json.loads(line)
            step_no = rec["step"]
            entries = [StepEntry(e["id"], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])])
                       for e in rec.get("entries", [])]
            ended = list(rec.get("end", []))
        except (json.JSONDecodeError, RecursionError, KeyError, TypeError, ValueError, AttributeError) as e:
            print(f"trace_run: line {line_no} is not a step ({type(e).__name__}: {e}); expected "
                  '{"step": n, "entries": [{"id": ..., "tokens": [...], "want": [...]}], "end": [...]}', file=sys.stderr)
            return 2
        if entries:
            try:
                logits = runner.step(entries)
            except ValueError as e:                 # what the step function refuses: tokens outside the vocabulary, no room, ...
                print(f"trace_run: step {step_no}: {e}", file=sys.stderr)
                return 2
            if logits.shape[0] > 0:
                host = logits.to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
                host.tofile(os.path.join(args.out, f"{step_no}.f32"))
            else:
                torch.cuda.current_stream(runner.device).synchronize()
            from ..csrc import ops
            ops.check_device_errors()
        for rid in ended:
            if runner.is_live(rid):
                runner.end(rid)
        print(f"done {step_no}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
