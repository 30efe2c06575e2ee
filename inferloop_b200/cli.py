"""Command line in the manner of the reference's `infer`
(crates/service/cli/src/arguments.rs:17-121, commands/options.rs:46-64).

    infer run --package DIR --requests FILE      canonical requests (token ids) in, JSON out
    infer generate DIR --tokens 1,2,3 ...        one prompt from the command line
    infer inspect-model DIR                      the typed configuration and the layer list

Options shared with the reference keep its names and meanings: --device,
--block-size, --num-gpu-blocks-override, --max-num-batched-tokens, --max-model-len,
--max-output-tokens, --max-num-seqs, --gpu-memory-utilization.  `--dtype` and
`--random-weights` are this engine's own; `--device-timing off|graph|node` is the reference's
(crates/service/cli/src/arguments.rs:69-73).  Serving over HTTP is not part of it.

The requests file is the reference's (examples/generate.json): one object or a list of
    {"id": 1, "model": 1, "input": {"Sequence": {"tokens": [..]}},
     "workload": {"Generate": {"max_new_tokens": 8}}, "sampling": {...}}
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import Any, Dict, List


def _add_engine_options(p: argparse.ArgumentParser) -> None:
    p.add_argument("--device", type=int, default=0, metavar="ORDINAL")
    p.add_argument("--num-gpu-blocks-override", type=int, default=None)
    p.add_argument("--block-size", type=int, default=16)
    p.add_argument("--max-num-batched-tokens", type=int, default=None)
    p.add_argument("--max-model-len", type=int, default=None, metavar="TOKENS")
    p.add_argument("--max-output-tokens", type=int, default=None, metavar="TOKENS")
    p.add_argument("--max-num-seqs", type=int, default=64, metavar="SEQUENCES")
    p.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    p.add_argument("--device-timing", choices=["off", "graph", "node"], default="off",
                   help="device time per step (graph) or per kernel and op class (node), reported under runtime")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                   help="ignore model.safetensors; make weights from config.json and this seed")


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="infer", description=__doc__.split("\n\n")[0])
    sub = p.add_subparsers(dest="command", required=True)
    run = sub.add_parser("run", help="run canonical requests")
    run.add_argument("--requests", required=True)
    g = run.add_mutually_exclusive_group(required=True)
    g.add_argument("--package")
    g.add_argument("--model")
    _add_engine_options(run)
    gen = sub.add_parser("generate", help="generate from one prompt of token ids")
    gen.add_argument("model_path", metavar="MODEL_PATH")
    gen.add_argument("--tokens", required=True, help="comma-separated token ids")
    gen.add_argument("--max-new-tokens", type=int, default=16)
    # what is not given comes from the folder's generation_config.json / config.json
    gen.add_argument("--temperature", type=float, default=None)
    gen.add_argument("--top-k", type=int, default=None, help="0 disables the filter")
    gen.add_argument("--top-p", type=float, default=None)
    gen.add_argument("--min-p", type=float, default=None)
    gen.add_argument("--presence-penalty", type=float, default=None)
    gen.add_argument("--repetition-penalty", type=float, default=None)
    gen.add_argument("--seed", type=int, default=None)
    gen.add_argument("--eos-token", type=int, default=None)
    _add_engine_options(gen)
    ins = sub.add_parser("inspect-model", help="print the typed configuration")
    ins.add_argument("model_path", metavar="MODEL_PATH")
    wr = sub.add_parser("write-random-model", help="write config.json + model.safetensors from a config and a seed")
    wr.add_argument("--config", required=True, help="a config.json to copy the sizes from")
    wr.add_argument("--seed", type=int, required=True)
    wr.add_argument("--out", required=True)
    wr.add_argument("--dtype", choices=["bfloat16", "float32"], default="float32")
    return p


def _engine(args, folder: str):
    from .engine.engine import Engine
    model: Any = folder
    if args.random_weights is not None:
        import os
        with open(os.path.join(folder, "config.json")) as fh:
            model = json.load(fh)
    return Engine(model, dtype=args.dtype, device=args.device, block_size=args.block_size,
                  num_gpu_blocks_override=args.num_gpu_blocks_override,
                  max_num_batched_tokens=args.max_num_batched_tokens, max_model_len=args.max_model_len,
                  max_output_tokens=args.max_output_tokens, max_num_seqs=args.max_num_seqs,
                  gpu_memory_utilization=args.gpu_memory_utilization,
                  random_weights_seed=args.random_weights, device_timing=args.device_timing)


def _sampling(engine, d: Dict[str, Any]):
    """A request's sampling fields over the folder's generation defaults, field by field
    (crates/model/package/src/generation/mod.rs:68-128); unknown fields are refused."""
    return engine.generation_defaults.resolve(d)


def read_requests(path: str) -> List[Dict[str, Any]]:
    """The requests file: one request object or a list of them, each
    {"id", "input": {"Sequence": {"tokens": [...]}}, "workload": {"Generate": {"max_new_tokens": n}},
    "sampling": {...}}.  Anything else is refused with a ValueError that names the request."""
    try:
        with open(path, encoding="utf-8") as fh:
            reqs = json.load(fh)
    except RecursionError:
        raise ValueError(f"{path}: nested too deep to be a requests file") from None
    if isinstance(reqs, dict):
        reqs = [reqs]
    if not isinstance(reqs, list):
        raise ValueError(f"{path}: expected a request object or a list of them")
    out = []
    for i, r in enumerate(reqs):
        where = f"{path}: request {i}"
        if not isinstance(r, dict) or "id" not in r or isinstance(r["id"], (dict, list)):
            raise ValueError(f"{where}: needs an object with an \"id\"")
        try:
            tokens = r["input"]["Sequence"]["tokens"]
            max_new = r["workload"]["Generate"]["max_new_tokens"]
        except (KeyError, TypeError):
            raise ValueError(f"{where} ({r['id']!r}): only Sequence input with a Generate workload is served") from None
        if not isinstance(tokens, list) or not tokens or any(isinstance(t, bool) or not isinstance(t, int) for t in tokens):
            raise ValueError(f"{where} ({r['id']!r}): tokens must be a non-empty list of integers")
        if isinstance(max_new, bool) or not isinstance(max_new, int) or max_new < 1:
            raise ValueError(f"{where} ({r['id']!r}): max_new_tokens must be a positive integer")
        sampling = r.get("sampling", {})
        if sampling is None:
            sampling = {}
        if not isinstance(sampling, dict):
            raise ValueError(f"{where} ({r['id']!r}): sampling must be an object")
        out.append({"id": r["id"], "tokens": tokens, "max_new_tokens": max_new, "sampling": sampling})
    return out


def cmd_run(args) -> int:
    folder = args.package or args.model
    reqs = read_requests(args.requests)
    engine = _engine(args, folder)
    t0 = time.time()
    ids = []
    for r in reqs:
        ids.append(engine.submit(r["tokens"], _sampling(engine, r["sampling"]), r["max_new_tokens"], request_id=r["id"]))
    while not engine.is_idle():
        engine.step()
    results = []
    for i in ids:
        r = engine.result(i)
        results.append({"id": r.id, "reason": {"eos": "Eos", "length": "Length"}.get(r.finish_reason, r.finish_reason),
                        "output": {"Tokens": r.generated}, "preemptions": r.preemptions})
    print(json.dumps({"runtime": engine.inspect(), "execution": {"backend": "cuda-sm100a", "dtype": args.dtype,
                      "seconds": round(time.time() - t0, 4)}, "results": results}))
    return 0


def cmd_generate(args) -> int:
    tokens = [int(t) for t in args.tokens.replace(" ", "").split(",") if t]
    engine = _engine(args, args.model_path)
    params = _sampling(engine, {k: getattr(args, k) for k in (
        "temperature", "top_k", "top_p", "min_p", "presence_penalty", "repetition_penalty", "seed", "eos_token")})
    out = engine.generate([tokens], params, args.max_new_tokens)[0]
    print(json.dumps({"tokens": out, "reason": engine.result(0).finish_reason}))
    return 0


def cmd_inspect(args) -> int:
    import os
    from .config.registry import read_model_config
    with open(os.path.join(args.model_path, "config.json")) as fh:
        arch, cfg, spec = read_model_config(fh.read())
    print(json.dumps({"architecture": arch.name, "config": cfg.to_dict(),
                      "layers": [{"prefix": l.prefix, "block": l.block.kind, "mixer": l.mixer.kind,
                                  "feed_forward": l.feed_forward.kind, "norm": l.norm.kind,
                                  "window": l.mixer.get("window")} for l in spec.layers],
                      "run_order": [[e.layer, e.cache_of] for e in spec.run_order]}, indent=2))
    return 0


def cmd_write_random(args) -> int:
    import torch
    from .weights import write_random_model
    with open(args.config) as fh:
        config = json.load(fh)
    write_random_model(args.out, config, args.seed, torch.float32 if args.dtype == "float32" else torch.bfloat16)
    print(args.out)
    return 0


def main(argv: List[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    try:
        return {"run": cmd_run, "generate": cmd_generate, "inspect-model": cmd_inspect,
                "write-random-model": cmd_write_random}[args.command](args)
    except (ValueError, RuntimeError, OSError, RecursionError) as e:
        print(f"infer: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
