"""The command line: parsing (no GPU) and a run through it (GPU)."""
import json
import os
import subprocess
import sys

import pytest

from helpers import CONFIGS, ROOT, make_model_folder, random_tokens
from inferloop_b200.cli import build_parser


def test_option_names_follow_the_reference():
    args = build_parser().parse_args([
        "run", "--package", "m", "--requests", "r.json", "--device", "0", "--block-size", "8",
        "--num-gpu-blocks-override", "32", "--max-num-batched-tokens", "64", "--max-model-len", "128",
        "--max-output-tokens", "16", "--max-num-seqs", "4", "--gpu-memory-utilization", "0.5",
        "--device-timing", "node"])
    assert (args.block_size, args.num_gpu_blocks_override, args.max_num_seqs) == (8, 32, 4)
    assert args.device_timing == "node"            # crates/service/cli/src/arguments.rs:69-73
    g = build_parser().parse_args(["generate", "m", "--tokens", "1,2,3", "--temperature", "0.7", "--seed", "4"])
    assert g.model_path == "m" and g.temperature == 0.7
    with pytest.raises(SystemExit):
        build_parser().parse_args(["run", "--requests", "r.json"])       # needs --package or --model


def test_inspect_model(tmp_path):
    d = make_model_folder(str(tmp_path / "m"), CONFIGS["C"][0], 1)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "infer"), "inspect-model", d],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    info = json.loads(out.stdout)
    assert info["architecture"] == "qwen3-dense" and [l["window"] for l in info["layers"]] == [None, 20, None, 20]


@pytest.mark.gpu
def test_run_requests_file(tmp_path):
    import plain_qwen3 as plain
    cfg, seed, page = CONFIGS["A"]
    d = make_model_folder(str(tmp_path / "m"), cfg, seed)
    prompts = [random_tokens(n, cfg["vocab_size"], n) for n in (5, 9)]
    reqs = [{"id": i + 1, "model": 1, "input": {"Sequence": {"tokens": p}},
             "workload": {"Generate": {"max_new_tokens": 6}}} for i, p in enumerate(prompts)]
    with open(tmp_path / "r.json", "w") as fh:
        json.dump(reqs, fh)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "infer"), "run", "--package", d,
                          "--requests", str(tmp_path / "r.json"), "--dtype", "float32", "--block-size", str(page),
                          "--num-gpu-blocks-override", "32", "--device-timing", "node"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    res = json.loads(out.stdout.strip().splitlines()[-1])
    timing = res["runtime"]["device_timing"]
    assert timing["mode"] == "node" and timing["steps"]["count"] == res["runtime"]["steps"]
    assert {"embedding", "norm", "attention.qkv_projection", "attention.attention", "attention.o_projection",
            "feed_forward.down", "head.output_matrix", "sampling"} <= set(timing["ops"])
    assert abs(sum(o["share"] for o in timing["ops"].values()) - 1.0) < 1e-2
    model = plain.PlainModel(d)
    for r, p in zip(res["results"], prompts):
        assert r["output"]["Tokens"] == plain.generate(model, p, 6) and r["reason"] == "Length"
    assert res["runtime"]["running"] == 0


def test_requests_file_is_checked_before_anything_is_built(tmp_path):
    """One request or a list; whatever is not a request is refused with a message that names
    it, and `main` answers with status 1 and one line instead of a traceback."""
    from inferloop_b200.cli import main, read_requests
    p = str(tmp_path / "r.json")

    def put(obj, raw=None):
        with open(p, "w") as fh:
            fh.write(raw if raw is not None else json.dumps(obj))

    good = {"id": "a", "input": {"Sequence": {"tokens": [1, 2, 3]}}, "workload": {"Generate": {"max_new_tokens": 4}}}
    put(good)
    assert read_requests(p) == [{"id": "a", "tokens": [1, 2, 3], "max_new_tokens": 4, "sampling": {}}]
    put([good, dict(good, id=2, sampling={"temperature": 0.5})])
    assert [r["id"] for r in read_requests(p)] == ["a", 2] and read_requests(p)[1]["sampling"] == {"temperature": 0.5}
    for bad, why in ((7, "request object or a list"), ([7], "needs an object"), ([{"input": {}}], "needs an object"),
                     ([dict(good, input={"Text": "hi"})], "only Sequence input"),
                     ([dict(good, workload={"Score": {}})], "only Sequence input"),
                     ([dict(good, input={"Sequence": {"tokens": []}})], "non-empty list of integers"),
                     ([dict(good, input={"Sequence": {"tokens": [1, "2"]}})], "non-empty list of integers"),
                     ([dict(good, input={"Sequence": {"tokens": [True]}})], "non-empty list of integers"),
                     ([dict(good, workload={"Generate": {"max_new_tokens": 0}})], "positive integer"),
                     ([dict(good, workload={"Generate": {"max_new_tokens": 2.5}})], "positive integer"),
                     ([dict(good, sampling=[1])], "sampling must be an object")):
        put(bad)
        with pytest.raises(ValueError, match=why):
            read_requests(p)
    for raw in ("{", "[" * 100000):
        put(None, raw)
        with pytest.raises(ValueError):
            read_requests(p)
        assert main(["run", "--package", str(tmp_path), "--requests", p]) == 1
    assert main(["run", "--package", str(tmp_path), "--requests", str(tmp_path / "missing.json")]) == 1
