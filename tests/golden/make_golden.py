"""Writes tests/golden/plain_logits.json: a few logits of the plain implementation
(tests/plain_qwen3.py) on the tiny random models A and B.

The oracle rests on the reference's formulas: 1994/inferloop is Rust (no toolchain on
this machine) and holds no Python model code, so there is nothing of its own to import or
compile on the CPU and compare with.  These numbers therefore pin the plain
implementation against accidental change; they do not come from the reference.

    python tests/golden/make_golden.py
"""
import json
import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import plain_qwen3 as plain  # noqa: E402
from helpers import CONFIGS, make_model_folder, random_tokens  # noqa: E402

out = {}
for name in ("A", "B"):
    cfg, seed, _ = CONFIGS[name]
    with tempfile.TemporaryDirectory() as tmp:
        d = make_model_folder(os.path.join(tmp, name), cfg, seed)
        toks = random_tokens(11, cfg["vocab_size"], 42)
        model = plain.PlainModel(d)
        out[name] = {"tokens": toks,
                     "last_logits_first16": model.logits(toks)[-1, :16].tolist(),
                     "greedy4": plain.generate(model, toks, 4)}
with open(os.path.join(HERE, "plain_logits.json"), "w") as fh:
    json.dump(out, fh, indent=1)
print("wrote", os.path.join(HERE, "plain_logits.json"))
