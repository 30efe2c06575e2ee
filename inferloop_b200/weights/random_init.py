"""Seeded random weights: tensors keyed by (seed, tensor name), so the values of one
tensor do not depend on the order in which tensors are made or on which other tensors
exist.  Distributions: matrices, tables and biases N(0, 0.02); norm weights
1 + N(0, 0.1), from a counter-based generator of this module that gives the same bits on
the CPU and on a CUDA device.  The reference has no such mode in the product; its probe script
(tools/bench/model-probe.py:122-131) writes N(0, 0.02) everywhere, and its golden
exporter (tools/fixtures/export-qwen-golden.py:63-72) moves norm weights away from 1 to
catch offset faults, which 1 + N(0, 0.1) does too.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Mapping, Sequence

import torch

from .decl import WeightDecl
from .loader import target_dtype
from .safetensors_io import write_safetensors


def tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{int(seed)}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


# ---------------------------------------------------------------- the generator
# Element i of a tensor is a function of (seed, tensor name, i) alone, computed with integer
# arithmetic and IEEE multiply/add only, so the CPU and a CUDA device produce the same bits:
#   h = splitmix64 finaliser of (key + (i + 1) * 0x9e3779b97f4a7c15)     64 random bits
#   cell = top 16 bits, f = next 24 bits as a fraction in (-1/2, 1/2)
#   x = Q[cell] + f * W[cell]
# where Q[k] is the standard normal quantile at (k + 1/2) / 65536 and W[k] the width of that
# cell: the normal density approximated by 65,536 cells of equal probability, uniform inside
# a cell, |x| < 4.6.  The table is made once on the host with Python's own inverse normal
# CDF (plain double arithmetic, the same on every machine) and copied to the device.
_GOLDEN = 0x9E3779B97F4A7C15 - (1 << 64)
_C1 = 0xBF58476D1CE4E5B9 - (1 << 64)
_C2 = 0x94D049BB133111EB - (1 << 64)
_CELLS = 1 << 16
_CHUNK = 1 << 25                 # elements made at a time (bounds the temporaries)
_TABLES: Dict[str, tuple] = {}


def _quantile_tables(device) -> tuple:
    key = str(device)
    if key not in _TABLES:
        if "cpu" not in _TABLES:
            from statistics import NormalDist
            nd = NormalDist()
            q = [nd.inv_cdf((k + 0.5) / _CELLS) for k in range(_CELLS)]
            w = [q[1] - q[0]] + [(q[k + 1] - q[k - 1]) / 2 for k in range(1, _CELLS - 1)] + [q[-1] - q[-2]]
            _TABLES["cpu"] = (torch.tensor(q, dtype=torch.float64), torch.tensor(w, dtype=torch.float64))
        _TABLES[key] = tuple(t.to(device) for t in _TABLES["cpu"])
    return _TABLES[key]


def _lsr(x: torch.Tensor, s: int) -> torch.Tensor:
    """Logical shift right of 64-bit words held as int64."""
    return (x >> s) & ((1 << (64 - s)) - 1)


def standard_normal(key: int, count: int, device) -> torch.Tensor:
    """`count` float32 values of the stream `key` (see above), the same on every device."""
    q, w = _quantile_tables(device)
    out = torch.empty(count, dtype=torch.float32, device=device)
    key = int(key) & ((1 << 63) - 1)
    for start in range(0, count, _CHUNK):
        n = min(_CHUNK, count - start)
        x = torch.arange(start + 1, start + 1 + n, dtype=torch.int64, device=device)
        x = x * _GOLDEN + key                    # wraps modulo 2^64
        x = (x ^ _lsr(x, 30)) * _C1
        x = (x ^ _lsr(x, 27)) * _C2
        x = x ^ _lsr(x, 31)
        cell = _lsr(x, 48)
        f = ((_lsr(x, 24) & 0xFFFFFF).to(torch.float64) + 0.5) * (1.0 / (1 << 24)) - 0.5
        v = f * w[cell]                          # product rounded, then the sum: no fused multiply-add
        v = v + q[cell]
        out[start:start + n] = v.to(torch.float32)
    return out


def random_tensor(decl: WeightDecl, seed: int, dtype: torch.dtype,
                  device: torch.device | str = "cpu") -> torch.Tensor:
    """The tensor `decl` names under `seed`, drawn in float32 and rounded to `dtype`; the
    same values whatever the device, so a model made on the GPU equals the folder written
    with the same seed."""
    if decl.role == "int":
        raise ValueError("integer tables have no random initialiser")
    if decl.init == "zeros":
        return torch.zeros(decl.shape, dtype=dtype, device=device)
    if decl.init not in ("normal", "bias", "norm"):
        raise ValueError(f"unknown initialiser {decl.init!r}")
    count = 1
    for n in decl.shape:
        count *= int(n)
    t = standard_normal(tensor_seed(seed, decl.name), count, device).view(tuple(decl.shape))
    if decl.init == "norm":
        t.mul_(0.1).add_(1.0)
    else:
        t.mul_(0.02)
    return t.to(dtype)


def random_weights(decls: Sequence[WeightDecl], seed: int, compute_dtype: torch.dtype,
                   device: torch.device | str) -> Dict[str, torch.Tensor]:
    """All declared tensors, made on `device` in the dtype their role asks for."""
    return {d.name: random_tensor(d, seed, target_dtype(d.role, compute_dtype), device)
            for d in decls}


def write_random_model(folder: str, config: Mapping[str, Any], seed: int,
                       dtype: torch.dtype = torch.float32, prefix: str = "model.",
                       registry=None) -> str:
    """Write `config.json` and `model.safetensors` for the architecture that `config`
    names.  Every tensor, norm weights and biases included, is stored in `dtype`."""
    from ..config.registry import read_model_config
    from ..models.decoder import declare_weights

    text = json.dumps(dict(config), indent=2)
    _, _, spec = read_model_config(text, registry)
    os.makedirs(folder, exist_ok=True)
    decls = declare_weights(spec)

    def items():
        for d in decls:
            name = d.name if d.root else prefix + d.name
            yield name, random_tensor(d, seed, dtype, "cpu")

    write_safetensors(os.path.join(folder, "model.safetensors"), list(items()),
                      metadata={"format": "pt", "seed": str(seed)})
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as fh:
        fh.write(text + "\n")
    return folder
