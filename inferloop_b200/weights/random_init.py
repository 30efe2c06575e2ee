"""Seeded random weights: tensors keyed by (seed, tensor name), so the values of one
tensor do not depend on the order in which tensors are made or on which other tensors
exist.  Distributions: matrices, tables and biases N(0, 0.02); norm weights
1 + N(0, 0.1).  The reference has no such mode in the product; its probe script
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


def random_tensor(decl: WeightDecl, seed: int, dtype: torch.dtype,
                  device: torch.device | str = "cpu") -> torch.Tensor:
    """Values are drawn in float32 by a generator on `device`, then rounded to `dtype`.
    CPU and CUDA generators give different streams: a model written to a folder on the
    CPU is the one to compare implementations with."""
    if decl.role == "int":
        raise ValueError("integer tables have no random initialiser")
    g = torch.Generator(device=device)
    g.manual_seed(tensor_seed(seed, decl.name))
    if decl.init == "zeros":
        t = torch.zeros(decl.shape, dtype=torch.float32, device=device)
    else:
        t = torch.empty(decl.shape, dtype=torch.float32, device=device)
        t.normal_(0.0, 1.0, generator=g)
        if decl.init == "normal" or decl.init == "bias":
            t.mul_(0.02)
        elif decl.init == "norm":
            t.mul_(0.1).add_(1.0)
        else:
            raise ValueError(f"unknown initialiser {decl.init!r}")
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
