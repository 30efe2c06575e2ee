"""Bind a model's declared tensors to the tensors of a folder, by name.

Reference behaviour kept: the weight prefix is the first of the architecture's
candidates under which the anchor tensor (the token table) exists
(crates/model/package/src/storage/package.rs:231-237); every declared tensor is checked
for presence, shape and a floating dtype (package.rs:249-261); non-finite values are
refused (storage/safetensors.rs:400-402).  Departure: all problems -- missing,
unexpected, wrongly shaped -- are collected into ONE error instead of stopping at the
first, and unexpected tensors are part of that error unless `allow_unexpected` is set
(the reference lists them as ignored, package.rs:281-285).
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import torch

from .decl import WeightDecl
from .safetensors_io import TensorSource

_FLOAT = ("F32", "BF16", "F16", "F64")
_INT = ("I64", "I32", "I16", "I8", "U8")


class WeightError(ValueError):
    """Lists every missing, unexpected and wrongly shaped tensor at once."""

    def __init__(self, where: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_dtype: Sequence[Tuple[str, str]] = (), other: Sequence[str] = ()) -> None:
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        self.other = list(other)
        lines = [f"{where}: weights do not match the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: expected {list(e)}, found {list(f)}" for n, e, f in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtype ({len(self.wrong_dtype)}): " + "; ".join(
                f"{n}: {d}" for n, d in self.wrong_dtype))
        for o in self.other:
            lines.append("  " + o)
        super().__init__("\n".join(lines))


def resolve_prefix(names: Iterable[str], prefixes: Sequence[str], anchor: str) -> Optional[str]:
    present = set(names)
    for p in prefixes:
        if p + anchor in present:
            return p
    return None


def target_dtype(role: str, compute_dtype: torch.dtype) -> torch.dtype:
    if role in ("matrix", "table"):
        return compute_dtype
    if role == "vector":
        return torch.float32
    if role == "int":
        return torch.int32
    raise ValueError(f"unknown weight role {role!r}")


def load_weights(folder: str, decls: Sequence[WeightDecl], prefixes: Sequence[str],
                 anchor: str, compute_dtype: torch.dtype, device: torch.device | str,
                 allow_unexpected: bool = False,
                 progress: Callable[[str], None] | None = None) -> Tuple[Dict[str, torch.Tensor], List[str]]:
    """Return ({declared name: tensor on device}, ignored tensor names).

    Declared names are prefix-relative (or root names); the returned dict is keyed by
    those same declared names, so the model never sees the file's prefix."""
    source = TensorSource(folder)
    try:
        stored = source.names()
        prefix = resolve_prefix(stored, prefixes, anchor)
        if prefix is None:
            raise WeightError(folder, [p + anchor for p in prefixes][-1:], [], [], other=[
                f"anchor tensor {anchor!r} not found under any of the prefixes {list(prefixes)}"])
        full = {(d.name if d.root else prefix + d.name): d for d in decls}
        missing = [n for n in full if n not in source.where]
        unexpected = sorted(n for n in stored if n not in full)
        wrong_shape, wrong_dtype = [], []
        for n, d in full.items():
            if n in source.where:
                e = source.entry(n)
                if tuple(e.shape) != tuple(d.shape):
                    wrong_shape.append((n, tuple(d.shape), tuple(e.shape)))
                ok = _INT if d.role == "int" else _FLOAT
                if e.dtype not in ok:
                    wrong_dtype.append((n, f"stored as {e.dtype}, need one of {list(ok)}"))
        if missing or wrong_shape or wrong_dtype or (unexpected and not allow_unexpected):
            raise WeightError(folder, missing, unexpected, wrong_shape, wrong_dtype)
        out: Dict[str, torch.Tensor] = {}
        nonfinite: List[str] = []
        for i, (n, d) in enumerate(full.items()):
            t = source.tensor(n)
            want = target_dtype(d.role, compute_dtype)
            dev = t.to(device=device, non_blocking=False)
            if dev.dtype != want:
                dev = dev.to(want)
            elif dev.data_ptr() == t.data_ptr():
                dev = dev.clone()   # never hand out a view of the read-only mapping
            if d.role != "int" and not bool(torch.isfinite(dev).all()):
                nonfinite.append(n)
            out[d.name] = dev
            if progress is not None and (i % 64 == 0):
                progress(f"loaded {i + 1}/{len(full)} tensors")
        if nonfinite:
            raise WeightError(folder, [], [], [], other=[
                "non-finite values in: " + ", ".join(nonfinite)])
        return out, unexpected
    finally:
        source.close()
