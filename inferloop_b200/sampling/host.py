"""The reference's sampler, step for step, on the host
(crates/engine/workloads/src/sampling.rs).  It serves requests that ask for filters or
penalties, for which the logits row is read back; plain greedy and plain temperature
requests are served on the device (:mod:`.device`) with the same rule and the same
uniform numbers.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import numpy as np

from .params import SamplingParams

_MASK = (1 << 64) - 1


def uniform(seed: int, request: int, position: int) -> float:
    """Stateless 53-bit uniform in [0, 1) from (seed, request, position), so that a
    trajectory does not depend on batching order (sampling.rs:9-23, :197-205)."""
    x = (int(seed) + ((int(request) * 0x9E3779B97F4A7C15) & _MASK) + int(position)) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    x ^= x >> 31
    return (x >> 11) / float(1 << 53)


def request_key(request) -> int:
    """The integer a request id contributes to the draw: an int is itself, anything
    else is hashed stably (not with Python's salted hash)."""
    if isinstance(request, (int, np.integer)) and not isinstance(request, bool):
        return int(request) & _MASK
    import hashlib
    return int.from_bytes(hashlib.sha256(repr(request).encode()).digest()[:8], "little")


def total_order_keys(values: np.ndarray) -> np.ndarray:
    """Unsigned keys whose order is the total order of 32-bit floats (-0 below +0), the
    order the reference compares logits in (`f32::total_cmp`)."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    return np.where(bits & np.uint32(0x80000000), ~bits, bits | np.uint32(0x80000000))


def greedy(logits: np.ndarray) -> int:
    """Highest value in the total order, lowest index among equals; non-finite input is
    an error (sampling.rs:175-192)."""
    if logits.size == 0 or not np.isfinite(logits).all():
        raise ValueError("invalid sampling logits")
    return int(np.argmax(total_order_keys(logits)))     # numpy returns the first maximum


def sample(logits: np.ndarray, params: SamplingParams, request: int, position: int,
           prompt: Sequence[int] = (), generated: Sequence[int] = ()) -> int:
    """One token from one row of 32-bit logits (sampling.rs:113-168)."""
    logits = np.asarray(logits, dtype=np.float32)
    if params.uses_plain_greedy():
        return greedy(logits)
    if logits.size == 0 or not np.isfinite(logits).all():
        raise ValueError("invalid sampling logits")
    values = logits.copy()
    # penalties (sampling.rs:231-280): repetition over prompt + generated, presence over generated
    if params.presence_penalty != 0.0 or params.repetition_penalty != 1.0:
        vocab = values.size
        for t in list(prompt) + list(generated):
            if not (0 <= int(t) < vocab):
                raise ValueError("history token outside vocabulary")
        seen = np.zeros(vocab, dtype=bool)
        seen[np.asarray(list(prompt) + list(generated), dtype=np.int64)] = True
        gen = np.zeros(vocab, dtype=bool)
        gen[np.asarray(list(generated), dtype=np.int64)] = True
        rp = np.float32(params.repetition_penalty)
        neg = seen & (values < 0)
        pos = seen & ~(values < 0)
        values[neg] = values[neg] * rp
        values[pos] = values[pos] / rp
        values[gen] = values[gen] - np.float32(params.presence_penalty)
    # descending by value, ascending index among equals (sampling.rs:146)
    # (total order: -0 sorts below +0; a stable sort keeps equals in index order)
    order = np.argsort(~total_order_keys(values), kind="stable")
    if params.temperature == 0.0:
        return int(order[0])
    if params.top_k is not None and params.top_k < order.size:
        order = order[:params.top_k]
    cand = values[order].astype(np.float64)
    t = float(np.float32(params.temperature))
    weights = np.exp((cand - cand[0]) / t)
    # min-p keeps the leading run of weights >= min_p, at least one (sampling.rs:282-290)
    below = np.nonzero(weights < float(np.float32(params.min_p)))[0]
    keep = max(int(below[0]) if below.size else weights.size, 1)
    weights, order = weights[:keep], order[:keep]
    # The running sums below are numpy's accumulate: one addition after the other in the
    # order of the candidates, the same 64-bit sums as a loop over them.
    if params.top_p < 1.0:              # sampling.rs:291-305
        threshold = float(np.sum(weights)) * float(np.float32(params.top_p))
        reached = np.nonzero(np.add.accumulate(weights) >= threshold)[0]
        n = int(reached[0]) + 1 if reached.size else weights.size
        weights, order = weights[:n], order[:n]
    # cumulative draw over F32-rounded normalised weights (sampling.rs:210-226)
    total = float(np.add.accumulate(weights)[-1])
    u = uniform(params.seed, request, position)
    steps = np.add.accumulate((weights / total).astype(np.float32).astype(np.float64))
    crossed = np.nonzero(u < steps)[0]
    return int(order[int(crossed[0])]) if crossed.size else int(order[-1])
