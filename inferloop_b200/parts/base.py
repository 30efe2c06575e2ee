"""Interfaces of the parts a layer is put together from.

A part is built from a :class:`PartSpec` (its sizes and constants), a
:class:`BuildContext` (compute dtype, device, scratch buffers) and the tensor-name
prefix it lives under.  It declares the tensors it needs by name, is handed them once,
and from then on only runs.  No part knows which model it is in: everything
model-specific reaches it through its spec.

  Norm              forward(x32, out)                       rows of x32 -> rows of out
  PositionEncoding  table(step) -> tensor | None            per-token data for a mixer
  Mixer             cache_needs(); forward(x, residual, step, cache)    residual += mix(x)
  FeedForward       forward(x, residual, step)                           residual += ffn(x)
  Block             cache_needs(); forward(hidden, step, cache)          hidden updated in place
  LogitsPost        forward(logits)                                      logits mapped in place

`hidden` / `residual` is the 32-bit residual stream [tokens, hidden]; `x` is a normed
copy in the compute dtype.  `step` is the :class:`~inferloop_b200.engine.batch.StepContext`
of the running batch; `cache` is the :class:`~inferloop_b200.cache.manager.LayerCache`
of the layer whose cache this run-order entry uses.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..config.spec import PartSpec
from ..weights.decl import WeightDecl


class Workspace:
    """Named scratch buffers that live as long as the model.  A buffer is reused by
    every layer that asks for the same tag; it only ever grows, so addresses are stable
    once the largest batch has been seen (or :meth:`reserve` was called)."""

    def __init__(self, device: Optional[torch.device]) -> None:
        self.device = device
        self._buffers: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self.generation = 0   # bumped whenever a buffer is reallocated

    def buffer(self, tag: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = (tag, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self.generation += 1
        return buf[:n].view(*shape)

    def zeroed(self, tag: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        """Like :meth:`buffer`, but zero when (re)allocated.  For counters that kernels
        leave at zero after every launch: the zero is written once, not per call."""
        n = 1
        for s in shape:
            n *= int(s)
        key = (tag, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.zeros(max(n, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self.generation += 1
        return buf[:n].view(*shape)

    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


@dataclass
class BuildContext:
    dtype: torch.dtype                       # compute dtype: bfloat16 or float32
    device: Optional[torch.device]           # None while only declaring weights
    workspace: Workspace
    cache_dtype: Optional[torch.dtype] = None

    def __post_init__(self) -> None:
        if self.cache_dtype is None:
            self.cache_dtype = self.dtype


@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every token, in pages.  Layers whose needs compare equal share
    one page group (one pool, one block table per request)."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None     # None: all keys are kept; n: only the last n are read


@dataclass(frozen=True)
class SlotStateNeed:
    """State of fixed size per request (independent of its length), zeroed at start."""
    name: str
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class CacheNeeds:
    paged: Optional[PagedKVNeed] = None
    slots: Tuple[SlotStateNeed, ...] = ()


class Part:
    # True when forward() only launches kernels that read the batch from device memory,
    # so that a recorded launch sequence can be replayed for another batch of the same
    # shape.  A part that loops over host-side batch facts must leave this False.
    graph_safe = False

    def __init__(self, spec: PartSpec, ctx: BuildContext, prefix: str = "") -> None:
        self.spec = spec
        self.ctx = ctx
        self.prefix = prefix

    def declare_weights(self) -> List[WeightDecl]:
        return []

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Take the declared tensors (keys are the declared names)."""

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds()

    def scratch_bytes(self, tokens: int) -> int:
        """Bytes of workspace buffers a step of `tokens` tokens makes this part ask for (an
        estimate from its sizes; the engine reserves this much beside the cache)."""
        return 0


class Norm(Part):
    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    def table(self, step) -> Optional[torch.Tensor]:
        raise NotImplementedError


class Mixer(Part):
    def forward(self, x: torch.Tensor, residual: torch.Tensor, step, cache) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, residual: torch.Tensor, step) -> None:
        raise NotImplementedError


class Block(Part):
    def forward(self, hidden: torch.Tensor, step, cache) -> None:
        raise NotImplementedError


class LogitsPost(Part):
    """Maps the 32-bit logits [rows, vocab] in place, after the output matrix."""

    def forward(self, logits: torch.Tensor) -> None:
        raise NotImplementedError
