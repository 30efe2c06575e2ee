"""The batch of one step, as the kernels see it.

A step is a list of entries (request, its next tokens, the places whose logits are
wanted).  The reference's task is either a prompt span or one decode token
(crates/foundation/ir/src/execution.rs:85-93); here both are simply "the next tokens of
a request", of any length, so a step may hold portions of prompts beside single decoded
tokens, cut anywhere.  All tokens are laid side by side, each request's tokens
contiguous and in order (which a mixer with sequential state relies on), with per-token
position and sequence index and per-sequence offsets, lengths, slots and block tables.
All of it travels to the device as ONE int32 buffer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch


@dataclass
class StepEntry:
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()      # indices into `tokens` whose logits are wanted
    # integer inputs per token that the model's description declares (`ModelSpec.token_extras`):
    # name -> len(tokens) * width values, token by token
    extras: Optional[dict] = None


@dataclass
class Drawn:
    """Token ids a step drew on the device with their flags side by side: `pair` is int32
    [2, capacity], row 0 the arg-max of each logits row, row 1 non-zero where that row held a
    non-finite value; the first `n` columns belong to the step."""
    pair: torch.Tensor
    n: int

    @property
    def ids(self) -> torch.Tensor:
        return self.pair[0, :self.n]

    @property
    def flags(self) -> torch.Tensor:
        return self.pair[1, :self.n]


@dataclass
class StepContext:
    n_tokens: int
    n_seqs: int
    n_logit_rows: int
    # device int32 tensors
    tokens: torch.Tensor           # [T]
    positions: torch.Tensor        # [T] absolute position of each token
    seq_of_token: torch.Tensor     # [T] index of the token's sequence in this batch
    cu_q: torch.Tensor             # [S + 1] offsets of each sequence's tokens
    kv_len: torch.Tensor           # [S] tokens in the cache after this step
    slots: torch.Tensor            # [S] state slot of each sequence
    logit_rows: torch.Tensor       # [R] token rows whose logits are wanted
    block_tables: Dict[int, torch.Tensor]   # group -> [S, max_blocks]
    extras: Dict[str, torch.Tensor] = field(default_factory=dict)   # declared per-token inputs: name -> [T, width]
    # host copies, for planning launches and for parts written in Python
    requests: List[Hashable] = field(default_factory=list)
    h_q_start: List[int] = field(default_factory=list)     # first position of each sequence's tokens
    h_q_len: List[int] = field(default_factory=list)
    h_kv_len: List[int] = field(default_factory=list)
    h_slots: List[int] = field(default_factory=list)
    max_q_len: int = 0
    max_kv_len: int = 0
    decode_only: bool = False
    position_tables: Dict[object, torch.Tensor] = field(default_factory=dict)


class StepStager:
    """Pinned host memory that a step's integer arrays are packed into (by the C++ host
    library) and the one transfer that takes them to the device.  Two staging buffers
    alternate, each guarded by an event, so packing step n+1 never overwrites memory that
    step n's copy still reads."""

    def __init__(self, device: torch.device, capacity: int = 1 << 16) -> None:
        self.device = device
        self._cap = 0
        self._host: List[torch.Tensor] = []
        self._events: List[Optional[torch.cuda.Event]] = [None, None]
        self._dev: Optional[torch.Tensor] = None
        self._turn = 0
        self._grow(capacity)

    def _grow(self, capacity: int) -> None:
        self._cap = int(capacity)
        self._host = [torch.empty(self._cap, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._events = [None, None]
        self._dev = torch.empty(self._cap, dtype=torch.int32, device=self.device)

    @staticmethod
    def layout(shapes: Sequence[Sequence[int]]) -> int:
        """int32 elements that arrays of these shapes occupy when staged."""
        total = 0
        for shp in shapes:
            n = 1
            for d in shp:
                n *= int(d)
            total += (n + 3) // 4 * 4
        return total

    def claim(self, elements: int) -> Tuple[int, torch.Tensor]:
        """A pinned host buffer of at least `elements` int32 that no copy in flight still
        reads: (its turn, the buffer).  Fill it, then `send` it."""
        if elements > self._cap:
            torch.cuda.current_stream(self.device).synchronize()
            self._grow(max(int(elements), 2 * self._cap))
        i = self._turn
        self._turn ^= 1
        if self._events[i] is not None:
            self._events[i].synchronize()
        return i, self._host[i]

    def release(self, turn: int) -> None:
        """Give a claimed buffer back unsent (the step was refused)."""
        self._turn = turn

    def send(self, turn: int, total: int, dest: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Copy the first `total` elements of the claimed buffer to the device (to `dest`
        if given, else to the stager's own buffer); returns the device buffer."""
        dev = self._dev if dest is None else dest
        if dev.numel() < total:
            raise ValueError(f"staging destination holds {dev.numel()} elements, {total} are needed")
        dev[:total].copy_(self._host[turn][:total], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self._events[turn] = ev
        self.last_elements = total
        return dev

    @property
    def bytes_last(self) -> int:
        """Bytes the last staged step sent to the device."""
        return getattr(self, "last_elements", 0) * 4
