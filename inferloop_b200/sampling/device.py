"""Token selection on the device: the highest logit, and a draw from softmax(logits / T)
after the reference's penalties (the request's prompt and output go up as token lists and
become bitmaps there) and filters (top-k, min-p, top-p).  Only token ids (and a finiteness
flag) come back to the host.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..csrc import ops
from .host import request_key, uniform
from .params import SamplingParams


class DeviceSampler:
    def __init__(self, device: torch.device, max_rows: int = 256) -> None:
        self.device = device
        self._cap = 0
        self._bits = None                  # [2, rows, words]: seen and generated token bitmaps
        self._grow(max_rows)

    def _grow(self, rows: int) -> None:
        self._cap = rows
        self.out = torch.empty(rows, dtype=torch.int32, device=self.device)
        self.bad = torch.empty(rows, dtype=torch.int32, device=self.device)
        self.temperature = torch.empty(rows, dtype=torch.float32, device=self.device)
        self.uniform = torch.empty(rows, dtype=torch.float64, device=self.device)
        self.h_out = torch.empty(2 * rows, dtype=torch.int32).pin_memory()
        self.h_error = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.h_temp = torch.empty(rows, dtype=torch.float32).pin_memory()
        self.h_uniform = torch.empty(rows, dtype=torch.float64).pin_memory()
        # per-row filters, staged as one block: top_k (int32 bits), top_p, min_p
        self.filters = torch.empty(3 * rows, dtype=torch.float32, device=self.device)
        self.h_filters = torch.empty(3 * rows, dtype=torch.float32).pin_memory()

    def greedy_launch(self, logits: torch.Tensor) -> None:
        """Arg-max of every row into `self.out` (no synchronisation)."""
        rows = logits.shape[0]
        if rows > self._cap:
            self._grow(max(rows, 2 * self._cap))
        ops.argmax(logits, self.out[:rows], self.bad[:rows])

    def temperature_launch(self, logits: torch.Tensor, temperatures: Sequence[float],
                           uniforms: Sequence[float], params: Sequence[SamplingParams] = (), histories=None) -> None:
        """One draw per row into `self.out` (no synchronisation).  `params`, if given, carry
        each row's top-k / top-p / min-p and penalties; `histories[i]` = (prompt, generated)
        token ids of row i for the rows that have a penalty."""
        rows = logits.shape[0]
        if rows > self._cap:
            self._grow(max(rows, 2 * self._cap))
        self.h_temp[:rows] = torch.tensor(list(temperatures), dtype=torch.float32)
        self.h_uniform[:rows] = torch.tensor(list(uniforms), dtype=torch.float64)
        self.temperature[:rows].copy_(self.h_temp[:rows], non_blocking=True)
        self.uniform[:rows].copy_(self.h_uniform[:rows], non_blocking=True)
        top_k = top_p = min_p = None
        if any(p.top_k is not None or p.top_p < 1.0 or p.min_p > 0.0 for p in params):
            cap = self._cap
            self.h_filters[:rows].view(torch.int32)[:] = torch.tensor([p.top_k or 0 for p in params], dtype=torch.int32)
            self.h_filters[cap:cap + rows] = torch.tensor([p.top_p for p in params], dtype=torch.float32)
            self.h_filters[2 * cap:2 * cap + rows] = torch.tensor([p.min_p for p in params], dtype=torch.float32)
            self.filters.copy_(self.h_filters, non_blocking=True)
            top_k = self.filters[:rows].view(torch.int32)
            top_p, min_p = self.filters[cap:cap + rows], self.filters[2 * cap:2 * cap + rows]
        penalties = None
        if histories is not None and any(p.presence_penalty != 0.0 or p.repetition_penalty != 1.0 for p in params):
            penalties = self._penalties(rows, logits.shape[1], params, histories)
        ops.sample_temperature(logits, self.temperature[:rows], self.uniform[:rows],
                               self.out[:rows], self.bad[:rows], top_k, top_p, min_p, penalties)

    def _penalties(self, rows: int, vocab: int, params: Sequence[SamplingParams], histories) -> tuple:
        """Token bitmaps of the rows that have a penalty (prompt + output, and output alone)
        and the per-row penalty values, on the device."""
        words = (vocab + 31) // 32
        if self._bits is None or self._bits.shape[1] < rows or self._bits.shape[2] != words:
            self._bits = torch.empty(2, max(rows, self._cap), words, dtype=torch.int32, device=self.device)
        bits = self._bits[:, :rows]
        bits.zero_()
        r_idx, toks, flags = [], [], []
        for i, (p, h) in enumerate(zip(params, histories)):
            if h is None or (p.presence_penalty == 0.0 and p.repetition_penalty == 1.0):
                continue
            prompt, generated = h
            for t in list(prompt) + list(generated):
                if not (0 <= int(t) < vocab):
                    raise ValueError("history token outside vocabulary")
            r_idx += [i] * (len(prompt) + len(generated))
            toks += list(prompt) + list(generated)
            flags += [0] * len(prompt) + [1] * len(generated)
        if toks:
            entries = torch.tensor([r_idx, toks, flags], dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
            ops.mark_tokens(entries[0], entries[1], entries[2], bits[0], bits[1], vocab)
        pen = torch.tensor([[p.repetition_penalty for p in params], [p.presence_penalty for p in params]],
                           dtype=torch.float32).pin_memory().to(self.device, non_blocking=True)
        return bits[0], bits[1], pen[0], pen[1]

    def read(self, rows: int) -> List[int]:
        """Token ids of the last launch (synchronises); raises on non-finite logits."""
        self.h_out[:rows].copy_(self.out[:rows], non_blocking=True)
        self.h_out[rows:2 * rows].copy_(self.bad[:rows], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        vals = self.h_out[:2 * rows].tolist()
        if any(vals[rows:]):
            raise ValueError("invalid sampling logits (a non-finite value)")
        return vals[:rows]

    def start_read(self, drawn):
        """Begin copying to the host what a step drew on the device (`Drawn`: the ids and
        the flags of non-finite rows, as one contiguous copy) and the flag that kernels raise when
        they give up a bounded wait; work that is launched after this call does not delay
        them.  Returns a handle for `finish_read`."""
        rows, width = drawn.n, drawn.pair.shape[1]
        if width > self._cap:
            self._grow(max(width, 2 * self._cap))
        self.h_out[:2 * width].copy_(drawn.pair.view(-1), non_blocking=True)
        self.d2h_bytes_last = 2 * width * 4
        error = ops.device_error_tensor(self.device)
        if error is not None:
            self.h_error.copy_(error, non_blocking=True)
            self.d2h_bytes_last += 4
        event = torch.cuda.Event()
        event.record(torch.cuda.current_stream(self.device))
        return rows, width, event

    def finish_read(self, handle) -> List[int]:
        """Wait for the copy begun by `start_read` and return the ids.  Raises, before any
        id is handed out, if a row held a non-finite logit (the reference's greedy refuses
        those: crates/engine/workloads/src/sampling.rs:175-180) or a kernel gave up a wait."""
        rows, width, event = handle
        event.synchronize()
        ids = self.h_out[:rows].tolist()
        if int(self.h_error[0]) != 0:
            self.h_error[0] = 0
            ops.check_device_errors()
        if any(self.h_out[width:width + rows].tolist()):
            raise ValueError("invalid sampling logits (a non-finite value)")
        return ids

    def read_ids(self, drawn) -> List[int]:
        """Token ids that a step already drew on the device (synchronises)."""
        return self.finish_read(self.start_read(drawn))
