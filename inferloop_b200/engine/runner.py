"""The step function: run a batch of (request, its next tokens) from the cache.

`ModelRunner.step(entries)` runs only the tokens it is given, as one batch, and returns
the 32-bit logits at the wanted places.  It is the single path from tokens to logits:
trace replay, the scheduler and the Python entry point all call it.  The reference's
counterpart is `BackendProvider::submit/poll` over a list of `ExecutionTask`s
(crates/foundation/spi/src/backend.rs:340-345, :403); there a task continues the
backend's own history cursor (crates/foundation/ir/src/tokens.rs:171-180), here the
cursor is the cache manager's committed length of the request.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Hashable, List, Mapping, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.pages import OutOfPages
from ..config.registry import read_model_config
from ..config.spec import ModelSpec
from ..models.decoder import DecoderModel
from ..parts.base import BuildContext, Workspace
from ..weights.loader import load_weights
from ..weights.random_init import random_weights
from .batch import StepContext, StepEntry, StepStager

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
          "f32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {name} is not served; use bfloat16 or float32")
        return name
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype {name!r}; use bfloat16 or float32") from None


def require_cuda(device) -> torch.device:
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError(f"inferloop_b200 runs on a CUDA device only, not on {dev}")
    if not torch.cuda.is_available():
        raise RuntimeError("inferloop_b200 needs a CUDA device (sm_100a) and found none; "
                           "there is no CPU path")
    return dev


def step_fits(cache: CacheManager, entries: Sequence[StepEntry]) -> bool:
    """Whether every group has the pages this step would take."""
    need: Dict[int, int] = {}
    for e in entries:
        cur = cache.length(e.request) if cache.has(e.request) else 0
        if cache.has(e.request):
            per = cache.pages_needed(e.request, cur + len(e.tokens))
        else:
            per = {g.index: -(-len(e.tokens) // cache.page_size) for g in cache.groups}
        for g, n in per.items():
            need[g] = need.get(g, 0) + n
    free = cache.free_pages()
    return all(need.get(g, 0) <= free[g] for g in free)



def prepare_step(cache: CacheManager, stager: StepStager, entries: Sequence[StepEntry],
                 vocab_size: int, max_positions: int, pad_seqs: int = 0,
                 max_blocks: Optional[int] = None, dest: Optional[torch.Tensor] = None) -> StepContext:
    """Take pages for the step (all entries or none) and stage its arrays.

    `pad_seqs` appends that many one-token dummy sequences (token 0, position 0, no pages,
    slot -1): their cache writes are dropped and their rows are never read, which lets a
    step of any size run in a launch shape made for a larger one.  `max_blocks` fixes the
    width of the block tables; `dest` receives the arrays instead of the stager's buffer."""
    if not entries:
        raise ValueError("a step needs at least one entry")
    seen = set()
    for e in entries:
        if e.request in seen:
            raise ValueError(f"request {e.request!r} appears twice in one step")
        seen.add(e.request)
        if len(e.tokens) == 0:
            raise ValueError(f"request {e.request!r} brings no tokens")
        for w in e.want:
            if not (0 <= w < len(e.tokens)):
                raise ValueError(f"request {e.request!r}: wanted place {w} is outside its {len(e.tokens)} tokens")
        for t in e.tokens:
            if not (0 <= int(t) < vocab_size):
                raise ValueError(f"request {e.request!r}: token {t} is outside the vocabulary of {vocab_size}")
    fresh = [e.request for e in entries if not cache.has(e.request)]
    for r in fresh:
        cache.begin(r)
    try:
        if not step_fits(cache, entries):
            raise OutOfPages(f"step of {sum(len(e.tokens) for e in entries)} tokens does not fit: "
                             f"free pages {cache.free_pages()}")
        for e in entries:
            new_len = cache.length(e.request) + len(e.tokens)
            if new_len > max_positions:
                raise ValueError(f"request {e.request!r} would reach {new_len} tokens; the model's "
                                 f"limit is {max_positions}")
        for e in entries:
            cache.ensure(e.request, cache.length(e.request) + len(e.tokens))
    except Exception:
        for r in fresh:
            cache.release(r)
        raise

    S = len(entries) + pad_seqs
    T = sum(len(e.tokens) for e in entries) + pad_seqs
    tokens = np.zeros(T, np.int32)
    positions = np.zeros(T, np.int32)
    seq_of = np.zeros(T, np.int32)
    cu_q = np.zeros(S + 1, np.int32)
    kv_len = np.zeros(S, np.int32)
    slots = np.full(S, -1, np.int32)
    rows: List[int] = []
    q_start, q_len = [], []
    off = 0
    for s, e in enumerate(entries):
        n = len(e.tokens)
        cur = cache.length(e.request)
        tokens[off:off + n] = np.asarray(e.tokens, dtype=np.int64)
        positions[off:off + n] = np.arange(cur, cur + n, dtype=np.int32)
        seq_of[off:off + n] = s
        cu_q[s + 1] = off + n
        kv_len[s] = cur + n
        slots[s] = cache.slot_of(e.request)
        rows.extend(off + int(w) for w in e.want)
        q_start.append(cur)
        q_len.append(n)
        off += n
    for s in range(len(entries), S):          # padding
        seq_of[off] = s
        cu_q[s + 1] = off + 1
        rows.append(off)
        off += 1
    reqs = [e.request for e in entries]
    need_blocks = cache.max_blocks(reqs)
    if max_blocks is None:
        max_blocks = (need_blocks + 7) // 8 * 8
    elif need_blocks > max_blocks:
        raise ValueError(f"a request holds {need_blocks} blocks, the table is {max_blocks} wide")
    tables = []
    for g in cache.groups:
        tb = np.full((S, max_blocks), -1, np.int32)
        for s, r in enumerate(reqs):
            row = cache.block_table(g.index, r)
            tb[s, :len(row)] = row
        tables.append(tb)
    logit_rows = np.asarray(rows, dtype=np.int32)
    staged = stager.stage([tokens, positions, seq_of, cu_q, kv_len, slots, logit_rows] + tables, dest)
    return StepContext(
        n_tokens=T, n_seqs=S, n_logit_rows=len(rows),
        tokens=staged[0], positions=staged[1], seq_of_token=staged[2], cu_q=staged[3],
        kv_len=staged[4], slots=staged[5], logit_rows=staged[6],
        block_tables={g.index: staged[7 + i] for i, g in enumerate(cache.groups)},
        requests=reqs, h_q_start=q_start, h_q_len=q_len, h_kv_len=[int(x) for x in kv_len],
        h_slots=[int(x) for x in slots[:len(entries)]], max_q_len=max(q_len), max_kv_len=int(kv_len.max()),
        decode_only=all(n == 1 for n in q_len))



class ModelRunner:
    def __init__(self, spec: ModelSpec, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype,
                 device: torch.device, page_size: int, num_pages: int, max_requests: int,
                 cuda_graphs: bool = True) -> None:
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.ctx = BuildContext(dtype=dtype, device=device, workspace=Workspace(device))
        self.model = DecoderModel(spec, self.ctx)
        self.model.bind(tensors)
        self.cache = CacheManager(self.model.cache_needs(), page_size, num_pages, max_requests,
                                  dtype=dtype, device=device, run_order=spec.run_order)
        self.stager = StepStager(device)
        self.steps_run = 0
        self.tokens_run = 0
        self.kernels_last_step = 0
        # Decode-only steps replay recorded graphs when every part reads its batch from
        # device memory (a part that loops over host-side batch facts cannot be replayed).
        self.graphs = None
        if cuda_graphs and all(b.graph_safe for b in self.model.blocks):
            from .graphs import DecodeGraphs
            self.graphs = DecodeGraphs(self, -(-spec.max_positions // page_size))

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, folder: str, dtype="bfloat16", device="cuda:0", page_size: int = 16,
                    num_pages: int = 256, max_requests: int = 64, registry=None,
                    allow_unexpected: bool = False,
                    progress: Optional[Callable[[str], None]] = None) -> "ModelRunner":
        dev = require_cuda(device)
        dt = parse_dtype(dtype)
        path = os.path.join(folder, "config.json")
        if not os.path.exists(path):
            raise FileNotFoundError(f"{folder}: no config.json")
        with open(path, "r", encoding="utf-8") as fh:
            text = fh.read(1 << 20)     # bounded read (storage/source.rs:265-313)
        _, _, spec = read_model_config(text, registry)
        decls = DecoderModel(spec, BuildContext(dt, None, Workspace(None))).declare_weights()
        tensors, _ = load_weights(folder, decls, spec.weight_prefixes, spec.embedding_name, dt, dev,
                                  allow_unexpected=allow_unexpected, progress=progress)
        return cls(spec, tensors, dt, dev, page_size, num_pages, max_requests)

    @classmethod
    def from_config(cls, config: Mapping, seed: int, dtype="bfloat16", device="cuda:0",
                    page_size: int = 16, num_pages: int = 256, max_requests: int = 64,
                    registry=None) -> "ModelRunner":
        """Random weights made on the device (no folder is written)."""
        dev = require_cuda(device)
        dt = parse_dtype(dtype)
        _, _, spec = read_model_config(json.dumps(dict(config)), registry)
        decls = DecoderModel(spec, BuildContext(dt, None, Workspace(None))).declare_weights()
        tensors = random_weights(decls, seed, dt, dev)
        return cls(spec, tensors, dt, dev, page_size, num_pages, max_requests)

    def resize_cache(self, num_pages: int, max_requests: int) -> None:
        """Replace the cache by one of another size; only while no request is live."""
        if self.cache.live_requests():
            raise RuntimeError("the cache cannot be resized while requests are live")
        page_size = self.cache.page_size
        self.cache = None
        torch.cuda.empty_cache()
        self.cache = CacheManager(self.model.cache_needs(), page_size, num_pages, max_requests,
                                  dtype=self.dtype, device=self.device, run_order=self.spec.run_order)
        if self.graphs is not None:          # recorded graphs point into the old cache
            from .graphs import DecodeGraphs
            self.graphs = DecodeGraphs(self, -(-self.spec.max_positions // page_size))

    # ------------------------------------------------------------------ requests
    def begin(self, request: Hashable) -> None:
        self.cache.begin(request)

    def end(self, request: Hashable) -> None:
        self.cache.release(request)

    def is_live(self, request: Hashable) -> bool:
        return self.cache.has(request)

    def can_run(self, entries: Sequence[StepEntry]) -> bool:
        """Whether every group has the pages this step would take."""
        return step_fits(self.cache, entries)

    # ------------------------------------------------------------------ the step
    def prepare(self, entries: Sequence[StepEntry]) -> StepContext:
        """Take pages for the step (all entries or none) and stage its arrays."""
        return prepare_step(self.cache, self.stager, entries, self.spec.vocab_size, self.spec.max_positions)

    def step(self, entries: Sequence[StepEntry], draw_greedy: bool = False):
        """Run the entries as one batch; returns logits [wanted, vocab] (32-bit, on the
        device, in the order of the entries and of each entry's `want`).  The tensor is a
        scratch buffer: it is valid until the next step.  With `draw_greedy` the arg-max
        of every row is computed in the same launch sequence and (logits, ids) is
        returned, ids being an int32 device tensor."""
        from ..csrc import ops
        before = ops.LAUNCHES
        drawn = None
        if self.graphs is not None and self.graphs.eligible(entries) and len(entries) <= 256:
            logits, drawn, kernels = self.graphs.step(entries, with_argmax=draw_greedy)
            self.kernels_last_step = kernels
            n_tokens = len(entries)
        else:
            ctx = self.prepare(entries)
            logits = self.model.forward(ctx, self.cache)
            n_tokens = ctx.n_tokens
            if draw_greedy and logits.shape[0]:
                drawn = self.ctx.workspace.buffer("runner.drawn", (logits.shape[0],), torch.int32)
                ops.argmax(logits, drawn, None)
            self.kernels_last_step = ops.LAUNCHES - before
        for e in entries:
            self.cache.commit(e.request, self.cache.length(e.request) + len(e.tokens))
        self.steps_run += 1
        self.tokens_run += n_tokens
        return (logits, drawn) if draw_greedy else logits
