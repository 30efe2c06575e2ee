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

import ctypes
import json
import os
import re
from typing import Callable, Dict, Hashable, List, Mapping, Optional, Sequence

import numpy as np
import torch

from .. import host
from ..cache.manager import CacheManager
from ..cache.pages import OutOfPages
from ..config.registry import read_model_config
from ..config.spec import ModelSpec
from ..models.decoder import DecoderModel
from ..parts.base import BuildContext, Workspace
from ..weights.loader import load_weights
from ..weights.random_init import random_weights
from .batch import Drawn, StepContext, StepEntry, StepStager
from .timing import DeviceTimer

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


class _Packed:
    """A step's entries as the flat arrays the host library reads."""

    def __init__(self, cache: CacheManager, entries: Sequence[StepEntry]) -> None:
        n = len(entries)
        self.n = n
        self.req = (ctypes.c_longlong * max(1, n))(*[(cache.id_of(e.request) if cache.has(e.request) else -1)
                                                     for e in entries])
        self.n_tok = (ctypes.c_int * max(1, n))(*[len(e.tokens) for e in entries])
        self.n_want = (ctypes.c_int * max(1, n))(*[len(e.want) for e in entries])
        total = sum(self.n_tok[:n])
        try:
            tok = np.fromiter((int(t) for e in entries for t in e.tokens), dtype=np.int64, count=total)
        except (TypeError, ValueError):
            raise ValueError("token ids must be integers") from None
        # an id that does not fit 32 bits becomes -1, which the check reports as outside the vocabulary
        self.tok = np.where((tok < 0) | (tok > 0x7FFFFFFF), -1, tok).astype(np.int32)
        self.want = np.fromiter((int(w) for e in entries for w in e.want), dtype=np.int32, count=sum(self.n_want[:n]))

    @staticmethod
    def ptr(a: np.ndarray):
        return a.ctypes.data_as(ctypes.POINTER(ctypes.c_int))

    def refresh(self, cache: CacheManager, entries: Sequence[StepEntry]) -> None:
        for i, e in enumerate(entries):
            self.req[i] = cache.id_of(e.request)


def _raise_step_error(code: int, entries: Sequence[StepEntry]) -> None:
    """The library names entries by index; the exception names the request."""
    msg = re.sub(r"request #(\d+)", lambda m: f"request {entries[int(m.group(1))].request!r}", host.last_error())
    if code == host.OUT_OF_PAGES:
        raise OutOfPages(msg)
    raise ValueError(msg)


def step_fits(cache: CacheManager, entries: Sequence[StepEntry]) -> bool:
    """Whether every group has the pages this step would take."""
    if not entries:
        return True
    n = len(entries)
    req = (ctypes.c_longlong * n)(*[(cache.id_of(e.request) if cache.has(e.request) else -1) for e in entries])
    n_tok = (ctypes.c_int * n)(*[len(e.tokens) for e in entries])
    rc = host.lib().ilb_step_fits(cache.handle, n, req, n_tok)
    if rc < 0:
        _raise_step_error(rc, entries)
    return rc == 1


def prepare_step(cache: CacheManager, stager: StepStager, entries: Sequence[StepEntry],
                 vocab_size: int, max_positions: int, pad_seqs: int = 0,
                 max_blocks: Optional[int] = None, dest: Optional[torch.Tensor] = None,
                 token_extras: Sequence = ()) -> StepContext:
    """Take pages for the step (all entries or none) and stage its arrays.

    `pad_seqs` appends that many one-token dummy sequences (token 0, position 0, no pages,
    slot -1): their cache writes are dropped and their rows are never read, which lets a
    step of any size run in a launch shape made for a larger one.  `max_blocks` fixes the
    width of the block tables; `dest` receives the arrays instead of the stager's buffer.
    `token_extras` = ((name, width), ...): per-token integer inputs that every entry must
    bring (`StepEntry.extras`); they travel in the same buffer, behind the block tables.
    Checking, page accounting and packing are the C++ host library's."""
    if not entries:
        raise ValueError("a step needs at least one entry")
    lib = host.lib()
    seen = set()
    for e in entries:
        if e.request in seen:
            raise ValueError(f"request {e.request!r} appears twice in one step")
        seen.add(e.request)
    for name, width in token_extras:
        for e in entries:
            got = None if e.extras is None else e.extras.get(name)
            if got is None or len(got) != len(e.tokens) * int(width):
                raise ValueError(f"request {e.request!r} must bring {len(e.tokens)} x {width} values of {name!r}")
    pk = _Packed(cache, entries)
    rc = lib.ilb_step_check(cache.handle, pk.n, pk.req, pk.n_tok, pk.ptr(pk.tok), pk.n_want, pk.ptr(pk.want),
                            int(vocab_size), int(max_positions))
    if rc < 0:
        _raise_step_error(rc, entries)
    fresh = [e.request for e in entries if not cache.has(e.request)]
    for r in fresh:
        cache.begin(r)
    try:
        if not step_fits(cache, entries):
            raise OutOfPages(f"step of {sum(len(e.tokens) for e in entries)} tokens does not fit: "
                             f"free pages {cache.free_pages()}")
        for e in entries:
            cache.ensure(e.request, cache.length(e.request) + len(e.tokens))
    except Exception:
        for r in fresh:
            cache.release(r)
        raise
    pk.refresh(cache, entries)

    reqs = [e.request for e in entries]
    S = len(entries) + pad_seqs
    T = int(pk.tok.size) + pad_seqs
    R = int(pk.want.size) + pad_seqs
    need_blocks = cache.max_blocks(reqs)
    if max_blocks is None:
        max_blocks = (need_blocks + 7) // 8 * 8
    elif need_blocks > max_blocks:
        raise ValueError(f"a request holds {need_blocks} blocks, the table is {max_blocks} wide")
    n_groups = len(cache.groups)
    bound = StepStager.layout([(T,), (T,), (T,), (S + 1,), (S,), (S,), (R,)] + [(S, max_blocks)] * n_groups
                              + [(T, int(w)) for _, w in token_extras])
    turn, hostbuf = stager.claim(bound)
    offsets = (ctypes.c_longlong * (7 + n_groups))()
    total = lib.ilb_step_build(cache.handle, pk.n, pk.req, pk.n_tok, pk.ptr(pk.tok), pk.n_want, pk.ptr(pk.want),
                               int(pad_seqs), int(max_blocks), int(vocab_size), int(max_positions),
                               ctypes.c_void_p(hostbuf.data_ptr()), hostbuf.numel(), offsets)
    if total < 0:
        _raise_step_error(int(total), entries)
    hv = hostbuf.numpy()
    end, extra_at = int(total), {}
    for name, width in token_extras:            # behind what the library packed: [T, width] each, dummy rows zero
        width = int(width)
        rows = hv[end:end + T * width]
        rows[:] = 0
        try:
            rows[:int(pk.tok.size) * width] = np.fromiter((int(x) for e in entries for x in e.extras[name]), dtype=np.int64,
                                                          count=int(pk.tok.size) * width).astype(np.int32)
        except (TypeError, ValueError, OverflowError):
            raise ValueError(f"values of {name!r} must be 32-bit integers") from None
        extra_at[name] = (end, width)
        end += (T * width + 3) // 4 * 4
    dev = stager.send(turn, end, dest)
    view = lambda k, n, shape=None: (dev[offsets[k]:offsets[k] + n] if shape is None
                                     else dev[offsets[k]:offsets[k] + n].view(*shape))
    kv_len = hv[offsets[4]:offsets[4] + S]
    slots = hv[offsets[5]:offsets[5] + len(entries)]
    q_len = [len(e.tokens) for e in entries]
    h_kv = [int(x) for x in kv_len]
    q_start = [h_kv[i] - q_len[i] for i in range(len(entries))]
    return StepContext(
        n_tokens=T, n_seqs=S, n_logit_rows=R,
        tokens=view(0, T), positions=view(1, T), seq_of_token=view(2, T), cu_q=view(3, S + 1),
        kv_len=view(4, S), slots=view(5, S), logit_rows=view(6, R),
        block_tables={g.index: view(7 + i, S * max_blocks, (S, max_blocks)) for i, g in enumerate(cache.groups)},
        extras={name: dev[at:at + T * w].view(T, w) for name, (at, w) in extra_at.items()},
        requests=reqs, h_q_start=q_start, h_q_len=q_len, h_kv_len=h_kv,
        h_slots=[int(x) for x in slots], max_q_len=max(q_len), max_kv_len=max(h_kv),
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
        self.timer = DeviceTimer(device, "off")
        # tokens per row tile of the many-token matrix kernel: a step a few tokens past a
        # multiple costs a whole tile more (the scheduler trims portions to it)
        self.token_multiple = 128 if dtype == torch.bfloat16 else 1
        # Decode-only steps replay recorded graphs: whole, when every part reads its batch from
        # device memory; in segments around the blocks that do not (they loop over host-side
        # batch facts and run kernel by kernel), when at least one block does.
        self.graphs = None
        if cuda_graphs and any(b.graph_safe for b in self.model.blocks):
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

    def resize_cache(self, num_pages, max_requests: int) -> None:
        """Replace the cache by one of another size (`num_pages`: one number, or one per page
        group); only while no request is live."""
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

    def set_device_timing(self, mode: str) -> None:
        """"off", "graph" (two events around every step) or "node" (two events around every
        kernel, steps run kernel by kernel): see engine/timing.py."""
        from ..csrc import ops
        self.timer = DeviceTimer(self.device, mode)
        ops.TIMER = self.timer if mode == "node" else None

    def _graphs_usable(self) -> bool:
        return self.graphs is not None and self.timer.mode != "node"

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

    def step_ahead(self, entries: Sequence[StepEntry], previous_drawn: Drawn) -> Optional[Drawn]:
        """Launch the decode step after one that is still running (see
        `DecodeGraphs.step_ahead`); the entries' tokens are placeholders.  Returns the device
        ids it will draw (still on the device), or None if it was not launched."""
        if not self._graphs_usable() or not self.graphs.eligible(entries):
            return None
        self.timer.step_begin()
        drawn = self.graphs.step_ahead(entries, previous_drawn)
        if drawn is None:
            return None
        self.timer.step_end(len(entries))
        n = len(entries)
        req = (ctypes.c_longlong * n)(*[self.cache.id_of(e.request) for e in entries])
        ones = (ctypes.c_int * n)(*([1] * n))
        rc = host.lib().ilb_step_commit(self.cache.handle, n, req, ones)
        if rc < 0:
            _raise_step_error(rc, entries)
        self.steps_run += 1
        self.tokens_run += n
        return drawn

    # ------------------------------------------------------------------ the step
    def prepare(self, entries: Sequence[StepEntry]) -> StepContext:
        """Take pages for the step (all entries or none) and stage its arrays."""
        return prepare_step(self.cache, self.stager, entries, self.spec.vocab_size, self.spec.max_positions,
                            token_extras=self.spec.token_extras)

    def step(self, entries: Sequence[StepEntry], draw_greedy: bool = False):
        """Run the entries as one batch; returns logits [wanted, vocab] (32-bit, on the
        device, in the order of the entries and of each entry's `want`).  The tensor is a
        scratch buffer: it is valid until the next step.  With `draw_greedy` the arg-max
        of every row is computed in the same launch sequence and (logits, ids) is
        returned, ids being a `Drawn` (the ids and, beside them, a flag per row that is set
        where the logits held a non-finite value)."""
        from ..csrc import ops
        before = ops.LAUNCHES
        drawn = None
        self.timer.step_begin()
        if self._graphs_usable() and self.graphs.eligible(entries) and len(entries) <= 256:
            logits, drawn, kernels = self.graphs.step(entries, with_argmax=draw_greedy)
            self.kernels_last_step = kernels
            n_tokens = len(entries)
        else:
            ctx = self.prepare(entries)
            logits = self.model.forward(ctx, self.cache)
            n_tokens = ctx.n_tokens
            if draw_greedy and logits.shape[0]:
                rows = logits.shape[0]
                pair = self.ctx.workspace.buffer("runner.drawn", (2, rows), torch.int32)
                ops.scope("sampling")
                ops.argmax(logits, pair[0], pair[1])
                ops.scope("other")
                drawn = Drawn(pair, rows)
            self.kernels_last_step = ops.LAUNCHES - before
        self.timer.step_end(n_tokens)
        n = len(entries)
        req = (ctypes.c_longlong * n)(*[self.cache.id_of(e.request) for e in entries])
        n_tok = (ctypes.c_int * n)(*[len(e.tokens) for e in entries])
        rc = host.lib().ilb_step_commit(self.cache.handle, n, req, n_tok)
        if rc < 0:
            _raise_step_error(rc, entries)
        self.steps_run += 1
        self.tokens_run += n_tokens
        return (logits, drawn) if draw_greedy else logits
