"""Decode steps as replayed CUDA graphs.

A step in which every request brings exactly one token is launch-bound when run kernel
by kernel.  Such steps are recorded once per batch-size bucket and replayed: the batch's
integer arrays live at fixed device addresses that are overwritten before each replay, and
every kernel reads the batch from there.  The reference does the same with one resident
decode graph whose control row is rewritten on-stream before each replay
(crates/backend/cuda/src/resident/program.rs; metadata row:
crates/backend/cuda-kernels/src/tile/state/metadata_kernels.rs:87-101); its fixed graph
widths are the buckets here.  A step smaller than its bucket is padded with dummy
sequences that hold no pages.

A recorded graph also holds the addresses of the model's scratch buffers; when one of
them has been reallocated since (a larger prompt step grew it), the graph is recorded
again.

A step is recorded in SEGMENTS.  A block is recorded only if it says that it reads the
batch from device memory alone (`graph_safe`); a block that loops over host-side batch
facts (a mixer with sequential state written in Python, say) runs kernel by kernel between
two recorded segments, with the step's host-side facts refreshed.  A model whose blocks are
all safe is one segment, and only such a model has its next step launched ahead.
"""
from __future__ import annotations

import gc
import weakref
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..csrc import ops
from .batch import Drawn, StepContext, StepEntry, StepStager

BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)


def bucket_for(n: int) -> Optional[int]:
    for b in BUCKETS:
        if n <= b:
            return b
    return None


@dataclass
class _Recorded:
    segments: List[tuple]              # ("graph", CUDAGraph) | ("entries", first, last) run kernel by kernel
    ints: torch.Tensor                 # the batch arrays, fixed address
    ctx: StepContext                   # views into `ints`
    logits: torch.Tensor
    workspace_generation: int
    kernels: int                       # launches recorded
    pair: Optional[torch.Tensor] = None       # [2, bucket]: drawn ids, and their non-finite flags

    @property
    def drawn(self) -> Optional[torch.Tensor]:
        return None if self.pair is None else self.pair[0]

    @property
    def whole(self) -> bool:
        """One recorded graph holds the whole step."""
        return len(self.segments) == 1 and self.segments[0][0] == "graph"

    @property
    def graph(self) -> torch.cuda.CUDAGraph:
        if not self.whole:
            raise RuntimeError("this step is recorded in several segments")
        return self.segments[0][1]


class DecodeGraphs:
    def __init__(self, runner, max_blocks: int) -> None:
        self._runner = weakref.ref(runner)     # the runner owns this object, not the reverse
        self.max_blocks = int(max_blocks)
        self._recorded: Dict[tuple, _Recorded] = {}
        self.replays = 0
        # run-order entries in maximal runs of blocks that may / may not be recorded
        model = runner.model
        self.plan: List[tuple] = []          # (recorded?, first entry, last entry)
        order = runner.spec.run_order
        i = 0
        while i < len(order):
            safe = bool(model.blocks[order[i].layer].graph_safe)
            j = i
            while j < len(order) and bool(model.blocks[order[j].layer].graph_safe) == safe:
                j += 1
            self.plan.append((safe, i, j))
            i = j
        self.head_safe = bool(model.graph_safe)
        self.whole = self.head_safe and all(safe for safe, _, _ in self.plan)

    @property
    def runner(self):
        r = self._runner()
        if r is None:
            raise RuntimeError("the model runner of these graphs is gone")
        return r

    @staticmethod
    def eligible(entries: Sequence[StepEntry]) -> bool:
        return all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)

    def _key(self, entries: Sequence[StepEntry], bucket: int, with_argmax: bool) -> tuple:
        """Recorded graphs are kept apart by size, by what follows the logits, and, for the
        few-sequence sizes whose attention launch depends on it, by whether the longest
        sequence has reached ops.DECODE_LONG_CONTEXT keys."""
        long_context = False
        if bucket <= 4:
            cache = self.runner.cache
            long_context = any(cache.has(e.request) and cache.length(e.request) + 1 >= ops.DECODE_LONG_CONTEXT
                               for e in entries)
        return (bucket, with_argmax, long_context)

    def _shapes(self, bucket: int) -> List[tuple]:
        groups = len(self.runner.cache.groups)
        return [(bucket,), (bucket,), (bucket,), (bucket + 1,), (bucket,), (bucket,), (bucket,)] + \
               [(bucket, self.max_blocks)] * groups + [(bucket, int(w)) for _, w in self.runner.spec.token_extras]

    def _prepare(self, entries: Sequence[StepEntry], bucket: int, ints: torch.Tensor) -> StepContext:
        from .runner import prepare_step
        r = self.runner
        return prepare_step(r.cache, r.stager, entries, r.spec.vocab_size, r.spec.max_positions,
                            pad_seqs=bucket - len(entries), max_blocks=self.max_blocks, dest=ints,
                            token_extras=r.spec.token_extras)

    def _record(self, key: tuple, entries: Sequence[StepEntry], bucket: int, with_argmax: bool) -> _Recorded:
        r = self.runner
        ints = torch.zeros(StepStager.layout(self._shapes(bucket)), dtype=torch.int32, device=r.device)
        ctx = self._prepare(entries, bucket, ints)
        pair = torch.zeros((2, bucket), dtype=torch.int32, device=r.device) if with_argmax else None
        # Once eagerly: builds kernels, sizes every scratch buffer, and does this step's work.
        logits = r.model.forward(ctx, r.cache)
        if with_argmax:
            ops.argmax(logits, pair[0], pair[1])
        torch.cuda.current_stream(r.device).synchronize()
        generation = r.ctx.workspace.generation
        before = ops.LAUNCHES
        ctx.position_tables.clear()
        # The step as pieces: embedding with the first run of blocks if that run is recorded,
        # the last run with the head if both are, eager runs in between.
        model, cache = r.model, r.cache
        pieces: List[tuple] = []               # (recorded?, [callables])
        hidden_of: Dict[str, torch.Tensor] = {}

        def embed():
            hidden_of["h"] = model.forward_embed(ctx)

        def entries(first, last):
            return lambda: model.forward_entries(hidden_of["h"], ctx, cache, first, last)

        def head():
            out = model.forward_head(hidden_of["h"], ctx)
            if with_argmax:
                ops.argmax(out, pair[0], pair[1])
            hidden_of["logits"] = out

        pieces.append((True, [embed]))
        for safe, first, last in self.plan:
            if safe and pieces[-1][0]:
                pieces[-1][1].append(entries(first, last))
            else:
                pieces.append((safe, [entries(first, last)] if safe else [("entries", first, last)]))
        if self.head_safe and pieces[-1][0]:
            pieces[-1][1].append(head)
        else:
            pieces.append((self.head_safe, [head] if self.head_safe else [("head",)]))
        segments: List[tuple] = []
        # Nothing may be destroyed on the device while a recording is open: an older
        # graph released by the garbage collector in that window invalidates it.
        gc.collect()
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            for recorded, calls in pieces:
                if recorded:
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        for call in calls:
                            call()
                    segments.append(("graph", graph))
                else:
                    # not recorded: nothing runs now (the eager pass above has done this step's
                    # work exactly once); it runs kernel by kernel at every replay
                    segments.extend(calls)
        finally:
            if gc_was_on:
                gc.enable()
        if "logits" in hidden_of:
            logits = hidden_of["logits"]          # (else the head is not recorded: the eager pass's buffer, same address)
        kernels = ops.LAUNCHES - before
        if r.ctx.workspace.generation != generation:
            raise RuntimeError("a scratch buffer was reallocated while a graph was recorded")
        rec = _Recorded(segments, ints, ctx, logits, generation, kernels, pair)
        self._recorded[key] = rec
        return rec

    def _prepare_replay(self, entries: Sequence[StepEntry], bucket: int, rec: "_Recorded") -> None:
        """What `_prepare` does for a recorded bucket, in one call of the host library and
        without building views nobody reads: check, pages, arrays into the graph's buffer."""
        import ctypes
        from .. import host
        from .runner import _raise_step_error
        r = self.runner
        cache = r.cache
        n = len(entries)
        if r.spec.token_extras:               # the library's fast path packs ids and positions only
            self._prepare(entries, bucket, rec.ints)
            return
        try:
            req = (ctypes.c_longlong * n)(*[cache.id_of(e.request) for e in entries])
            tok = (ctypes.c_int * n)(*[int(e.tokens[0]) for e in entries])
        except KeyError:                      # a request that is not live yet: the general path begins it
            self._prepare(entries, bucket, rec.ints)
            return
        except (OverflowError, TypeError, ValueError):
            raise ValueError("token ids must be integers of the vocabulary") from None
        turn, hostbuf = r.stager.claim(rec.ints.numel())
        offsets = (ctypes.c_longlong * (7 + len(cache.groups)))()
        total = host.lib().ilb_step_decode(cache.handle, n, req, tok, bucket - n, self.max_blocks,
                                           r.spec.vocab_size, r.spec.max_positions,
                                           ctypes.c_void_p(hostbuf.data_ptr()), hostbuf.numel(), offsets)
        if total < 0:
            r.stager.release(turn)
            _raise_step_error(int(total), entries)
        r.stager.send(turn, int(total), rec.ints)

    def step(self, entries: Sequence[StepEntry], with_argmax: bool = False):
        """Run a decode-only step.  Returns (logits[:n], drawn[:n] or None, kernels
        launched).  The very first step of a bucket runs eagerly while it is recorded."""
        n = len(entries)
        bucket = bucket_for(n)
        if bucket is None:
            raise ValueError(f"{n} sequences exceed the largest decode bucket {BUCKETS[-1]}")
        key = self._key(entries, bucket, with_argmax)
        rec = self._recorded.get(key)
        if rec is not None and rec.workspace_generation != self.runner.ctx.workspace.generation:
            del self._recorded[key]
            rec = None
        if rec is None:
            rec = self._record(key, entries, bucket, with_argmax)     # ran the step eagerly
        elif rec.whole:
            self._prepare_replay(entries, bucket, rec)
            rec.graph.replay()
            self.replays += 1
        else:
            self._replay_segments(entries, bucket, rec, with_argmax)
        return rec.logits[:n], (Drawn(rec.pair, n) if with_argmax else None), rec.kernels

    def _replay_segments(self, entries: Sequence[StepEntry], bucket: int, rec: "_Recorded", with_argmax: bool) -> None:
        """A step recorded in several segments: the recorded ones are replayed, the others run
        kernel by kernel with this step's host-side facts (the device arrays are the ones the
        recorded segments read)."""
        r = self.runner
        ctx = self._prepare(entries, bucket, rec.ints)
        hidden = r.ctx.workspace.buffer("model.hidden", (ctx.n_tokens, r.spec.hidden_size), torch.float32)
        for seg in rec.segments:
            if seg[0] == "graph":
                seg[1].replay()
            elif seg[0] == "entries":
                r.model.forward_entries(hidden, ctx, r.cache, seg[1], seg[2])
            else:
                logits = r.model.forward_head(hidden, ctx)
                if with_argmax:
                    ops.argmax(logits, rec.pair[0], rec.pair[1])
        if r.ctx.workspace.generation != rec.workspace_generation:
            raise RuntimeError("a scratch buffer was reallocated by a part that runs between recorded segments")
        self.replays += 1

    def step_ahead(self, entries: Sequence[StepEntry], previous_drawn: Drawn) -> Optional[Drawn]:
        """The decode step that follows one whose tokens are still being computed: the same
        requests in the same order, each continuing with the token the previous step draws.
        The ids never visit the host: they are copied on the device from `previous_drawn`
        into this step's token array before the replay.  Returns the ids the step will draw
        (on the device), or None when the step cannot be launched this way (no recorded graph
        for this size yet, or not enough pages), in which case nothing has changed."""
        from ..cache.pages import OutOfPages
        n = len(entries)
        bucket = bucket_for(n)
        if bucket is None:
            return None
        if self.runner.spec.token_extras:     # the next step's extra inputs are the caller's to give
            return None
        rec = self._recorded.get(self._key(entries, bucket, True))
        if rec is None or not rec.whole or rec.workspace_generation != self.runner.ctx.workspace.generation:
            return None
        try:
            self._prepare_replay(entries, bucket, rec)
        except OutOfPages:
            return None
        rec.ctx.tokens[:n].copy_(previous_drawn.ids)
        rec.graph.replay()
        self.replays += 1
        return Drawn(rec.pair, n)

    def recorded(self, n: int, with_argmax: bool) -> Optional[_Recorded]:
        """The graph recorded for this many sequences (the short-context one if both exist)."""
        for long_context in (False, True):
            rec = self._recorded.get((bucket_for(n), with_argmax, long_context))
            if rec is not None:
                return rec
        return None

    def run_greedy(self, entries: Sequence[StepEntry], n_steps: int) -> torch.Tensor:
        """`n_steps` greedy decode steps back to back without a host round trip: each
        step's arg-max becomes the next step's token on the device.  `entries` hold each
        request's next token.  Pages for all steps are taken up front.  Returns the drawn
        ids [n_steps, len(entries)] (int32, device); the requests' cache lengths advance by
        n_steps."""
        r = self.runner
        n = len(entries)
        if not self.eligible(entries):
            raise ValueError("run_greedy takes one token per request, logits wanted")
        if not self.whole or r.spec.token_extras:
            raise ValueError("run_greedy needs a model whose whole step is recorded as one graph and that "
                             "takes no inputs per token beside ids and positions")
        bucket = bucket_for(n)
        if bucket is None:
            raise ValueError(f"{n} sequences exceed the largest decode bucket")
        for e in entries:                       # all pages first, or none
            if not r.cache.has(e.request):
                raise ValueError(f"request {e.request!r} is not live")
        need: Dict[int, int] = {}
        for e in entries:
            for g, k in r.cache.pages_needed(e.request, r.cache.length(e.request) + n_steps).items():
                need[g] = need.get(g, 0) + k
        free = r.cache.free_pages()
        if any(need.get(g, 0) > free[g] for g in free):
            from ..cache.pages import OutOfPages
            raise OutOfPages(f"{n_steps} decode steps of {n} requests need {need}, free {free}")
        for e in entries:
            r.cache.ensure(e.request, r.cache.length(e.request) + n_steps)
        out = torch.empty((n_steps, bucket), dtype=torch.int32, device=r.device)
        key = self._key(entries, bucket, True)
        rec = self._recorded.get(key)
        if rec is not None and rec.workspace_generation != r.ctx.workspace.generation:
            del self._recorded[key]
            rec = None
        first = 0
        if rec is None:
            rec = self._record(key, entries, bucket, True)      # step 0 ran eagerly
            out[0].copy_(rec.drawn)
            ops.decode_advance(rec.ctx.tokens, rec.ctx.positions, rec.ctx.kv_len, rec.drawn, n)
            first = 1
        else:
            self._prepare(entries, bucket, rec.ints)
        for i in range(first, n_steps):
            rec.graph.replay()
            out[i].copy_(rec.drawn)
            ops.decode_advance(rec.ctx.tokens, rec.ctx.positions, rec.ctx.kv_len, rec.drawn, n)
        self.replays += n_steps - first
        for e in entries:
            r.cache.commit(e.request, r.cache.length(e.request) + n_steps)
        r.steps_run += n_steps
        r.tokens_run += n_steps * n
        return out[:, :n]
