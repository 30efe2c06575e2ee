"""Continuous batching above the step function (policy in C++, see `Scheduler`).

Each call of :meth:`Scheduler.plan` builds ONE step under a token budget and a sequence
cap: every request that is decoding brings one token, prompts are cut into portions,
waiting requests are admitted first come first served while budget, sequences and pages
allow.  It decides; it runs nothing and takes no pages (the step function takes them
when it prepares the step the plan describes).

What the reference does and what is kept of it:
  * a request is `Decode` once `prefill_done == prefill_target`, else `Prefill` with the
    remainder of its prompt (crates/engine/runtime/src/pipeline/scheduling/ready.rs:105-117);
  * per-step budgets `max_num_seqs` and `max_num_batched_tokens`
    (crates/foundation/ir/src/execution.rs:233-245), portion cap `prefill_chunk_tokens`
    (crates/foundation/ir/src/scheduling.rs:7-12), decode before prefill on ties
    (crates/engine/scheduler/src/policy.rs:203-233);
  * a prompt portion is granted whole if the remaining budget funds it; when decodes have
    eaten into the budget it gets the remainder only if that is at least half a portion,
    else it waits (crates/engine/scheduler/src/policy/packing.rs:328-347); this engine's own
    addition: a whole portion that shares its step is trimmed to the next lower multiple of
    `step_token_multiple` tokens for the step (the matrix kernels' token tile), under the
    same half-portion floor;
  * finish on an end-of-sequence token or on `max_new_tokens`
    (crates/engine/runtime/src/pipeline/completion/mod.rs:402-408);
  * when pages run out: the blocked work waits if something else can run; if a decoding
    request is blocked, victims are preempted BY RECOMPUTE in reverse priority order --
    pages returned, prefill restarted over prompt + generated tokens, generated tokens and
    sampling positions kept (crates/engine/scheduler/src/preemption.rs:59-119;
    crates/engine/runtime/src/pipeline/scheduling/preemption.rs:67-76).
Left out: tenants, SLO classes, the cost model and time budgets -- priority here is
arrival order.
"""
from __future__ import annotations

import ctypes
import re
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

from .. import host
from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 64               # reference default: the submission batch limit
    max_num_batched_tokens: int = 2048
    prefill_chunk_tokens: int = 512
    max_model_len: int = 4096
    # A whole portion that shares a step with other work is trimmed so that the step's tokens
    # are a multiple of this (the token tile of the matrix kernels; 1 = never trimmed).
    step_token_multiple: int = 1

    def __post_init__(self) -> None:
        for name in ("max_num_seqs", "max_num_batched_tokens", "prefill_chunk_tokens", "max_model_len"):
            if int(getattr(self, name)) <= 0:
                raise ValueError(f"{name} must be positive")
        # A step must be able to hold one portion beside every other sequence's decode
        # token (crates/service/cli/src/support/serving.rs:93-115).
        floor = min(self.prefill_chunk_tokens, self.max_model_len) + self.max_num_seqs - 1
        if self.max_num_batched_tokens < floor:
            self.max_num_batched_tokens = floor


@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    params: SamplingParams
    max_new_tokens: int
    arrival: int = 0
    generated: List[int] = field(default_factory=list)
    status: str = WAITING
    finish_reason: Optional[str] = None
    preemptions: int = 0
    # per-token integer inputs the model's description declares (name -> values of the prompt's
    # tokens, token by token); a generated token continues them: every value of the last
    # prompt token plus the token's index among the generated ones plus one (what position-like
    # inputs do when text continues)
    extras: Optional[Dict[str, List[int]]] = None

    def extras_of(self, name: str, width: int, start: int, count: int) -> List[int]:
        """Values of `name` for tokens start .. start + count - 1 of the sequence."""
        values = (self.extras or {}).get(name)
        n = len(self.prompt)
        if values is None or len(values) != n * width:
            raise ValueError(f"request {self.id!r} has no {n} x {width} values of {name!r}")
        out: List[int] = []
        for t in range(start, start + count):
            if t < n:
                out += values[t * width:(t + 1) * width]
            else:
                out += [v + (t - n + 1) for v in values[(n - 1) * width:n * width]]
        return out

    @property
    def sequence(self) -> List[int]:
        """Everything that must be in the cache before the next token is drawn."""
        return self.prompt + self.generated

    def total_len(self) -> int:
        return len(self.prompt) + len(self.generated)


@dataclass
class PlannedWork:
    request: Request
    start: int          # first position this step computes
    count: int          # how many tokens
    samples: bool       # the step's last token is the last known one: draw the next

    @property
    def tokens(self) -> List[int]:
        r, a, b = self.request, self.start, self.start + self.count
        n = len(r.prompt)                    # without joining the two lists every step
        if b <= n:
            return r.prompt[a:b]
        if a >= n:
            return r.generated[a - n:b - n]
        return r.prompt[a:] + r.generated[:b - n]


@dataclass
class StepPlan:
    work: List[PlannedWork] = field(default_factory=list)
    preempted: List[Hashable] = field(default_factory=list)

    @property
    def n_tokens(self) -> int:
        return sum(w.count for w in self.work)


class CapacityError(RuntimeError):
    """A single request cannot fit the cache even when it is alone."""


class Scheduler:
    """The planning itself is the C++ host library's (`host/ilb_host.cpp`, `Sched`): it works
    on the ledger directly and knows requests by the ledger's numbers and by their lengths.
    This class keeps the request objects (token values, sampling options), gives each
    request its number, and turns the library's answers into plans."""

    def __init__(self, cache: CacheManager, config: SchedulerConfig) -> None:
        self.cache = cache
        self.config = config
        self._lib = host.lib()
        h = ctypes.c_void_p()
        rc = self._lib.ilb_sched_new(cache.handle, config.max_num_seqs, config.max_num_batched_tokens,
                                     config.prefill_chunk_tokens, config.max_model_len, ctypes.byref(h))
        if rc:
            raise ValueError(host.last_error())
        self._h = h
        self._by_number: Dict[int, Request] = {}
        self.finished: Dict[Hashable, Request] = {}
        cap = max(config.max_num_seqs, 1) + 8
        self._work = (ctypes.c_longlong * (4 * cap))()
        self._victims = (ctypes.c_longlong * (4 * cap))()
        self._cap = cap

    def __del__(self) -> None:
        h = getattr(self, "_h", None)
        if h is not None and h.value:
            self._lib.ilb_sched_free(h)
            self._h = None

    def _message(self) -> str:
        """The library names requests by number; the message names them as the caller does."""
        return re.sub(r"request #(\d+)", lambda m: f"request {self._by_number[int(m.group(1))].id!r}"
                      if int(m.group(1)) in self._by_number else m.group(0), host.last_error())

    def _listed(self, which: int) -> List[Request]:
        n = self._lib.ilb_sched_list(self._h, which, self._victims, 0)
        if n == 0:
            return []
        buf = (ctypes.c_longlong * n)()
        self._lib.ilb_sched_list(self._h, which, buf, n)
        return [self._by_number[i] for i in buf]

    @property
    def waiting(self) -> List[Request]:
        return self._listed(0)

    @property
    def running(self) -> List[Request]:
        """In admission order."""
        return self._listed(1)

    @property
    def stats(self) -> Dict[str, int]:
        out = (ctypes.c_longlong * 6)()
        self._lib.ilb_sched_stats(self._h, out)
        return {"steps": out[0], "preemptions": out[1], "admitted": out[2], "finished": out[3]}

    def count_step(self) -> None:
        """A step that was launched without a plan of its own (the engine's lookahead)."""
        self._lib.ilb_sched_count_step(self._h)

    # ------------------------------------------------------------------ intake
    def add(self, request: Request) -> None:
        known = self.cache.ids.of(request.id) in self._by_number      # queued already: the library will refuse it
        number = self.cache.ids.pin(request.id)
        if not known:
            self._by_number[number] = request
        rc = self._lib.ilb_sched_add(self._h, number, len(request.prompt), int(request.max_new_tokens))
        if rc:
            msg = self._message()
            if not known:
                del self._by_number[number]
                self.cache.ids.unpin(request.id)
                if not self.cache.has(request.id):
                    self.cache.ids.forget(request.id)
            if rc == host.CAPACITY:
                raise CapacityError(msg)
            raise ValueError(msg)
        request.status = WAITING

    def has_work(self) -> bool:
        out = (ctypes.c_longlong * 6)()
        self._lib.ilb_sched_stats(self._h, out)
        return bool(out[4] or out[5])

    def counts(self):
        """(waiting, running)."""
        out = (ctypes.c_longlong * 6)()
        self._lib.ilb_sched_stats(self._h, out)
        return out[4], out[5]

    # ------------------------------------------------------------------ planning
    def plan(self) -> StepPlan:
        """One step.  If nothing can run although requests hold pages (every one of them
        blocked on pages the others hold), the youngest is preempted and the plan is made
        again, so the oldest request always makes progress."""
        c = self.config                     # the limits may be changed between steps
        if c.max_num_seqs + 8 > self._cap:
            self._cap = c.max_num_seqs + 8
            self._work = (ctypes.c_longlong * (4 * self._cap))()
            self._victims = (ctypes.c_longlong * (4 * self._cap))()
        if self._lib.ilb_sched_set_limits(self._h, c.max_num_seqs, c.max_num_batched_tokens, c.prefill_chunk_tokens,
                                          c.max_model_len) or \
                self._lib.ilb_sched_set_token_multiple(self._h, int(c.step_token_multiple)):
            raise ValueError(host.last_error())
        n_work, n_victims = ctypes.c_int(), ctypes.c_int()
        rc = self._lib.ilb_sched_plan(self._h, self._work, self._cap, ctypes.byref(n_work), self._victims,
                                      ctypes.byref(n_victims))
        plan = StepPlan()
        for i in range(n_victims.value):
            r = self._by_number[self._victims[i]]
            r.status = WAITING
            r.preemptions += 1
            self.cache.released_in_ledger(r.id)
            plan.preempted.append(r.id)
        if rc:
            msg = self._message()
            if rc == host.CAPACITY:
                raise CapacityError(msg)
            raise ValueError(msg)
        w = self._work
        for i in range(n_work.value):
            r = self._by_number[w[4 * i]]
            r.status = RUNNING
            plan.work.append(PlannedWork(r, w[4 * i + 1], w[4 * i + 2], bool(w[4 * i + 3])))
        return plan

    # ------------------------------------------------------------------ results
    def complete(self, plan: StepPlan, sampled: Dict[Hashable, int]) -> List[Request]:
        """Record the tokens drawn for the work that sampled; returns requests that
        finished (their pages are released here)."""
        done: List[Request] = []
        for w in plan.work:
            if not w.samples:
                continue
            r = w.request
            token = int(sampled[r.id])
            r.generated.append(token)
            number = self.cache.ids.of(r.id)
            reason = self._lib.ilb_sched_token(self._h, number, 1 if r.params.is_eos(token) else 0)
            if reason < 0:
                raise ValueError(self._message())
            if reason:
                r.status = FINISHED
                r.finish_reason = "eos" if reason == 1 else "length"
                self._retire(r, number)
                done.append(r)
        return done

    def _retire(self, r: Request, number: int) -> None:
        self.cache.ids.unpin(r.id)
        self.cache.released_in_ledger(r.id)
        self.cache.ids.forget(r.id)
        self._by_number.pop(number, None)
        self.finished[r.id] = r

    def abort(self, request_id: Hashable) -> None:
        for number, r in list(self._by_number.items()):
            if r.id == request_id and self._lib.ilb_sched_abort(self._h, number):
                r.status, r.finish_reason = FINISHED, "abort"
                self._retire(r, number)
