"""Continuous batching above the step function.

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
    else it waits (crates/engine/scheduler/src/policy/packing.rs:328-347);
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

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 64               # reference default: the submission batch limit
    max_num_batched_tokens: int = 2048
    prefill_chunk_tokens: int = 512
    max_model_len: int = 4096

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
    def __init__(self, cache: CacheManager, config: SchedulerConfig) -> None:
        self.cache = cache
        self.config = config
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []          # in admission order
        self.finished: Dict[Hashable, Request] = {}
        self._arrivals = 0
        self.stats = {"steps": 0, "preemptions": 0, "admitted": 0, "finished": 0}

    # ------------------------------------------------------------------ intake
    def add(self, request: Request) -> None:
        if request.max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be positive")
        if not request.prompt:
            raise ValueError("empty input")
        if any(r.id == request.id for r in self.waiting) or any(r.id == request.id for r in self.running):
            raise ValueError(f"request id {request.id!r} is already queued")
        total = len(request.prompt) + request.max_new_tokens
        if total > self.config.max_model_len:
            # reserved_tokens = prompt + max_new_tokens must fit the context
            # (crates/engine/workloads/src/native.rs:91-111)
            raise ValueError(f"request {request.id!r}: prompt {len(request.prompt)} + max_new_tokens "
                             f"{request.max_new_tokens} exceeds max_model_len {self.config.max_model_len}")
        pages = -(-total // self.cache.page_size)
        for g in self.cache.groups:
            reach = pages if g.need.window is None else min(
                pages, -(-(g.need.window + self.config.prefill_chunk_tokens) // self.cache.page_size) + 1)
            if reach > g.pool.num_pages:
                raise CapacityError(f"request {request.id!r} needs {reach} pages of group {g.index}, "
                                    f"the pool has {g.pool.num_pages}")
        request.arrival = self._arrivals
        self._arrivals += 1
        request.status = WAITING
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ planning
    def _computed(self, r: Request) -> int:
        return self.cache.length(r.id) if self.cache.has(r.id) else 0

    def _pages_for(self, r: Request, new_len: int) -> Dict[int, int]:
        if self.cache.has(r.id):
            return self.cache.pages_needed(r.id, new_len)
        return {g.index: -(-new_len // self.cache.page_size) for g in self.cache.groups}

    def _preempt(self, victim: Request, plan: StepPlan) -> None:
        """Recompute preemption: give everything back, restart its prefill later."""
        if self.cache.has(victim.id):
            self.cache.release(victim.id)
        self.running.remove(victim)
        victim.status = WAITING
        victim.preemptions += 1
        self.waiting.appendleft(victim)       # it keeps its place ahead of newer arrivals
        plan.preempted.append(victim.id)
        self.stats["preemptions"] += 1

    def plan(self) -> StepPlan:
        """One step.  If nothing can run although requests hold pages (every one of them
        blocked on pages the others hold), the youngest is preempted and the plan is made
        again, so the oldest request always makes progress."""
        plan = StepPlan()
        while True:
            self._fill(plan)
            if plan.work or not self.running:
                break
            if len(self.running) == 1:
                raise CapacityError(
                    f"request {self.running[0].id!r} cannot grow: the cache is too small for it alone")
            self._preempt(self.running[-1], plan)
        if not plan.work and self.waiting and not self.running:
            raise CapacityError(
                f"request {self.waiting[0].id!r} cannot start: the cache is too small for it alone")
        if plan.work:
            self.stats["steps"] += 1
        return plan

    def _held(self, r: Request) -> Dict[int, int]:
        if not self.cache.has(r.id):
            return {}
        return {g.index: sum(1 for p in self.cache.block_table(g.index, r.id) if p >= 0)
                for g in self.cache.groups}

    def _fill(self, plan: StepPlan) -> None:
        cfg = self.config
        budget = cfg.max_num_batched_tokens
        free = dict(self.cache.free_pages())
        page = self.cache.page_size

        def fits(need: Dict[int, int]) -> bool:
            return all(need.get(g, 0) <= free[g] for g in free)

        def charge(need: Dict[int, int]) -> None:
            for g, n in need.items():
                free[g] -= n

        def planned(r: Request) -> bool:
            return any(w.request is r for w in plan.work)

        def is_decode(r: Request) -> bool:
            return self._computed(r) == r.total_len() - 1

        # 1. decoding requests, oldest first; a blocked one preempts the youngest running
        for r in [r for r in self.running if is_decode(r)]:
            if r not in self.running:          # became a victim meanwhile
                continue
            if budget <= 0 or len(plan.work) >= cfg.max_num_seqs:
                break
            need = self._pages_for(r, r.total_len())
            while not fits(need):
                victims = [v for v in reversed(self.running) if v is not r and not planned(v)]
                if not victims:
                    break
                held = self._held(victims[0])
                self._preempt(victims[0], plan)
                for g, n in held.items():
                    free[g] += n
            if not fits(need):
                continue                       # waits; something else may finish first
            charge(need)
            plan.work.append(PlannedWork(r, r.total_len() - 1, 1, True))
            budget -= 1

        # 2. prompt portions: requests already running, then new arrivals in order
        def grant(r: Request) -> Optional[PlannedWork]:
            nonlocal budget
            done = self._computed(r)
            portion = min(cfg.prefill_chunk_tokens, r.total_len() - done)
            if budget >= portion:
                count = portion
            elif budget >= 1 and budget * 2 >= portion:
                count = budget
            else:
                return None
            need = self._pages_for(r, done + count)
            if not fits(need):
                # take what the free pages can hold, if that is still progress
                held = self._held(r)
                room = min((len(self.cache.block_table(g.index, r.id)) if self.cache.has(r.id) else 0)
                           + free[g.index] for g in self.cache.groups) * page if self.cache.groups else done + count
                count = min(count, room - done)
                if count <= 0:
                    return None
                need = self._pages_for(r, done + count)
                if not fits(need):
                    return None
            charge(need)
            budget -= count
            return PlannedWork(r, done, count, done + count == r.total_len())

        for r in list(self.running):
            if planned(r) or is_decode(r):
                continue
            if budget <= 0 or len(plan.work) >= cfg.max_num_seqs:
                break
            w = grant(r)
            if w is not None:
                plan.work.append(w)

        while (self.waiting and budget > 0 and len(plan.work) < cfg.max_num_seqs
               and len(self.running) < cfg.max_num_seqs and self.cache.slots.num_free > len(
                   [w for w in plan.work if not self.cache.has(w.request.id)])):
            r = self.waiting[0]
            if r.id in plan.preempted and self.running:
                break          # a victim of this very step waits for the next one
            w = grant(r)
            if w is None:
                break          # first come first served: nobody overtakes the head
            self.waiting.popleft()
            r.status = RUNNING
            self.running.append(r)
            self.stats["admitted"] += 1
            plan.work.append(w)

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
            reason = None
            if r.params.is_eos(token):
                reason = "eos"
            elif len(r.generated) >= r.max_new_tokens:
                reason = "length"
            elif r.total_len() >= self.config.max_model_len:
                reason = "length"
            if reason is not None:
                r.status = FINISHED
                r.finish_reason = reason
                self.running.remove(r)
                if self.cache.has(r.id):
                    self.cache.release(r.id)
                self.finished[r.id] = r
                self.stats["finished"] += 1
                done.append(r)
        return done

    def abort(self, request_id: Hashable) -> None:
        for r in list(self.running):
            if r.id == request_id:
                self.running.remove(r)
                if self.cache.has(r.id):
                    self.cache.release(r.id)
                r.status, r.finish_reason = FINISHED, "abort"
                self.finished[r.id] = r
        for r in list(self.waiting):
            if r.id == request_id:
                self.waiting.remove(r)
                r.status, r.finish_reason = FINISHED, "abort"
                self.finished[r.id] = r
