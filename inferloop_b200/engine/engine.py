"""The Python entry point: `Engine(model, ...)`, `submit`, `step`, `generate`.

The reference has no Python in its serving path; its programming surface is the Rust
`Engine::{new, submit, tick, poll_completed, take_completed}`
(crates/engine/runtime/src/engine/mod.rs:118-159) driven by the `infer run` loop
`while !engine.is_idle() { engine.tick(now) }`
(crates/service/cli/src/support/execution.rs:16-46).  This class keeps those verbs and
the option names of its command line (crates/service/cli/src/arguments.rs:17-93):
block_size, num_gpu_blocks_override, max_num_batched_tokens, max_model_len,
max_output_tokens, max_num_seqs, gpu_memory_utilization, device.
"""
from __future__ import annotations

import dataclasses

import os
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Mapping, Optional, Sequence, Union

import torch

from ..sampling import host as host_sampler
from ..sampling.device import DeviceSampler
from ..sampling.defaults import GenerationDefaults
from ..sampling.params import SamplingParams
from .batch import StepEntry
from .runner import ModelRunner, parse_dtype, require_cuda
from .scheduler import CapacityError, PlannedWork, Request, Scheduler, SchedulerConfig, StepPlan

DEFAULT_BLOCK_SIZE = 16            # crates/engine/runtime/src/config.rs:19
DEFAULT_GPU_MEMORY_UTILIZATION = 0.9


@dataclass
class _Flight:
    """A step that is on the device."""
    plan: StepPlan
    sampling_work: list
    drawn: Optional[object]                     # `Drawn`: ids still on the device (plain greedy), or None
    sampled: Optional[Dict[Hashable, int]]      # ids on the host, once known
    dropped: set = field(default_factory=set)   # requests that ended before this step's ids were read


@dataclass
class TokenOutput:
    request: Hashable
    token: int
    index: int                  # index among the request's generated tokens
    finished: bool
    finish_reason: Optional[str] = None


class Engine:
    def __init__(self, model: Union[str, Mapping], dtype="bfloat16", device: Union[int, str] = 0,
                 block_size: int = DEFAULT_BLOCK_SIZE, num_gpu_blocks_override: Optional[int] = None,
                 max_num_batched_tokens: Optional[int] = None, max_model_len: Optional[int] = None,
                 max_output_tokens: Optional[int] = None, max_num_seqs: int = 64,
                 gpu_memory_utilization: float = DEFAULT_GPU_MEMORY_UTILIZATION,
                 prefill_chunk_tokens: int = 512, random_weights_seed: Optional[int] = None,
                 cuda_graphs: bool = True, device_timing: str = "off", runner=None) -> None:
        """`model`: a folder with config.json and safetensors, or a config mapping
        together with `random_weights_seed` (weights are then made on the device)."""
        self.block_size = int(block_size)
        self.max_output_tokens = max_output_tokens
        # what a request without sampling fields gets, and the folder's stop tokens
        # (generation_config.json / eos_token_id: crates/model/package/src/generation/read.rs:9-100)
        if isinstance(model, (str, os.PathLike)):
            self.generation_defaults = GenerationDefaults.from_folder(str(model))
        elif isinstance(model, Mapping):
            self.generation_defaults = GenerationDefaults.from_configs(model)
        else:
            self.generation_defaults = GenerationDefaults()
        if runner is not None:
            self.runner = runner
        else:
            dev = require_cuda(f"cuda:{device}" if isinstance(device, int) else device)
            dt = parse_dtype(dtype)
            pages = num_gpu_blocks_override
            first_pages = pages if pages is not None else 1
            if isinstance(model, (str, os.PathLike)):
                self.runner = ModelRunner.from_folder(
                    str(model), dtype=dt, device=dev, page_size=self.block_size,
                    num_pages=first_pages, max_requests=max(max_num_seqs, 1))
            else:
                if random_weights_seed is None:
                    raise ValueError("a config mapping needs random_weights_seed")
                self.runner = ModelRunner.from_config(
                    model, random_weights_seed, dtype=dt, device=dev, page_size=self.block_size,
                    num_pages=first_pages, max_requests=max(max_num_seqs, 1))
            if pages is None:
                step_tokens = max_num_batched_tokens or max(prefill_chunk_tokens + max_num_seqs - 1, 1)
                self.runner.resize_cache(self._pages_from_memory(dev, gpu_memory_utilization, max_num_seqs,
                                                                 max_model_len, step_tokens), max(max_num_seqs, 1))
        spec_len = self.runner.spec.max_positions
        self.max_model_len = min(int(max_model_len), spec_len) if max_model_len else spec_len
        cfg = SchedulerConfig(
            max_num_seqs=max_num_seqs,
            max_num_batched_tokens=max_num_batched_tokens or max(prefill_chunk_tokens + max_num_seqs - 1, 1),
            prefill_chunk_tokens=prefill_chunk_tokens, max_model_len=self.max_model_len,
            step_token_multiple=int(getattr(self.runner, "token_multiple", 1)))
        if device_timing != "off":
            self.runner.set_device_timing(device_timing)      # off | graph | node (engine/timing.py)
        self.scheduler = Scheduler(self.runner.cache, cfg)
        self.sampler = DeviceSampler(self.runner.device) if getattr(self.runner, "device", None) is not None else None
        self.cuda_graphs = cuda_graphs
        self._next_id = 0
        self._steps_since_check = 0
        self._ahead: Optional[_Flight] = None
        self.steps_launched_ahead = 0
        self.lookahead = True                   # launch the next decode step before reading this one's ids
        self.max_finished_kept = 1024
        self.step_log: Optional[List[dict]] = None   # set to a list to have every launched step described in it
        self.requests: Dict[Hashable, Request] = {}

    # ------------------------------------------------------------------ sizing
    def _pages_from_memory(self, dev, utilization: float, max_num_seqs: int,
                           max_model_len: Optional[int], step_tokens: int):
        """budget = min(total * utilization - used, free - 1 GiB)
        (crates/service/cli/src/backend/cuda.rs:52-64), less what the largest step's
        activations, logits and kernel scratch take: that is computed from the model's own
        sizes (`scratch_bytes`), with a quarter on top and 256 MiB for the fixed scratch of
        the kernels and the sampler."""
        free, total = torch.cuda.mem_get_info(dev)
        used = total - free
        budget = min(total * utilization - used, free - (1 << 30))
        reserve = self.runner.model.scratch_bytes(int(step_tokens), max(max_num_seqs, 1))
        self.activation_reserve = reserve + reserve // 4 + (256 << 20)
        budget -= self.activation_reserve
        groups = self.runner.cache.groups
        if not groups:
            return 1
        element = torch.empty((), dtype=self.runner.cache.dtype).element_size()
        want = (max_model_len or self.runner.spec.max_positions)
        # Pages one request holds at full length, per group: every key, or (with a window) the
        # window, the largest step's own tokens and a page of slack.  Every group gets room
        # for the same number of such requests; no set of requests can use more than
        # max_num_seqs of them.
        per_request = [-(-(want if g.need.window is None else min(want, g.need.window + int(step_tokens) + self.block_size))
                         // self.block_size) + (0 if g.need.window is None else 1) for g in groups]
        bytes_per_request = sum(n * g.page_bytes(element) for n, g in zip(per_request, groups))
        requests = min(max(budget, 0) / bytes_per_request, float(max(max_num_seqs, 1)))
        pages = [int(requests * n) for n in per_request]
        if min(pages) < 1:
            raise CapacityError("no device memory is left for the cache")
        return pages

    # ------------------------------------------------------------------ requests
    def submit(self, tokens: Sequence[int], sampling: Optional[SamplingParams] = None,
               max_new_tokens: int = 16, request_id: Optional[Hashable] = None,
               extras: Optional[Mapping[str, Sequence[int]]] = None) -> Hashable:
        """`extras`: for a model whose description declares per-token inputs beside ids and
        positions (`ModelSpec.token_extras`), their values for the prompt's tokens."""
        params = (self.generation_defaults.base if sampling is None
                  else self.generation_defaults.with_stop_tokens(sampling))
        if request_id is None:
            while self._next_id in self.requests:
                self._next_id += 1
            request_id = self._next_id
            self._next_id += 1
        elif request_id in self.requests and self.requests[request_id].status != "finished":
            raise ValueError(f"duplicate request id {request_id!r}")
        vocab = self.runner.spec.vocab_size
        toks = [int(t) for t in tokens]
        for t in toks:
            if not (0 <= t < vocab):
                raise ValueError(f"token {t} is outside the vocabulary of {vocab}")
        if self.max_output_tokens is not None:
            max_new_tokens = min(max_new_tokens, int(self.max_output_tokens))
        req = Request(request_id, toks, params, int(max_new_tokens))
        declared = getattr(getattr(self.runner, "spec", None), "token_extras", ()) or ()
        if declared:
            req.extras = {k: [int(x) for x in v] for k, v in (extras or {}).items()}
            for name, width in declared:
                req.extras_of(name, int(width), 0, 0)          # raises if the prompt's values are missing
        self.scheduler.add(req)
        self.requests[request_id] = req
        # finished requests stay readable (`result`) until taken (`take_completed`); beyond
        # `max_finished_kept` the oldest are forgotten so that a long run does not grow
        finished = self.scheduler.finished
        while len(finished) > self.max_finished_kept:
            old = next(iter(finished))
            del finished[old]
            self.requests.pop(old, None)
        return request_id

    def abort(self, request_id: Hashable) -> None:
        """End a request now (the reference's cancel: its resources are released at once,
        crates/engine/runtime/src/pipeline/lifecycle.rs:242-251)."""
        if self._ahead is not None:
            self._ahead.dropped.add(request_id)
        self.scheduler.abort(request_id)

    def is_idle(self) -> bool:
        return not self.scheduler.has_work()

    # ------------------------------------------------------------------ one step
    def step(self) -> List[TokenOutput]:
        """Plan one step, run it, draw the tokens it yields; returns them.

        While the device runs a greedy decode step, the step after it is usually known
        already: the same requests, each with whatever token this step draws.  That step is
        then launched before this step's ids are read back (its tokens are copied on the
        device), so the device does not wait for the host between steps.  If a request
        turns out to have finished (an end-of-sequence token), its row of the step already
        running is computed in vain and dropped."""
        flight = self._ahead
        self._ahead = None
        if flight is None:
            flight = self._launch()
            if flight is None:
                return []
        if flight.sampled is None:
            handle = self.sampler.start_read(flight.drawn)
            self._ahead = self._launch_ahead(flight)
            ids = self.sampler.finish_read(handle)
            flight.sampled = {w.request.id: t for w, t in zip(flight.sampling_work, ids)}
        # a kernel that gave up a bounded wait leaves a flag on the device; looking costs a
        # small read, so it is done now and then and at the end of generate()
        self._steps_since_check += 1
        if self.sampler is not None and self._steps_since_check >= 64:
            self.check_device()
        plan, work = flight.plan, flight.sampling_work
        if flight.dropped:
            work = [w for w in work if w.request.id not in flight.dropped]
            plan = StepPlan([w for w in plan.work if w.request.id not in flight.dropped], plan.preempted)
        finished = {r.id for r in self.scheduler.complete(plan, flight.sampled)}
        if self._ahead is not None:
            self._ahead.dropped |= finished
            if all(w.request.id in self._ahead.dropped for w in self._ahead.plan.work):
                self._ahead = None               # nothing of it is wanted any more
        out = []
        for w in work:
            r = w.request
            out.append(TokenOutput(r.id, flight.sampled[r.id], len(r.generated) - 1, r.id in finished,
                                   r.finish_reason if r.id in finished else None))
        return out

    def _launch(self) -> Optional["_Flight"]:
        """Plan a step and put it on the device.  Plain greedy steps come back with their
        ids still on the device; every other kind is sampled before returning."""
        plan = self.scheduler.plan()
        if not plan.work:
            return None
        if self.step_log is not None:
            self.step_log.append(self._describe(plan.work, len(plan.preempted)))
        declared = getattr(getattr(self.runner, "spec", None), "token_extras", ()) or ()
        entries = [StepEntry(w.request.id, w.tokens, [w.count - 1] if w.samples else [],
                             {name: w.request.extras_of(name, int(width), w.start, w.count) for name, width in declared}
                             if declared else None) for w in plan.work]
        sampling_work = [w for w in plan.work if w.samples]
        if (self.sampler is not None and sampling_work
                and all(w.request.params.uses_plain_greedy() for w in sampling_work)):
            # the arg-max rides in the step's own launch sequence; only ids come back
            _, drawn = self.runner.step(entries, draw_greedy=True)
            return _Flight(plan, sampling_work, drawn, None)
        logits = self.runner.step(entries)
        return _Flight(plan, sampling_work, None, self._sample(logits, sampling_work))

    def _launch_ahead(self, flight: "_Flight") -> Optional["_Flight"]:
        """Launch the step after `flight` if it is certain what it holds: `flight` is a
        decode step of every running request, nobody waits, and nobody can reach a length
        limit with the token being drawn.  (A stop token may still end a request; its row
        is then dropped.)"""
        if not self.cuda_graphs or self.lookahead is False or getattr(self.runner, "step_ahead", None) is None:
            return None
        s = self.scheduler
        work = flight.plan.work
        n_waiting, n_running = s.counts()
        if (flight.plan.preempted or n_waiting or len(work) != n_running or flight.dropped
                or len(flight.sampling_work) != len(work)):
            return None
        for w in work:
            r = w.request
            if (w.count != 1 or len(r.generated) + 2 > r.max_new_tokens
                    or r.total_len() + 2 > s.config.max_model_len or not r.params.uses_plain_greedy()):
                return None
        entries = [StepEntry(w.request.id, [0], [0]) for w in work]
        drawn = self.runner.step_ahead(entries, flight.drawn)
        if drawn is None:
            return None
        s.count_step()
        self.steps_launched_ahead += 1
        nxt = [PlannedWork(w.request, w.start + 1, 1, True) for w in work]
        if self.step_log is not None:
            self.step_log.append(self._describe(nxt, 0))
        return _Flight(StepPlan(nxt, []), nxt, drawn, None)

    @staticmethod
    def _describe(work, preempted: int) -> dict:
        """What a step holds, for measurements: tokens, sequences, how many of them bring one
        token, keys in the cache after it, (query, key) pairs its attention covers, logits rows."""
        return {"tokens": sum(w.count for w in work), "seqs": len(work),
                "single_token_seqs": sum(1 for w in work if w.count == 1),
                "keys": sum(w.start + w.count for w in work),
                "pairs": sum(w.count * w.start + w.count * (w.count + 1) // 2 for w in work),
                "logit_rows": sum(1 for w in work if w.samples), "preempted": preempted}

    def _sample(self, logits: torch.Tensor, work) -> Dict[Hashable, int]:
        """Row i of `logits` belongs to work[i].  Every row is drawn on the device: the
        highest logit, or a draw after the reference's penalties and filters (top-k, min-p,
        top-p).  Only over a vocabulary the filtering kernel is not built for are rows with
        filters or penalties read back and drawn by the host sampler.
        The draw's position is the index of the token being generated
        (crates/engine/runtime/src/pipeline/completion/cpu.rs:104)."""
        if not work:
            return {}
        rows = len(work)
        out: Dict[Hashable, int] = {}
        filters_fit = self._filters_fit(logits.shape[1])
        kinds = ["greedy" if w.request.params.uses_plain_greedy()
                 else "temperature" if (w.request.params.uses_plain_temperature() or filters_fit) else "host" for w in work]
        if self.sampler is None:
            kinds = ["host"] * rows
        if "greedy" in kinds:
            self.sampler.greedy_launch(logits)
            ids = self.sampler.read(rows)
            for w, k, t in zip(work, kinds, ids):
                if k == "greedy":
                    out[w.request.id] = t
        if "temperature" in kinds:
            # a row without a temperature but with penalties is the best of the penalised logits: top-k 1
            plain = SamplingParams(temperature=1.0)
            drawn_with = [plain if k != "temperature" else w.request.params if w.request.params.temperature > 0.0
                          else dataclasses.replace(w.request.params, temperature=1.0, top_k=1, top_p=1.0, min_p=0.0)
                          for w, k in zip(work, kinds)]
            temps = [p.temperature for p in drawn_with]
            us = [host_sampler.uniform(w.request.params.seed, host_sampler.request_key(w.request.id),
                                       len(w.request.generated)) for w in work]
            histories = [(w.request.prompt, w.request.generated) if k == "temperature" else None for w, k in zip(work, kinds)]
            self.sampler.temperature_launch(logits, temps, us, drawn_with, histories)
            ids = self.sampler.read(rows)
            for w, k, t in zip(work, kinds, ids):
                if k == "temperature":
                    out[w.request.id] = t
        if "host" in kinds:
            idx = [i for i, k in enumerate(kinds) if k == "host"]
            host = logits[idx].float().cpu().numpy() if hasattr(logits, "cpu") else logits[idx]
            for j, i in enumerate(idx):
                r = work[i].request
                out[r.id] = host_sampler.sample(
                    host[j], r.params, host_sampler.request_key(r.id), len(r.generated),
                    prompt=r.prompt, generated=r.generated)
        return out

    def _filters_fit(self, vocab: int) -> bool:
        """Whether the device draws with filters over a vocabulary of this size."""
        if self.sampler is None:
            return False
        if getattr(self, "_filter_max_vocab", None) is None:
            from ..csrc import ops
            self._filter_max_vocab = ops.sample_filter_max_vocab()
        return vocab <= self._filter_max_vocab

    def check_device(self) -> None:
        """Raise if any kernel reported that it gave up waiting (its outputs are invalid)."""
        from ..csrc import ops
        self._steps_since_check = 0
        ops.check_device_errors()

    # ------------------------------------------------------------------ whole jobs
    def generate(self, prompts: Sequence[Sequence[int]], sampling: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 max_new_tokens: Union[int, Sequence[int]] = 16) -> List[List[int]]:
        """Generate for every prompt (token ids in, token ids out); returns the generated
        tokens in the order of the prompts."""
        n = len(prompts)
        params = list(sampling) if isinstance(sampling, (list, tuple)) else [sampling] * n
        limits = list(max_new_tokens) if isinstance(max_new_tokens, (list, tuple)) else [max_new_tokens] * n
        ids = [self.submit(p, s, m) for p, s, m in zip(prompts, params, limits)]
        while not self.is_idle():
            self.step()
        if self.sampler is not None:
            self.check_device()
        return [list(self.requests[i].generated) for i in ids]

    def result(self, request_id: Hashable) -> Request:
        return self.requests[request_id]

    def take_completed(self) -> List[Request]:
        """Hand over every finished request and forget it (the reference's
        `Engine::take_completed`, crates/engine/runtime/src/engine/mod.rs:118-159): a
        long-running caller drains results this way, so that the engine's memory does not
        grow with the number of requests it has served."""
        done = list(self.scheduler.finished.values())
        for r in done:
            self.requests.pop(r.id, None)
        self.scheduler.finished.clear()
        return done

    def inspect(self) -> dict:
        """Counterpart of the reference's RuntimeInspection
        (crates/engine/runtime/src/engine/mod.rs:49-90)."""
        s = self.scheduler
        return {
            "waiting": len(s.waiting), "running": len(s.running), "finished": len(s.finished),
            "steps": getattr(self.runner, "steps_run", 0), "tokens": getattr(self.runner, "tokens_run", 0),
            "scheduler": dict(s.stats), "steps_launched_ahead": self.steps_launched_ahead,
            "cache": self.runner.cache.inspect(),
            "max_model_len": self.max_model_len,
            "max_num_seqs": s.config.max_num_seqs,
            "max_num_batched_tokens": s.config.max_num_batched_tokens,
            **({"device_timing": self.runner.timer.summary()}
               if getattr(getattr(self.runner, "timer", None), "mode", "off") != "off" else {}),
        }
