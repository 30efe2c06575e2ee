"""A runner that executes nothing: it keeps the cache ledger as the real one does and
returns logits that are a pure function of the request's tokens so far, so any schedule
must yield the same tokens.  (The reference tests its scheduler against a `ProtocolBackend`
double in the same spirit: crates/engine/runtime/tests/support/mod.rs:8-16.)"""
from __future__ import annotations

import hashlib
from types import SimpleNamespace

import numpy as np

from inferloop_b200.cache import CacheManager, OutOfPages
from inferloop_b200.parts.base import CacheNeeds, PagedKVNeed


class FakeRunner:
    device = None

    def __init__(self, vocab=50, page_size=4, num_pages=16, max_requests=8, max_positions=512, window=None):
        needs = [CacheNeeds(paged=PagedKVNeed(1, 16, None)), CacheNeeds(paged=PagedKVNeed(1, 16, window))]
        self.cache = CacheManager(needs, page_size, num_pages, max_requests)
        self.spec = SimpleNamespace(vocab_size=vocab, max_positions=max_positions)
        self.history = {}
        self.steps = []
        self.steps_run = 0
        self.tokens_run = 0

    def step(self, entries):
        for e in entries:
            if not self.cache.has(e.request):
                self.cache.begin(e.request)
                self.history[e.request] = []
        need = {}
        for e in entries:
            for g, n in self.cache.pages_needed(e.request, self.cache.length(e.request) + len(e.tokens)).items():
                need[g] = need.get(g, 0) + n
        free = self.cache.free_pages()
        assert all(need[g] <= free[g] for g in free), f"the plan does not fit the pages: {need} vs {free}"
        rows = []
        for e in entries:
            cur = self.cache.length(e.request)
            assert cur == len(self.history[e.request]), "tokens must continue the request's cursor"
            self.cache.ensure(e.request, cur + len(e.tokens))
            self.history[e.request] += list(e.tokens)
            for w in e.want:
                seq = tuple(self.history[e.request][:cur + w + 1])
                h = hashlib.sha256(repr(seq).encode()).digest()
                rng = np.random.default_rng(int.from_bytes(h[:8], "little"))
                rows.append(rng.standard_normal(self.spec.vocab_size).astype(np.float32))
            self.cache.commit(e.request, cur + len(e.tokens))
        self.steps.append([(e.request, len(e.tokens)) for e in entries])
        self.steps_run += 1
        self.tokens_run += sum(len(e.tokens) for e in entries)
        self.cache.check()
        # forget requests the scheduler released (preempted or finished)
        for r in list(self.history):
            if not self.cache.has(r):
                del self.history[r]
        return np.stack(rows) if rows else np.zeros((0, self.spec.vocab_size), np.float32)
