"""A stand-in for the engine on the CPU: the real cache manager, a step function that only
counts (next token = last token + 1). For scheduler tests; mirrors the reference's FakeExecutor
(tests/test_scheduler.py:31-54,914-929)."""
from types import SimpleNamespace

import torch

from damendaemon_b200.cache import CacheManager, PagedKeyValues


class FakeEngine:
    def __init__(self, kv_tokens=256, page_size=16, max_requests=4, max_context=128, vocab=100, eos=(9,), window=None):
        needs = [[PagedKeyValues(2, 16, None)], [PagedKeyValues(2, 16, window)]] if window else [[PagedKeyValues(2, 16, None)]]
        self.cache = CacheManager(needs, kv_tokens, page_size, max_requests, max_context)
        self.max_context = max_context
        self.spec = SimpleNamespace(vocab_size=vocab, eos_token_ids=tuple(eos))
        self.calls = []
        self.fail_next = None

    def reserve(self, request, total, max_step):
        fresh = request not in self.cache.slot_of
        if fresh:
            self.cache.admit(request)
        try:
            self.cache.reserve(request, total, max_step)
        except Exception:
            if fresh:
                self.cache.release(request)
            raise

    def finish(self, request):
        self.cache.release(request)

    def length(self, request):
        return self.cache.length.get(request, 0)

    def step(self, entries):
        if self.fail_next:
            error, self.fail_next = self.fail_next, None
            raise error
        fresh = [e.request for e in entries if e.request not in self.cache.slot_of]
        for r in fresh:
            self.cache.admit(r)
        try:
            self.cache.extend([(e.request, self.cache.length[e.request] + len(e.tokens)) for e in entries])
        except Exception:
            for r in fresh:
                self.cache.release(r)
            raise
        self.calls.append([(e.request, len(e.tokens), list(e.want)) for e in entries])
        rows = []
        for e in entries:
            self.cache.advance(e.request, self.cache.length[e.request] + len(e.tokens))
            for w in e.want:
                row = torch.zeros(self.spec.vocab_size)
                row[(e.tokens[w] + 1) % self.spec.vocab_size] = 1.0
                rows.append(row)
        self.cache.check()
        return torch.stack(rows) if rows else torch.zeros(0, self.spec.vocab_size)


def greedy_cpu(logits, samplers):
    return logits.argmax(-1).tolist()
