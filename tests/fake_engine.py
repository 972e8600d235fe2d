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
        self.ahead_calls = []        # per call: were the token values taken from the sampler's output?
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

    accepts_device_ids = True

    def step(self, entries, device_ids=None):
        """device_ids: the token values of the step (one per entry) as the sampler left them, in place of
        the entries' own: a list stands in for the device tensor."""
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
        self.ahead_calls.append(device_ids is not None)
        rows = []
        for i, e in enumerate(entries):
            self.cache.advance(e.request, self.cache.length[e.request] + len(e.tokens))
            tokens = e.tokens if device_ids is None else [int(device_ids[i])]
            for w in e.want:
                row = torch.zeros(self.spec.vocab_size)
                row[(tokens[w] + 1) % self.spec.vocab_size] = 1.0
                rows.append(row)
        self.cache.check()
        return torch.stack(rows) if rows else torch.zeros(0, self.spec.vocab_size)


def greedy_cpu(logits, samplers):
    return logits.argmax(-1).tolist()


class _Pending:
    def __init__(self, ids):
        self.ids = ids


def greedy_cpu_in_two_parts(logits, samplers):
    """The same choice, also offered as launch() and read(): the scheduler may then run ahead."""
    return logits.argmax(-1).tolist()


greedy_cpu_in_two_parts.launch = lambda logits, samplers: _Pending(logits.argmax(-1).tolist())
greedy_cpu_in_two_parts.read = lambda pending: list(pending.ids)
