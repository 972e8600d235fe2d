"""The scheduler's decisions, with a counting stand-in for the engine and the real cache manager."""
import pytest

from damendaemon_b200.engine.scheduler import Request, Scheduler
from fake_engine import FakeEngine, greedy_cpu, greedy_cpu_in_two_parts


def make(engine=None, **kw):
    engine = engine or FakeEngine()
    return engine, Scheduler(engine, sample_fn=greedy_cpu, **kw)


def drain(s):
    return list(s.run())


def test_one_request_counts_up_and_frees():
    engine, s = make()
    r = s.submit(Request([1, 2, 3], max_tokens=4, ignore_eos=True))
    events = drain(s)
    assert r.output == [4, 5, 6, 7] and r.finish_reason == "length"
    assert [e.token for e in events] == [4, 5, 6, 7] and events[-1].finished
    assert engine.cache.used_tokens == 0 and not engine.cache.slot_of


def test_eos_stops_unless_ignored():
    engine, s = make()
    a = s.submit(Request([7], max_tokens=10))
    b = s.submit(Request([7], max_tokens=5, ignore_eos=True))
    drain(s)
    assert a.output == [8, 9] and a.finish_reason == "stop"
    assert b.output == [8, 9, 10, 11, 12] and b.finish_reason == "length"


def test_portions_under_a_token_budget_and_decodes_first():
    engine, s = make(FakeEngine(kv_tokens=512, max_context=128), token_budget=16, chunk_size=10)
    a = s.submit(Request(list(range(1, 4)), max_tokens=6, ignore_eos=True))
    b = s.submit(Request(list(range(20, 45)), max_tokens=2, ignore_eos=True))
    drain(s)
    # step 0: a whole (3) and b's first 10; step 1: a decodes beside b's next 10; ...
    assert engine.calls[0] == [(a.id, 3, [2]), (b.id, 10, [])]
    assert engine.calls[1] == [(a.id, 1, [0]), (b.id, 10, [])]
    assert engine.calls[2] == [(a.id, 1, [0]), (b.id, 5, [4])]
    assert all(sum(n for _, n, _ in call) <= 16 for call in engine.calls)
    assert b.output == [45, 46] and a.output == [4, 5, 6, 7, 8, 9]


def test_budget_is_shared_in_admission_order():
    engine, s = make(FakeEngine(kv_tokens=512), token_budget=8)
    rs = [s.submit(Request(list(range(10, 16)), max_tokens=1, ignore_eos=True)) for _ in range(3)]
    s.step()
    assert engine.calls[0] == [(rs[0].id, 6, [5]), (rs[1].id, 2, [])]


def test_queue_waits_for_pages_in_order_then_reuses_them():
    # pool of 4 pages (64 tokens): each request reserves 3 pages
    engine, s = make(FakeEngine(kv_tokens=64, max_requests=4), token_budget=64)
    a = s.submit(Request([1] * 30, max_tokens=10, ignore_eos=True))
    b = s.submit(Request([2] * 30, max_tokens=10, ignore_eos=True))
    c = s.submit(Request([3], max_tokens=1, ignore_eos=True))        # small, but must not overtake b
    s.step()
    assert [r.id for r in s.live()] == [a.id] and list(s.waiting) == [b, c]
    drain(s)
    assert all(r.finish_reason == "length" for r in (a, b, c))
    first_b = next(i for i, call in enumerate(engine.calls) if any(r == b.id for r, _, _ in call))
    first_c = next(i for i, call in enumerate(engine.calls) if any(r == c.id for r, _, _ in call))
    last_a = max(i for i, call in enumerate(engine.calls) if any(r == a.id for r, _, _ in call))
    assert first_b > last_a and first_c >= first_b
    assert engine.cache.used_tokens == 0


def test_request_larger_than_the_pool_fails_at_once():
    engine, s = make(FakeEngine(kv_tokens=32, max_context=128))
    big = s.submit(Request([1] * 40, max_tokens=8))
    small = s.submit(Request([1, 2], max_tokens=2, ignore_eos=True))
    events = drain(s)
    assert big.finish_reason == "error" and "pages" in big.error
    assert small.output == [3, 4]
    assert any(e.request is big and e.token is None and e.finished for e in events)


def test_length_policy():
    engine, s = make(FakeEngine(max_context=32, kv_tokens=64))
    with pytest.raises(ValueError, match="exceeds"):
        s.submit(Request([1] * 30, max_tokens=10))
    engine, s = make(FakeEngine(max_context=32, kv_tokens=64), length_policy="clamp")
    r = s.submit(Request([1] * 30, max_tokens=10, ignore_eos=True))
    drain(s)
    assert len(r.output) == 2 and r.finish_reason == "length"
    for bad in (Request([], 1), Request([1000], 1), Request([1], 0), Request("ab", 1)):
        with pytest.raises(ValueError):
            s.submit(bad)


def test_failed_step_fails_its_requests_and_frees_them():
    engine, s = make(FakeEngine(kv_tokens=256))
    a = s.submit(Request([1, 2], max_tokens=5, ignore_eos=True))
    s.step()
    engine.fail_next = RuntimeError("boom")
    b = s.submit(Request([5], max_tokens=2, ignore_eos=True))
    events = s.step()
    assert a.finish_reason == b.finish_reason == "error" and "boom" in a.error
    assert engine.cache.used_tokens == 0 and not engine.cache.slot_of
    c = s.submit(Request([5], max_tokens=2, ignore_eos=True))
    drain(s)
    assert c.output == [6, 7]


def test_without_reservations_the_youngest_waits_and_at_worst_fails():
    # 4 pages; two requests that together outgrow them while decoding
    engine, s = make(FakeEngine(kv_tokens=64, max_context=64), reserve=False, token_budget=64)
    a = s.submit(Request([1] * 30, max_tokens=30, ignore_eos=True))
    b = s.submit(Request([2] * 30, max_tokens=30, ignore_eos=True))
    drain(s)
    assert a.finish_reason == "length" and len(a.output) == 30      # the oldest always gets through
    assert b.finish_reason == "error" and b.error == "cache_full"
    assert engine.cache.used_tokens == 0
    engine.cache.check()


def test_max_live_and_slots():
    engine, s = make(FakeEngine(kv_tokens=1024, max_requests=2), max_live=8)
    rs = [s.submit(Request([i + 1], max_tokens=3, ignore_eos=True)) for i in range(5)]
    s.step()
    assert len(s.live()) == 2
    drain(s)
    assert [r.output for r in rs] == [[i + 2, i + 3, i + 4] for i in range(5)]


def test_window_group_gives_pages_back_while_running():
    engine, s = make(FakeEngine(kv_tokens=128, max_context=128, window=20), token_budget=16)
    r = s.submit(Request([1] * 100, max_tokens=20, ignore_eos=True))
    drain(s)
    full, window = engine.cache.groups
    assert full.pool.high_water_pages == 8 and window.pool.high_water_pages <= 4
    assert r.finish_reason == "length" and engine.cache.used_tokens == 0


# ---------------------------------------------------------------- running one decode step ahead

def make_ahead(engine=None, **kw):
    engine = engine or FakeEngine()
    return engine, Scheduler(engine, sample_fn=greedy_cpu_in_two_parts, **kw)


def test_running_ahead_gives_the_same_tokens_in_the_same_order():
    prompts = [([1, 2, 3], 9), ([20], 5), ([40, 41], 12)]
    runs = []
    for ahead in (False, True):
        engine, s = make_ahead(FakeEngine(kv_tokens=512), run_ahead=ahead)
        rs = [s.submit(Request(list(p), max_tokens=n, ignore_eos=True)) for p, n in prompts]
        events = drain(s)
        runs.append(([r.output for r in rs], [(rs.index(e.request), e.token, e.finished) for e in events], s.steps))
        assert (s.steps_ahead > 0) == ahead
        assert any(engine.ahead_calls) == ahead
        assert engine.cache.used_tokens == 0 and not engine.cache.slot_of
    assert runs[0] == runs[1]


def test_running_ahead_stops_before_a_request_can_end_by_length():
    engine, s = make_ahead()
    r = s.submit(Request([1, 2, 3], max_tokens=4, ignore_eos=True))
    drain(s)
    assert r.output == [4, 5, 6, 7] and r.finish_reason == "length"
    # the prompt, the first decode step, then two steps launched before the tokens of the step before were read; the
    # last of them samples the token with which the request ends, so nothing is launched after it
    assert len(engine.calls) == 4 and engine.ahead_calls == [False, False, True, True]


def test_end_of_sequence_while_running_ahead_drops_one_row():
    engine, s = make_ahead(FakeEngine(kv_tokens=512))
    a = s.submit(Request([5], max_tokens=20))                       # 6, 7, 8, 9 = end of sequence
    b = s.submit(Request([30], max_tokens=8, ignore_eos=True))
    events = drain(s)
    assert a.output == [6, 7, 8, 9] and a.finish_reason == "stop"
    assert b.output == list(range(31, 39)) and b.finish_reason == "length"
    assert [e.token for e in events if e.request is a] == [6, 7, 8, 9]
    # a took part in one step after its last token: that step had been launched already
    assert sum(1 for call in engine.calls for (rid, n, want) in call if rid == a.id) == 5
    assert engine.cache.used_tokens == 0 and not engine.cache.slot_of


def test_a_request_that_arrives_while_running_ahead_joins_after_the_step_in_flight():
    engine, s = make_ahead(FakeEngine(kv_tokens=512))
    a = s.submit(Request([1], max_tokens=30, ignore_eos=True))
    for _ in range(4):
        s.step()
    assert s.steps_ahead >= 2
    b = s.submit(Request([50, 51], max_tokens=3, ignore_eos=True))
    drain(s)
    assert a.output == list(range(2, 32)) and b.output == [52, 53, 54]
    assert engine.cache.used_tokens == 0


def test_a_failing_step_ahead_fails_its_requests_only_once():
    engine, s = make_ahead(FakeEngine(kv_tokens=512))
    a = s.submit(Request([1], max_tokens=30, ignore_eos=True))
    s.step()
    engine.fail_next = RuntimeError("device lost")
    events = s.step() + drain(s)
    assert a.finish_reason == "error" and "device lost" in a.error
    assert sum(1 for e in events if e.request is a and e.token is None) == 1
    assert engine.cache.used_tokens == 0 and not engine.cache.slot_of


def test_running_ahead_goes_on_while_the_queue_is_blocked_and_admission_follows_the_end():
    # pool of 4 pages (64 tokens): each request reserves 3 pages, so b waits until a has ended
    engine, s = make_ahead(FakeEngine(kv_tokens=64, max_requests=4), token_budget=64)
    a = s.submit(Request([1] * 30, max_tokens=10, ignore_eos=True))
    b = s.submit(Request([2] * 30, max_tokens=10, ignore_eos=True))
    drain(s)
    assert a.output == list(range(2, 12)) and b.output == list(range(3, 13))
    first_b = next(i for i, call in enumerate(engine.calls) if any(rid == b.id for rid, _, _ in call))
    assert any(engine.ahead_calls[:first_b]), "a's decode steps did not run ahead while b waited"
    assert all(rid == a.id for call in engine.calls[:first_b] for rid, _, _ in call)
    assert engine.cache.used_tokens == 0 and not engine.cache.slot_of


def test_a_prompt_is_cut_at_the_multiples_the_engine_asks_for():
    engine = FakeEngine(kv_tokens=2048, max_context=1024)
    engine.portion_multiple = 128
    _, s = make(engine, token_budget=300)
    a = s.submit(Request(list(range(1, 91)) * 7 + [5] * 70, max_tokens=2, ignore_eos=True))       # 700 tokens
    drain(s)
    assert [call[0][1] for call in engine.calls[:3]] == [256, 256, 188]
    assert len(a.output) == 2
    # a portion no longer than the multiple is left as the budget cuts it
    engine = FakeEngine(kv_tokens=2048, max_context=1024)
    engine.portion_multiple = 128
    _, s = make(engine, token_budget=100)
    s.submit(Request([3] * 250, max_tokens=1, ignore_eos=True))
    drain(s)
    assert [call[0][1] for call in engine.calls] == [100, 100, 50]


@pytest.mark.parametrize("seed", range(8))
def test_running_ahead_under_random_arrivals_and_ends(seed):
    """Random prompts, lengths, ends of sequence (the stand-in counts up and 9 ends a sequence) and arrivals between
    steps, with a pool that makes requests wait: every request gets the same tokens and the same end with and
    without running ahead, nothing is lost from the cache, and steps were in fact launched ahead."""
    import random
    outcomes = []
    for ahead in (False, True):
        rng = random.Random(seed)
        engine, s = make_ahead(FakeEngine(kv_tokens=160, max_requests=3, max_context=64), token_budget=48, run_ahead=ahead)
        requests, arrivals = [], sorted(rng.randrange(0, 40) for _ in range(10))
        step = 0
        while arrivals or not s.idle:
            while arrivals and arrivals[0] <= step:
                arrivals.pop(0)
                prompt = [rng.randrange(0, 100) for _ in range(rng.randrange(1, 30))]
                requests.append(s.submit(Request(prompt, max_tokens=rng.randrange(1, 25), ignore_eos=rng.random() < 0.3)))
            s.step()
            engine.cache.check()
            step += 1
            assert step < 2000
        assert engine.cache.used_tokens == 0 and not engine.cache.slot_of
        outcomes.append([(r.output, r.finish_reason) for r in requests])
        if ahead:
            assert s.steps_ahead > 0
    assert outcomes[0] == outcomes[1]


# ---------------------------------------------------------------- withdrawing a request; waiting too long

class Clock:
    def __init__(self):
        self.now = 0.0

    def __call__(self):
        return self.now


def ended(events, request):
    return [e for e in events if e.request is request and e.finished and e.token is None]


def test_cancel_while_waiting_lets_the_next_one_move_up():
    # pool of 4 pages: a holds 3, b (3 pages) waits at the head, c (1 page) behind it
    engine, s = make(FakeEngine(kv_tokens=64, max_requests=4), token_budget=64)
    a = s.submit(Request([1] * 30, max_tokens=10, ignore_eos=True))
    b = s.submit(Request([2] * 30, max_tokens=10, ignore_eos=True))
    c = s.submit(Request([3], max_tokens=2, ignore_eos=True))
    s.step()
    assert list(s.waiting) == [b, c]
    assert s.cancel(b) and not s.cancel("nobody")
    events = s.step()
    assert b.finish_reason == "cancelled" and b.error is None and len(ended(events, b)) == 1 and not b.output
    assert c in s.live(), "c fits beside a once b is gone"
    assert not s.cancel(b), "it has ended already"
    drain(s)
    assert a.finish_reason == c.finish_reason == "length" and c.output == [4, 5]
    assert engine.cache.used_tokens == 0 and not engine.cache.slot_of
    engine.cache.check()


def test_cancel_between_portions_gives_pages_and_promise_back():
    engine, s = make(FakeEngine(kv_tokens=128, max_context=128), token_budget=16)
    a = s.submit(Request([1] * 50, max_tokens=10, ignore_eos=True))
    s.step(); s.step()
    assert a.fed == 32 and engine.cache.used_tokens == 32
    pool = engine.cache.groups[0].pool
    assert pool.unpromised_pages < pool.n_pages - 2
    s.cancel(a.id)
    events = s.step()
    assert a.finish_reason == "cancelled" and len(ended(events, a)) == 1
    assert engine.cache.used_tokens == 0 and pool.unpromised_pages == pool.n_pages and not engine.cache.slot_of
    assert s.idle and len(engine.calls) == 2, "no step ran for it after the cancellation"
    engine.cache.check()


@pytest.mark.parametrize("ahead", [False, True])
def test_cancel_while_decoding(ahead):
    """With a step launched ahead that still holds the request, that step's row for it is dropped; the other
    request's tokens are what they would have been."""
    engine, s = make_ahead(FakeEngine(kv_tokens=512), run_ahead=ahead)
    a = s.submit(Request([1], max_tokens=40, ignore_eos=True))
    b = s.submit(Request([50], max_tokens=12, ignore_eos=True))
    for _ in range(5):
        s.step()
    assert (s._in_flight is not None) == ahead
    had = len(a.output)
    s.cancel(a)
    events = s.step()
    assert a.finish_reason == "cancelled" and len(a.output) == had and len(ended(events, a)) == 1
    assert a.id not in engine.cache.slot_of
    rest = events + drain(s)
    assert b.output == list(range(51, 63)) and b.finish_reason == "length"
    assert not [e for e in rest if e.request is a and e.token is not None]
    assert engine.cache.used_tokens == 0 and not engine.cache.slot_of
    engine.cache.check()


def test_cancel_of_the_only_request_with_a_step_in_flight():
    engine, s = make_ahead(FakeEngine(kv_tokens=512))
    a = s.submit(Request([1], max_tokens=40, ignore_eos=True))
    for _ in range(4):
        s.step()
    assert s._in_flight is not None
    s.cancel(a)
    events = s.step()
    assert [e.token for e in events] == [None] and a.finish_reason == "cancelled"
    assert s.idle and s._in_flight is None and engine.cache.used_tokens == 0
    b = s.submit(Request([7], max_tokens=2, ignore_eos=True))        # the scheduler goes on as before
    drain(s)
    assert b.output == [8, 9]


def test_queue_timeout_fails_a_request_that_waits_too_long():
    clock = Clock()
    engine, s = make(FakeEngine(kv_tokens=64, max_requests=4), token_budget=64, queue_timeout=5.0, clock=clock)
    a = s.submit(Request([1] * 30, max_tokens=30, ignore_eos=True))
    b = s.submit(Request([2] * 30, max_tokens=10, ignore_eos=True))      # cannot be promised pages beside a
    clock.now = 1.0
    c = s.submit(Request([3] * 30, max_tokens=10, ignore_eos=True))
    s.step()
    assert list(s.waiting) == [b, c]
    clock.now = 5.5
    events = s.step()
    assert b.finish_reason == "error" and b.error == "KV admission timeout" and len(ended(events, b)) == 1
    assert list(s.waiting) == [c], "c came later and has waited 4.5 s"
    clock.now = 6.5
    s.step()
    assert c.finish_reason == "error" and c.error == "KV admission timeout"
    drain(s)
    assert a.finish_reason == "length" and len(a.output) == 30
    assert engine.cache.used_tokens == 0 and not engine.cache.slot_of
    engine.cache.check()
    # an admitted request is never timed out, however long it runs
    d = s.submit(Request([4] * 10, max_tokens=20, ignore_eos=True))
    s.step()
    clock.now = 100.0
    drain(s)
    assert d.finish_reason == "length"
    with pytest.raises(ValueError):
        Scheduler(FakeEngine(), queue_timeout=0)


def test_max_context_below_the_models_positions():
    engine, s = make(FakeEngine(kv_tokens=256, max_context=128), max_context=40)
    with pytest.raises(ValueError, match="exceeds"):
        s.submit(Request([1] * 30, max_tokens=11))
    r = s.submit(Request([1] * 30, max_tokens=10, ignore_eos=True))
    drain(s)
    assert len(r.output) == 10
    engine, s = make(FakeEngine(kv_tokens=256, max_context=128), max_context=40, length_policy="clamp")
    r = s.submit(Request([1] * 30, max_tokens=100, ignore_eos=True))
    drain(s)
    assert len(r.output) == 10 and r.finish_reason == "length"
    with pytest.raises(ValueError):
        Scheduler(FakeEngine(max_context=128), max_context=129)


@pytest.mark.parametrize("seed", range(6))
def test_random_cancellations_lose_nothing(seed):
    """Random arrivals, ends and cancellations at any stage, with and without running ahead: every request ends exactly
    once, a cancelled one gets no token after its cancellation took effect, and nothing is lost from the cache."""
    import random
    for ahead in (False, True):
        rng = random.Random(seed)
        engine, s = make_ahead(FakeEngine(kv_tokens=160, max_requests=3, max_context=64), token_budget=24, run_ahead=ahead)
        requests, terminal, step = [], {}, 0
        arrivals = sorted(rng.randrange(0, 40) for _ in range(12))
        while arrivals or not s.idle:
            while arrivals and arrivals[0] <= step:
                arrivals.pop(0)
                prompt = [rng.randrange(0, 100) for _ in range(rng.randrange(1, 40))]
                requests.append(s.submit(Request(prompt, max_tokens=rng.randrange(1, 20), ignore_eos=rng.random() < 0.5)))
            if requests and rng.random() < 0.2:
                s.cancel(rng.choice(requests))
            for e in s.step():
                if e.finished:
                    assert e.request.id not in terminal
                    terminal[e.request.id] = e
                else:
                    assert e.request.id not in terminal, "a token after the terminal event"
            engine.cache.check()
            step += 1
            assert step < 2000
        assert set(terminal) == {r.id for r in requests}
        assert any(r.finish_reason == "cancelled" for r in requests)
        assert engine.cache.used_tokens == 0 and not engine.cache.slot_of
        assert engine.cache.groups[0].pool.unpromised_pages == engine.cache.groups[0].pool.n_pages
