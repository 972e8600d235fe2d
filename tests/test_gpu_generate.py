"""Generation through the Python entry point and the command line, sampling against the plain rule,
and decode steps replayed from CUDA graphs against eager steps."""
import json
import random
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from conftest import TINY_A, TINY_B
from model_tools import make_model, random_requests
from plain_gpt2 import PlainGpt2, adjust_logits, sample_token

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("gen")
    return {"A": make_model(root / "A", TINY_A, 0, "float32"), "B": make_model(root / "B", TINY_B, 1, "float32")}


def test_greedy_generation_matches_plain(folders):
    """Config A's workload: prompts of 5, 17 and 33 tokens, 16 greedy tokens each, page size 16."""
    from damendaemon_b200.runtime import Runtime, generate
    plain = PlainGpt2(folders["A"])
    prompts = list(random_requests(TINY_A, [5, 17, 33], 7).values())
    want = [plain.greedy(p, 16) for p in prompts]
    for dtype in ("float32", "bfloat16"):
        runtime = Runtime(folders["A"], dtype=dtype, max_batch=4, page_size=16)
        got = runtime.generate_batch(prompts, 16, ignore_eos=True)
        if dtype == "float32":
            assert got == want
        else:   # rounding may flip a near-tie; then the plain logits at the flip must be a near-tie
            for p, g, w in zip(prompts, got, want):
                if g != w:
                    i = next(i for i in range(16) if g[i] != w[i])
                    row = plain.logits(p + w[:i])[-1]
                    assert abs(float(row[g[i]] - row[w[i]])) < 4e-2
        assert runtime.engine.cache.used_tokens == 0
    assert generate(folders["A"], prompts[:1], 4, dtype="float32") == [want[0][:4]]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_a_step_ahead_changes_no_token(folders, dtype):
    """The scheduler launches the next decode step before it has read this step's tokens (the engine takes the ids
    from the sampler's output on the device). Same tokens as when every step's tokens are read first: greedy and
    seeded sampling with penalties, requests of different lengths, and an end-of-sequence token that ends one
    request while a step with it is in flight."""
    import dataclasses
    from damendaemon_b200.runtime import Runtime
    prompts = list(random_requests(TINY_B, [3, 9, 21, 40], 3).values())
    lengths = [25, 12, 30, 18]
    results = {}
    for ahead in (False, True):
        runtime = Runtime(folders["B"], dtype=dtype, max_batch=4, page_size=8, run_ahead=ahead)
        greedy = runtime.generate_batch(prompts, lengths, ignore_eos=True)
        assert (runtime.last_scheduler.steps_ahead > 0) == ahead
        sampled = runtime.generate_batch(prompts, lengths, ignore_eos=True, temperature=0.9, top_k=40, top_p=0.95,
                                         seed=11, repetition_penalty=1.2, presence_penalty=0.3)
        # a token that the third request emits in the middle of its greedy run ends it there, as end of sequence
        stop = greedy[2][10]
        runtime.engine.spec = dataclasses.replace(runtime.engine.spec, eos_token_ids=(stop,))
        stopped = runtime.generate_batch(prompts, lengths)
        assert runtime.engine.cache.used_tokens == 0
        results[ahead] = (greedy, sampled, stopped)
        first = greedy[2].index(stop)
        assert stopped[2] == greedy[2][:first + 1]
    assert results[True][:2] == results[False][:2]
    # with an unforeseen end the request stays in the batch for one step more than without running ahead; the
    # others' logits in that step are the same only up to rounding (other split counts), so hold 32-bit to equality
    if dtype == "float32":
        assert results[True][2] == results[False][2]


def test_streaming_generate_events(folders):
    from damendaemon_b200.runtime import Runtime
    plain = PlainGpt2(folders["A"])
    runtime = Runtime(folders["A"], dtype="float32", max_batch=1)
    events = list(runtime.generate([3, 1, 4, 1, 5], max_tokens=6, ignore_eos=True))
    assert [e["token"] for e in events[:-1]] == plain.greedy([3, 1, 4, 1, 5], 6)
    last = events[-1]
    assert last["finish_reason"] == "length" and last["usage"] == {"prompt_tokens": 5, "completion_tokens": 6, "total_tokens": 11}
    assert last["timing"]["first_token_seconds"] > 0
    with pytest.raises(ValueError, match="exceeds"):
        list(runtime.generate([1] * 120, max_tokens=20))
    with pytest.raises(ValueError, match="tokenizer"):
        list(runtime.generate("some text", max_tokens=2))


def test_temperature_workload_matches_plain_rule(folders):
    """Config B's workload: prompts 1, 9, 64, 200; portions of 32 beside decodes; temperature 0.8, seed 7;
    up to 40 new tokens capped at the positions; page size 8. Teacher-forced on the engine's own tokens."""
    from damendaemon_b200.runtime import Runtime
    plain = PlainGpt2(folders["B"])
    prompts = list(random_requests(TINY_B, [1, 9, 64, 200], 9).values())
    runtime = Runtime(folders["B"], dtype="float32", max_batch=4, page_size=8, prefill_chunk_size=32, token_budget=48)
    got = runtime.generate_batch(prompts, 40, ignore_eos=True, temperature=0.8, seed=7, length_policy="clamp")
    assert [len(g) for g in got] == [40, 40, 40, 40]
    assert any(p > 0 and d > 0 for p, d in runtime.last_scheduler.step_log), "no step mixed a portion with decodes"
    for i, (p, g) in enumerate(zip(prompts, got)):
        stream = random.Random(7 + i)
        logits = plain.logits(p + g)
        for j, token in enumerate(g):
            want = sample_token(logits[len(p) - 1 + j], 0.8, stream.random())
            assert token == want, f"request {i} token {j}"
    # capped at the model's positions
    long = runtime.generate_batch([list(range(250))], 40, ignore_eos=True, length_policy="clamp")
    assert len(long[0]) == 6


def test_sampling_filters_and_penalties():
    from damendaemon_b200.sampling import Sampler, Sampling, sample_rows
    g = torch.Generator().manual_seed(3)
    V = 777
    logits = torch.randn(24, V, generator=g) * 2.5
    options = []
    for r in range(24):
        options.append(Sampling(temperature=[0.7, 1.0, 1.3][r % 3], top_k=[0, 5, 40, 0][r % 4], top_p=[1.0, 0.9, 0.5][r % 3],
                                seed=r))
    samplers = [Sampler(o) for o in options]
    got = sample_rows(logits.cuda(), samplers)
    for r, o in enumerate(options):
        u = random.Random(r).random()
        assert got[r] == sample_token(logits[r], o.temperature, u, o.top_k, o.top_p), f"row {r}: {o}"
    # penalties and bias change the logits before the choice
    o = Sampling(repetition_penalty=1.7, frequency_penalty=0.4, presence_penalty=0.3, logit_bias={"5": 3.0, 9: -100})
    s = Sampler(o)
    prompt, generated = [1, 2, 3, 9], [2, 2, 7]
    s.prepare(prompt, V)
    for t in generated:
        s.observe(t)
    row = logits[0].clone()
    row[[1, 2, 7, 5, 9]] = torch.tensor([4.0, 4.1, 3.9, 2.0, 9.0])
    want = int(adjust_logits(row, prompt, generated, 1.7, 0.4, 0.3, {5: 3.0, 9: -100}).argmax())
    assert sample_rows(row[None].cuda(), [s]) == [want]
    from damendaemon_b200.sampling import NonFiniteLogits
    bad = logits[:1].clone(); bad[0, 3] = float("nan")
    with pytest.raises(NonFiniteLogits):
        sample_rows(bad.cuda(), [Sampler(Sampling())])
    for kw in ({"temperature": -1}, {"top_p": 0}, {"top_k": -1}, {"seed": -1}, {"repetition_penalty": 0},
               {"presence_penalty": 3}, {"logit_bias": {"x": 1}}, {"temperature": float("nan")}):
        with pytest.raises(ValueError):
            Sampling(**kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_replay_equals_eager(folders, dtype):
    from damendaemon_b200.engine import Engine, StepEntry
    prompts = random_requests(TINY_B, [9, 40, 3], 5)
    outs = []
    for use_graph in (False, True):
        engine = Engine(folders["B"], dtype=dtype, kv_tokens=512, page_size=8, max_requests=4, use_graph=use_graph)
        engine.step([StepEntry(r, t, []) for r, t in prompts.items()])
        rows = []
        for i in range(12):
            live = list(prompts)[: 3 if i < 8 else 2]       # the batch shrinks: another graph
            rows.append(engine.step([StepEntry(r, [(i * 7 + k) % 1000], [0]) for k, r in enumerate(live)]).clone())
        outs.append(rows)
        if use_graph:
            assert len(engine._graphs) == 2
    for a, b in zip(*outs):
        assert (a - b).abs().max() < (2e-6 if dtype == "float32" else 3e-2)


def test_command_line(folders, tmp_path):
    out = subprocess.run([sys.executable, "-m", "damendaemon_b200", "run", str(folders["A"]), "--prompt-ids", "3,1,4,1,5",
                          "--max-tokens", "5", "--dtype", "float32", "--ignore-eos", "--context", "128"],
                         capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert [int(t) for t in out.stdout.split()] == PlainGpt2(folders["A"]).greedy([3, 1, 4, 1, 5], 5)
    final = json.loads(out.stderr.strip().splitlines()[-1])
    assert final["finish_reason"] == "length" and final["usage"]["completion_tokens"] == 5
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(TINY_A))
    made = subprocess.run([sys.executable, "-m", "damendaemon_b200", "init-random", str(cfg), str(tmp_path / "m"), "--seed", "4"],
                          capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert made.returncode == 0 and (tmp_path / "m" / "model.safetensors").is_file()


@pytest.mark.parametrize("ahead", [False, True])
def test_a_kernel_error_bit_fails_the_requests_of_its_step_and_generation_goes_on(folders, ahead):
    """The generation path does not synchronise to read the kernels' error word: the word comes with the sampled ids.
    A bit that stands in it when a step's tokens are read (here put there by hand, as a kernel that met a missing page
    would) fails that step's requests with a message that names it, gives their pages back and clears the word; the
    next requests generate what they should. The same with a step launched ahead."""
    from damendaemon_b200 import kernels
    from damendaemon_b200.engine.scheduler import Request, Scheduler
    from damendaemon_b200.runtime import Runtime
    plain = PlainGpt2(folders["A"])
    runtime = Runtime(folders["A"], dtype="float32", max_batch=4, page_size=16, run_ahead=ahead)
    scheduler = Scheduler(runtime.engine, run_ahead=ahead)
    a = scheduler.submit(Request([5, 17, 3], max_tokens=20, ignore_eos=True))
    b = scheduler.submit(Request([9, 8], max_tokens=20, ignore_eos=True))
    for _ in range(4):
        scheduler.step()
    assert len(a.output) >= 3 and not a.finished
    kernels.error_flag(runtime.engine.device).fill_(4)           # "a page was missing on a read"
    events = []
    while not (a.finished and b.finished):
        events += scheduler.step()
    assert a.finish_reason == b.finish_reason == "error" and "0x4" in a.error and "DeviceStepError" in a.error
    assert sum(1 for e in events if e.token is None and e.finished) == 2
    assert runtime.engine.cache.used_tokens == 0 and not runtime.engine.live_requests()
    assert kernels.read_error_flag(runtime.engine.device) == 0      # the word was cleared
    assert runtime.generate_batch([[5, 17, 3]], 6, ignore_eos=True) == [plain.greedy([5, 17, 3], 6)]


def test_stop_strings_and_text_deltas(folders, tmp_path):
    """With a tokenizer in the folder ``generate`` hands out text: a stop string that completes in the middle of the
    generation ends it there ('stop'), nothing of the stop string or after it is shown, the request's pages go back,
    and the pieces of text add up to what was decoded before the stop."""
    import shutil
    from damendaemon_b200.runtime import Runtime
    folder = tmp_path / "with_tokenizer"
    shutil.copytree(folders["A"], folder)
    vocab = {f"w{i}": i for i in range(TINY_A["vocab_size"])}
    (folder / "tokenizer.json").write_text(json.dumps({
        "version": "1.0", "truncation": None, "padding": None, "added_tokens": [], "normalizer": None,
        "pre_tokenizer": {"type": "Whitespace"}, "post_processor": None, "decoder": None,
        "model": {"type": "WordLevel", "vocab": vocab, "unk_token": "w0"}}))
    runtime = Runtime(folder, dtype="float32", max_batch=2, page_size=16)
    assert runtime.tokenizer is not None
    prompt = "w5 w17 w3 w200"
    free = list(runtime.generate(prompt, 10, ignore_eos=True))
    tokens = [e["token"] for e in free[:-1]]
    assert tokens == PlainGpt2(folders["A"]).greedy([5, 17, 3, 200], 10) and free[-1]["finish_reason"] == "length"
    assert "".join(e["text"] for e in free[:-1]) == " ".join(f"w{t}" for t in tokens)
    k = next(i for i in range(2, 9) if tokens[i] not in tokens[:i])      # a word that has not come before
    stop = f"w{tokens[k]} "                                  # complete once the next token's word follows it
    events = list(runtime.generate(prompt, 10, ignore_eos=True, stop=[stop, "never"]))
    final = events[-1]
    shown = "".join(e["text"] for e in events[:-1])
    assert final["finish_reason"] == "stop" and final["usage"]["completion_tokens"] == k + 2
    assert [e["token"] for e in events[:-1]] == tokens[:k + 2]
    assert shown == "".join(f"w{t} " for t in tokens[:k]) and stop not in shown
    assert runtime.engine.cache.used_tokens == 0 and not runtime.engine.live_requests()
    with pytest.raises(ValueError, match="stop"):
        list(runtime.generate(prompt, 4, stop=[""]))
    with pytest.raises(ValueError, match="tokenizer"):
        list(Runtime(folders["A"], dtype="float32", max_batch=1).generate([5, 17], 4, stop="x"))


@pytest.mark.parametrize("seed", [0, 1])
@pytest.mark.parametrize("ahead", [False, True])
def test_random_arrivals_and_cancellations_generate_what_plain_does(folders, seed, ahead):
    """Requests arrive between steps, a pool of few pages makes some wait, some are withdrawn at random moments (while
    waiting, between portions of their prompt, while decoding, with a step launched ahead): every request that runs to
    its end has the plain implementation's greedy tokens, every withdrawn one a beginning of them, and nothing is left
    in the cache. float32, so that the tokens are the plain ones exactly."""
    from damendaemon_b200.engine.scheduler import Request, Scheduler
    from damendaemon_b200.runtime import Runtime
    plain = PlainGpt2(folders["A"])
    rng = random.Random(seed)
    runtime = Runtime(folders["A"], dtype="float32", max_batch=3, page_size=16, kv_cache_tokens=160, run_ahead=ahead)
    scheduler = Scheduler(runtime.engine, token_budget=24, chunk_size=16, run_ahead=ahead)
    arrivals = sorted(rng.randrange(0, 30) for _ in range(10))
    requests, cancelled, step = [], set(), 0
    while arrivals or not scheduler.idle:
        while arrivals and arrivals[0] <= step:
            arrivals.pop(0)
            prompt = [rng.randrange(0, TINY_A["vocab_size"]) for _ in range(rng.randrange(1, 40))]
            requests.append(scheduler.submit(Request(prompt, max_tokens=rng.randrange(1, 14), ignore_eos=True)))
        if requests and rng.random() < 0.15:
            victim = rng.choice(requests)
            if scheduler.cancel(victim):
                cancelled.add(victim.id)
        scheduler.step()
        runtime.engine.cache.check()
        step += 1
        assert step < 1000
    assert cancelled, "no request was withdrawn: the test shows nothing about cancellation"
    for r in requests:
        want = plain.greedy(r.prompt, r.max_tokens)
        if r.id in cancelled and r.finish_reason == "cancelled":
            assert r.output == want[:len(r.output)] and len(r.output) < len(want)
        else:
            assert r.finish_reason == "length" and r.output == want, (r.id, r.finish_reason)
    assert runtime.engine.cache.used_tokens == 0 and not runtime.engine.live_requests()
    assert runtime.engine.cache.groups[0].pool.unpromised_pages == runtime.engine.cache.groups[0].pool.n_pages
