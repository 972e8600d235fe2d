"""The engine against the plain implementation, in 32-bit and in bfloat16, under every way of
cutting the work: whole, last 32 tokens one by one, portions of changing size, and mixed with
so few pages that they are used again."""
import pytest
import torch

from conftest import TINY_A, TINY_B, TINY_C, TINY_D, TINY_E, TINY_F
from model_tools import make_model, random_requests
from plain_gpt2 import PlainGpt2
from trace_tools import mixed_steps, portion_steps, run_trace, tail_steps, whole_steps

pytestmark = pytest.mark.gpu

# name: (config, seed, request lengths, factor on the QKV projection that makes attention peaky)
CASES = {"A": (TINY_A, 0, [5, 17, 33, 100, 128, 64], 8.0), "B": (TINY_B, 1, [1, 9, 64, 200, 256, 77], 8.0),
         "C": (TINY_C, 2, [1, 70, 320, 129, 64, 200], 3.0), "D": (TINY_D, 3, [3, 40, 96, 17, 65], 8.0),
         "E": (TINY_E, 4, [2, 130, 192, 65, 31], 2.0), "F": (TINY_F, 5, [1, 80, 33, 17, 64, 80, 48, 70], 1.0)}
# float32: the engine's contract. bfloat16: three times what rounding the stored activations to
# bfloat16 does to the plain implementation's own logits for that model (measured in the fixture,
# about 0.005 for these models), plus a small floor.
FLOAT32_TOL = 1e-4
TOL = {}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    out = {}
    for name, (config, seed, lengths, sharpen) in CASES.items():
        for dtype in ("float32", "bfloat16"):
            folder = make_model(root / f"{name}-{dtype}", config, seed, dtype, sharpen)
            requests = random_requests(config, lengths, 100 + seed)
            plain = PlainGpt2(folder)
            want = {r: plain.logits(t).float() for r, t in requests.items()}
            out[name, dtype] = (folder, config, requests, want)
            if dtype == "bfloat16":
                moved = max((plain.logits(t, rounded=torch.bfloat16).float() - want[r]).abs().max().item()
                            for r, t in requests.items())
                TOL[name, dtype] = 3.0 * moved + 2e-3
            else:
                TOL[name, dtype] = FLOAT32_TOL
    return out


def engine_for(folder, dtype, kv_tokens, page_size, poison=True):
    from damendaemon_b200.engine import Engine
    engine = Engine(folder, dtype=dtype, kv_tokens=kv_tokens, page_size=page_size, max_requests=8)
    if poison:
        for g in engine.cache.groups:
            g.arena.fill_(float("nan"))      # whatever was never written must never be read
    return engine


def replay(engine, builder):
    from damendaemon_b200.engine import StepEntry
    got = {}
    for s in builder.steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]
        if entries:
            logits = engine.step(entries).cpu()
            for (request, position), row in zip(builder.where[s["step"]], logits):
                got.setdefault(request, {})[position] = row
        for r in s["end"]:
            engine.finish(r)
        engine.cache.check()
    return got


def compare(got, want, tol, what):
    worst = 0.0
    for r, rows in got.items():
        for p, row in rows.items():
            assert torch.isfinite(row).all(), f"{what}: non-finite logits at request {r} position {p}"
            err = (row - want[r][p]).abs().max().item()
            worst = max(worst, err)
            assert err < tol, f"{what}: request {r} position {p} differs by {err:.3e} (first wrong place)"
    for r in want:
        assert set(got[r]) == set(range(len(want[r]))), f"{what}: request {r} misses positions"
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_cuttings(models, name, dtype, mode):
    folder, config, requests, want = models[name, dtype]
    page = {"A": 16, "B": 8, "C": 16, "D": 32, "E": 64, "F": 16}[name]
    if mode == "mixed":
        builder, peak = mixed_steps(requests, seed=3)
        kv = peak
    else:
        builder = {"whole": whole_steps, "tail": tail_steps, "portions": portion_steps}[mode](requests)
        kv = 64 * ((config["n_positions"] + 63) // 64)
    engine = engine_for(folder, dtype, kv, page)
    got = replay(engine, builder)
    compare(got, want, TOL[name, dtype], f"{name} {dtype} {mode}")
    assert engine.cache.used_tokens == 0 and not engine.live_requests()
    if mode == "mixed":
        handed_out = sum((len(t) + page - 1) // page for t in requests.values())
        assert engine.cache.groups[0].pool.n_pages < handed_out, "the pool is too large for pages to be used again"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_float32_cuttings_agree_to_rounding(models, dtype):
    """The same position under different cuttings: equal beyond rounding, far inside the tolerance to plain."""
    folder, config, requests, want = models["A", dtype]
    a = replay(engine_for(folder, dtype, 512, 16), whole_steps(requests))
    b = replay(engine_for(folder, dtype, 512, 16), portion_steps(requests))
    worst = max((a[r][p] - b[r][p]).abs().max().item() for r in a for p in a[r])
    assert worst < (2e-6 if dtype == "float32" else 3e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(models, dtype):
    """One token at a time from the very first token up to the model's last position."""
    from damendaemon_b200.engine import StepEntry, StepError
    folder, config, requests, want = models["B", dtype]
    tokens = requests["r4"]                 # 256 tokens = n_positions
    engine = engine_for(folder, dtype, 256, 8)
    for p, t in enumerate(tokens):
        row = engine.step([StepEntry("x", [t], [0])]).cpu()[0]
        err = (row - want["r4"][p]).abs().max().item()
        assert err < TOL["B", dtype], f"position {p}: {err:.3e}"
    # the learned positions end here: one more token must be refused and change nothing
    before = engine.length("x")
    with pytest.raises(StepError, match="positions"):
        engine.step([StepEntry("x", [1], [0])])
    assert engine.length("x") == before == 256
    engine.finish("x")
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_single_tokens_anywhere_among_portions(models, name, dtype):
    """A step that names portions and single tokens in any order: inside, the engine lays the single tokens out first
    (a decode kernel takes them, a prompt kernel the portions); the logits come back in the order of the entries as
    given and of their wanted places. Twice, so that the second step reads what the first one cached."""
    from damendaemon_b200.engine import StepEntry
    folder, config, requests, want = models[name, dtype]
    names = [r for r in requests if len(requests[r]) >= 17][:4]
    engine = engine_for(folder, dtype, 64 * 16, 16)
    held = {r: 0 for r in names}
    plans = [[(names[0], 9, [0, 8]), (names[1], 1, [0]), (names[2], 5, []), (names[3], 1, [0])],
             [(names[3], 1, [0]), (names[0], 3, [2]), (names[1], 1, []), (names[2], 7, [6, 0, 3])]]
    for plan in plans:
        entries, places = [], []
        for r, n, wanted in plan:
            entries.append(StepEntry(r, requests[r][held[r]:held[r] + n], wanted))
            places += [(r, held[r] + w) for w in wanted]
            held[r] += n
        if plan is plans[1]:
            # the ids come from the device this time (in the order given, so nothing is moved inside): the entries
            # only carry the counts
            ids = torch.tensor([t for e in entries for t in e.tokens], dtype=torch.int32, device=engine.device)
            entries = [StepEntry(e.request, [0] * len(e.tokens), e.want) for e in entries]
            rows = engine.step(entries, device_ids=ids).cpu()
        else:
            rows = engine.step(entries).cpu()
        assert rows.shape[0] == len(places)
        for (r, position), row in zip(places, rows):
            err = (row - want[r][position]).abs().max().item()
            assert err < TOL[name, dtype], f"request {r} position {position}: {err:.3e}"
    for r in names:
        engine.finish(r)
    engine.cache.check()


def test_step_validation_changes_nothing(models):
    from damendaemon_b200.cache import PageCapacityError
    from damendaemon_b200.engine import StepEntry, StepError
    folder, config, requests, want = models["A", "float32"]
    engine = engine_for(folder, "float32", 64, 16)
    engine.step([StepEntry("a", [1, 2, 3])])
    for bad in ([StepEntry("a", [1]), StepEntry("a", [2])], [StepEntry("b", [])], [StepEntry("b", [512])],
                [StepEntry("b", [-1])], [StepEntry("b", [1, 2], [2])], [StepEntry("b", [1] * 129)], [],
                [StepEntry("a", [1], [0, 0])], [StepEntry("b", [1, 2], [1, 1])]):
        with pytest.raises(StepError):
            engine.step(bad)
        assert engine.live_requests() == ["a"] and engine.length("a") == 3
    with pytest.raises(PageCapacityError):
        engine.step([StepEntry("a", [1]), StepEntry("b", [1] * 60)])     # 64 tokens of pages in all
    assert engine.live_requests() == ["a"] and engine.length("a") == 3
    engine.cache.check()
    none = engine.step([StepEntry("a", [4, 5])])
    assert tuple(none.shape) == (0, 512)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_token_ids_from_the_device(models, dtype):
    """A decode step whose token ids come from a device tensor (the sampler's output of the step before) gives the
    logits of the same step fed from the host, bit for bit, eagerly and replayed from a graph; a tensor of the wrong
    type or size is refused with nothing changed."""
    from damendaemon_b200.engine import StepEntry, StepError
    folder, config, requests, want = models["B", dtype]
    prompts = {r: t[:9] for r, t in list(requests.items())[2:5]}
    feed = [[(7 * s + 3 * i + 1) % config["vocab_size"] for i in range(len(prompts))] for s in range(5)]
    host, device = engine_for(folder, dtype, 256, 8), engine_for(folder, dtype, 256, 8)
    for engine in (host, device):
        engine.step([StepEntry(r, t) for r, t in prompts.items()])
    for ids in feed:
        a = host.step([StepEntry(r, [ids[i]], [0]) for i, r in enumerate(prompts)]).clone()
        on_device = torch.tensor(ids, dtype=torch.int32, device="cuda:0")
        b = device.step([StepEntry(r, [0], [0]) for r in prompts], device_ids=on_device).clone()
        assert torch.equal(a, b)
    fresh = engine_for(folder, dtype, 256, 8)           # a first step with a bad tensor: refused in the same way
    with pytest.raises(StepError):
        fresh.step([StepEntry("x", [1], [0])], device_ids=torch.tensor([1], dtype=torch.int32))
    assert not fresh.live_requests()
    for bad in (torch.tensor(feed[0], dtype=torch.int64, device="cuda:0"), torch.zeros(2, dtype=torch.int32, device="cuda:0"),
                torch.tensor(feed[0], dtype=torch.int32), feed[0]):
        with pytest.raises(StepError):
            device.step([StepEntry(r, [0], [0]) for r in prompts], device_ids=bad)
        assert all(device.length(r) == host.length(r) for r in prompts)
    device.cache.check()
    assert device.raise_device_errors() is None


def test_cache_that_does_not_fit_is_refused(models, monkeypatch):
    """The cache, a step's activations and the headroom are held against the free memory before the cache is
    allocated: a pool that cannot fit raises MemoryError and names what was asked for."""
    from damendaemon_b200.engine import Engine
    folder, config, requests, want = models["A", "float32"]
    free_before = torch.cuda.mem_get_info(0)[0]
    monkeypatch.setattr(Engine, "HEADROOM_BYTES", 1 << 50)
    with pytest.raises(MemoryError, match="kv_tokens"):
        Engine(folder, dtype="float32", kv_tokens=64, page_size=16, max_requests=4, device="cuda:0")
    monkeypatch.undo()
    torch.cuda.empty_cache()
    assert torch.cuda.mem_get_info(0)[0] >= free_before - (64 << 20)
    engine = Engine(folder, dtype="float32", kv_tokens=64, page_size=16, max_requests=4, device="cuda:0")
    assert engine.cache.bytes_needed(4) == 64 * 2 * 2 * 64 * 4          # tokens x layers x (K, V) x width x 4 bytes


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(models, dtype, tmp_path):
    """The replay program itself, as a user runs it: mixed trace, few pages."""
    folder, config, requests, want = models["A", dtype]
    builder, peak = mixed_steps(requests, seed=11)
    outputs = run_trace(folder, dtype, builder.steps, tmp_path / "out", max_tokens=peak, page_size=16)
    got = {r: {p: torch.from_numpy(row.copy()) for p, row in rows.items()} for r, rows in builder.collect(outputs).items()}
    compare(got, want, TOL["A", dtype], f"trace_run {dtype}")


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("C", "bfloat16"), ("E", "bfloat16"), ("B", "bfloat16")])
def test_random_traces_with_graphs_on(models, name, dtype, seed):
    """Random mixed traces (other seeds, other numbers of live requests, other portion sizes than the fixed ones above)
    through an engine that captures every step shape when it comes back and replays it from then on, with a pool so
    small that pages are used again: every position against the plain implementation."""
    from damendaemon_b200.engine import Engine
    folder, config, requests, want = models[name, dtype]
    page = {"A": 16, "B": 8, "C": 16, "E": 64}[name]
    portions = [(2, 3, 5, 8, 13, 17, 32), (1, 2, 64), (16, 128, 130), (4, 4, 4, 31)][seed % 4]
    builder, peak = mixed_steps(requests, seed=100 + seed, max_live=2 + seed % 3, prompt_share=0.3 + 0.1 * (seed % 5), portions=portions)
    engine = Engine(folder, dtype=dtype, kv_tokens=peak, page_size=page, max_requests=8, use_graph=True)
    engine.capture_after = {True: 1, False: 1}
    for g in engine.cache.groups:
        g.arena.fill_(float("nan"))
    got = replay(engine, builder)
    compare(got, want, TOL[name, dtype], f"{name} {dtype} random trace {seed}")
    assert engine.cache.used_tokens == 0 and not engine.live_requests()
    assert engine.raise_device_errors() is None
