"""Two layers of the benchmark's own layer sizes (GPT-2 XL: width 1600, 25 heads of 64, inner 6400,
vocabulary 50257, 1024 positions) against the plain implementation, in 32-bit and in bfloat16:
a prompt portion of several hundred tokens, a second portion, then single decoded tokens."""
import pytest
import torch

from model_tools import make_model
from plain_gpt2 import PlainGpt2

pytestmark = pytest.mark.gpu

XL2 = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_layer": 2, "n_embd": 1600, "n_head": 25,
       "n_inner": 6400, "vocab_size": 50257, "n_positions": 1024, "layer_norm_epsilon": 1e-5,
       "activation_function": "gelu_new"}


@pytest.fixture(scope="module")
def xl(tmp_path_factory):
    folder = make_model(tmp_path_factory.mktemp("xl") / "xl2", XL2, seed=5, dtype="bfloat16", sharpen=2.0)
    g = torch.Generator().manual_seed(6)
    tokens = torch.randint(0, 50257, (331,), generator=g).tolist()
    rows = [0, 1, 63, 64, 200, 299, 300] + list(range(321, 331))
    plain = PlainGpt2(folder)
    want = plain.logits(tokens, rows=rows).float()
    moved = (plain.logits(tokens, rounded=torch.bfloat16, rows=rows).float() - want).abs().max().item()
    return folder, tokens, rows, want, moved


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_xl_layer_sizes(xl, dtype):
    from damendaemon_b200.engine import Engine, StepEntry
    folder, tokens, rows, want, moved = xl
    engine = Engine(folder, dtype=dtype, kv_tokens=384, page_size=16, max_requests=2, use_graph=True)
    for g in engine.cache.groups:
        g.arena.fill_(float("nan"))
    got = {}
    first = engine.step([StepEntry("r", tokens[:300], [r for r in rows if r < 300])])
    for r, row in zip([r for r in rows if r < 300], first.cpu()):
        got[r] = row
    second = engine.step([StepEntry("r", tokens[300:321], [0])])
    got[300] = second.cpu()[0]
    for p in range(321, 331):
        got[p] = engine.step([StepEntry("r", [tokens[p]], [0])]).cpu()[0].clone()
    tol = 1e-4 if dtype == "float32" else 3.0 * moved + 2e-3
    for i, r in enumerate(rows):
        err = (got[r] - want[i]).abs().max().item()
        assert err < tol, f"{dtype}: position {r} differs by {err:.3e} (allowed {tol:.3e})"
        if dtype == "float32":
            assert int(got[r].argmax()) == int(want[i].argmax())
    engine.finish("r")
    assert engine.cache.used_tokens == 0


def test_xl_portions_on_key_block_boundaries(xl):
    """Portions that start at positions 0 and 128: there the prompt attention kernel writes the cache itself (no
    separate cache-write kernel). A third portion starts inside a key block and reads what the first two left; the
    decoded tokens read all of it. The cache starts out poisoned."""
    from damendaemon_b200.engine import Engine, StepEntry
    folder, tokens, rows, want, moved = xl
    engine = Engine(folder, dtype="bfloat16", kv_tokens=384, page_size=16, max_requests=2, use_graph=True)
    for g in engine.cache.groups:
        g.arena.fill_(float("nan"))
    got = {}
    for lo, hi in [(0, 128), (128, 300), (300, 321)]:
        asked = [r for r in rows if lo <= r < hi]
        out = engine.step([StepEntry("r", tokens[lo:hi], [r - lo for r in asked])]).cpu()
        for r, row in zip(asked, out):
            got[r] = row
    for p in range(321, 331):
        got[p] = engine.step([StepEntry("r", [tokens[p]], [0])]).cpu()[0].clone()
    tol = 3.0 * moved + 2e-3
    for i, r in enumerate(rows):
        err = (got[r] - want[i]).abs().max().item()
        assert err < tol, f"position {r} differs by {err:.3e} (allowed {tol:.3e})"
    engine.finish("r")
    assert engine.cache.used_tokens == 0


@pytest.mark.parametrize("use_graph", [False, True])
def test_xl_decode_of_eight_requests(xl, use_graph):
    """Eight requests of different lengths decoded together, in bfloat16: 8 x 25 heads is where the engine switches to
    the decode attention kernel that streams whole cache pages, with and without CUDA graphs. Every decoded position of
    every request is held against the plain implementation run on that request alone."""
    from damendaemon_b200.engine import Engine, StepEntry
    folder = xl[0]
    plain = PlainGpt2(folder)
    g = torch.Generator().manual_seed(11)
    lengths, n_decode = [5, 17, 33, 64, 100, 130, 16, 250], 6
    tokens = [torch.randint(0, 50257, (n + n_decode,), generator=g).tolist() for n in lengths]
    want, moved = [], 0.0
    for n, seq in zip(lengths, tokens):
        rows = list(range(n - 1, n + n_decode))
        exact = plain.logits(seq, rows=rows).float()
        moved = max(moved, (plain.logits(seq, rounded=torch.bfloat16, rows=rows).float() - exact).abs().max().item())
        want.append(exact)
    engine = Engine(folder, dtype="bfloat16", kv_tokens=1024, page_size=16, max_requests=8, use_graph=use_graph)
    for group in engine.cache.groups:
        group.arena.fill_(float("nan"))
    tol = 3.0 * moved + 2e-3
    out = engine.step([StepEntry(r, tokens[r][:n], [n - 1]) for r, n in enumerate(lengths)]).cpu()
    for r in range(8):
        assert (out[r] - want[r][0]).abs().max().item() < tol, f"prompt of request {r}"
    for step in range(n_decode):
        out = engine.step([StepEntry(r, [tokens[r][n + step]], [0]) for r, n in enumerate(lengths)]).cpu()
        for r in range(8):
            err = (out[r] - want[r][1 + step]).abs().max().item()
            assert err < tol, f"request {r}, decoded token {step}: differs by {err:.3e} (allowed {tol:.3e})"
    for r in range(8):
        engine.finish(r)
    assert engine.cache.used_tokens == 0
