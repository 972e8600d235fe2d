"""The benchmark's own model at its full depth (GPT-2 XL: 48 layers, width 1600, 25 heads of 64, inner 6400,
vocabulary 50257, 1024 positions; seeded random weights) against the plain implementation, under every way of
cutting the work, in 32-bit (1e-4 and the same greedy token) and in bfloat16 (the tolerance derived from what
rounding does to the plain logits of this very model).

The plain implementation runs in float64 on the GPU here (its functions compute wherever their weights lie);
it is still the file of formulas under tests/, it shares nothing with the engine. Request lengths follow the
reference's stress check (scripts/verify_stress.py:196-227: prompts of 31, 255, 257 and context - 16 tokens), two
more make the pool turn over. Logits are compared at a spread of positions per request: the first tokens, both
sides of page and key-block edges, every 97th position and the last 34, in whatever step they fall.
"""
import pytest
import torch

from trace_tools import mixed_steps, portion_steps, tail_steps, whole_steps

pytestmark = pytest.mark.gpu

XL = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_layer": 48, "n_embd": 1600, "n_head": 25,
      "n_inner": 6400, "vocab_size": 50257, "n_positions": 1024, "layer_norm_epsilon": 1e-5,
      "activation_function": "gelu_new"}
LENGTHS = [31, 255, 257, 1008, 129, 64]
EDGES = (0, 1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 129, 255, 256, 511, 512, 513)
FLOAT32_TOL = 1e-4


def positions_of(n):
    return sorted({p for p in EDGES if p < n} | set(range(0, n, 97)) | set(range(max(0, n - 34), n)))


@pytest.fixture(scope="module")
def xl():
    """{dtype: (tensors on the device, requests, wanted positions, plain logits, bfloat16 tolerance)}."""
    from damendaemon_b200.registry import architecture_of
    import plain_gpt2
    arch = architecture_of(XL)
    typed = arch.parse_config(XL)
    g = torch.Generator().manual_seed(21)
    requests = {f"r{i}": torch.randint(0, XL["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate(LENGTHS)}
    wanted = {r: positions_of(len(t)) for r, t in requests.items()}
    out = {}
    for dtype in ("float32", "bfloat16"):
        tensors = arch.random_tensors(typed, 17, torch.float32, device="cuda")
        for name, t in tensors.items():
            if name.endswith("attn.c_attn.weight"):
                t.mul_(2.0)                 # attention that is not nearly uniform, so that a wrong key shows
            if dtype == "bfloat16" and t.dim() == 2:
                tensors[name] = t.to(torch.bfloat16)
        w = {name: t.double() for name, t in tensors.items()}
        want, moved = {}, 0.0
        for r, tokens in requests.items():
            exact = plain_gpt2.logits_of(XL, w, tokens, rows=wanted[r])
            if dtype == "bfloat16":
                rounded = plain_gpt2.logits_of(XL, w, tokens, rounded=torch.bfloat16, rows=wanted[r])
                moved = max(moved, (rounded - exact).abs().max().item())
            want[r] = dict(zip(wanted[r], exact.float().cpu()))
        del w
        torch.cuda.empty_cache()
        out[dtype] = (tensors, requests, wanted, want, FLOAT32_TOL if dtype == "float32" else 3.0 * moved + 2e-3)
    return out


@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_depth_cuttings(xl, dtype, mode):
    from damendaemon_b200.engine import Engine, StepEntry
    tensors, requests, wanted, want, tol = xl[dtype]
    page = 16
    if mode == "mixed":
        builder, kv = mixed_steps(requests, seed=5, max_live=3, wanted=wanted, portions=(2, 3, 17, 64, 130, 256))
    else:
        builder = {"whole": whole_steps, "tail": tail_steps, "portions": portion_steps}[mode](requests, wanted=wanted)
        kv = 1024
    engine = Engine(config=XL, tensors=tensors, dtype=dtype, kv_tokens=kv, page_size=page, max_requests=4)
    for g in engine.cache.groups:
        g.arena.fill_(float("nan"))
    seen, worst = {r: set() for r in requests}, 0.0
    for s in builder.steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]
        if entries:
            logits = engine.step(entries).cpu()
            for (r, p), row in zip(builder.where[s["step"]], logits):
                assert torch.isfinite(row).all(), f"{dtype} {mode}: non-finite logits at request {r} position {p}"
                err = (row - want[r][p]).abs().max().item()
                assert err < tol, f"{dtype} {mode}: request {r} position {p} differs by {err:.3e} (allowed {tol:.1e})"
                worst = max(worst, err)
                if dtype == "float32":
                    a, b = int(row.argmax()), int(want[r][p].argmax())
                    # the same greedy token, unless the plain logits of the two candidates are closer than rounding
                    assert a == b or abs(float(want[r][p][a] - want[r][p][b])) <= 2 * err, \
                        f"{mode}: request {r} position {p}: greedy token {a}, plain {b}"
                seen[r].add(p)
        for r in s["end"]:
            engine.finish(r)
        engine.cache.check()
    assert all(seen[r] == set(wanted[r]) for r in requests)
    assert engine.cache.used_tokens == 0 and not engine.live_requests()
    if mode == "mixed":
        handed_out = sum((len(t) + page - 1) // page for t in requests.values())
        assert engine.cache.groups[0].pool.n_pages < handed_out, "the pool is too large for pages to be used again"
    print(f"\nGPT-2 XL, 48 layers, {dtype}, {mode}: max |logit - plain| = {worst:.3e} (allowed {tol:.3e})")
