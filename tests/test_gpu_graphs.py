"""Steps replayed from captured CUDA graphs, as generation runs them: the same counts (tokens, entries, wanted rows)
come back with other lengths per entry, other start positions and other pages, in bfloat16 with the tensor-core
prompt attention (head size 64), its fused cache write, the separate cache write for portions that start inside a
key block, and mixed steps of decoded tokens beside portions. And a decode step of 64 requests of unequal length
at the benchmark's layer sizes, whose block tables are wider than one block of the page-streaming kernel holds."""
import pytest
import torch

from conftest import TINY_C
from model_tools import make_model
from plain_gpt2 import PlainGpt2, read_folder, logits_of

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model_c(tmp_path_factory):
    folder = make_model(tmp_path_factory.mktemp("graphs") / "C", TINY_C, seed=2, dtype="bfloat16", sharpen=3.0)
    return folder, PlainGpt2(folder)


def three_places(n):
    return sorted({0, n // 2, n - 1}) if n >= 3 else None


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_replayed_prompt_and_mixed_steps(model_c, dtype):
    from damendaemon_b200.engine import Engine, StepEntry
    folder, plain = model_c
    vocab = TINY_C["vocab_size"]
    g = torch.Generator().manual_seed(9)
    engine = Engine(folder, dtype=dtype, kv_tokens=1024, page_size=16, max_requests=8, use_graph=True)
    engine.capture_after = {True: 1, False: 1}      # every shape is captured when it comes back for the first time
    for group in engine.cache.groups:
        group.arena.fill_(float("nan"))
    # (first portions, second portions, a newcomer's prompt): each trial has the counts of the others
    trials = [((100, 156), (20, 12), 31), ((156, 100), (12, 20), 31), ((128, 128), (16, 16), 31), ((60, 196), (5, 27), 31),
              ((130, 126), (27, 5), 31)]
    tol, checked = None, 0
    for t, (first, second, newcomer) in enumerate(trials):
        a, b, c = f"a{t}", f"b{t}", f"c{t}"
        tokens = {a: torch.randint(0, vocab, (first[0] + second[0] + 4,), generator=g).tolist(),
                  b: torch.randint(0, vocab, (first[1] + second[1] + 4,), generator=g).tolist(),
                  c: torch.randint(0, vocab, (newcomer + 3,), generator=g).tolist()}
        want = {r: plain.logits(ids).float() for r, ids in tokens.items()}
        if dtype == "bfloat16":
            moved = max((plain.logits(ids, rounded=torch.bfloat16).float() - want[r]).abs().max().item()
                        for r, ids in tokens.items())
            tol = max(tol or 0.0, 3.0 * moved + 2e-3)
        else:
            tol = 1e-4
        at = {r: 0 for r in tokens}

        def run(parts):
            """parts: [(request, n tokens, wanted places)]; checks every wanted row against the plain logits."""
            nonlocal checked
            entries = [StepEntry(r, tokens[r][at[r]:at[r] + n], places) for r, n, places in parts]
            out = engine.step(entries).cpu()
            i = 0
            for r, n, places in parts:
                for w in places:
                    err = (out[i] - want[r][at[r] + w]).abs().max().item()
                    assert err < tol, f"trial {t}: request {r} position {at[r] + w} differs by {err:.3e} (allowed {tol:.1e})"
                    i += 1
                    checked += 1
                at[r] += n
        # whole first portions from position 0 (every entry on a key-block boundary: the prompt kernel writes the cache)
        run([(a, first[0], [0, first[0] // 2, first[0] - 1]), (b, first[1], [0, first[1] // 2, first[1] - 1])])
        # second portions that start inside a key block (separate cache write), read what the first left
        run([(a, second[0], [0, second[0] - 1]), (b, second[1], [0, second[1] - 1])])
        # decoded tokens of a and b beside the whole prompt of a newcomer
        run([(a, 1, [0]), (b, 1, [0]), (c, newcomer, [newcomer - 1])])
        # decode steps of all three
        for _ in range(3):
            run([(a, 1, [0]), (b, 1, [0]), (c, 1, [0])])
        for r in tokens:
            engine.finish(r)
        engine.cache.check()
    # Four shapes come back; each is captured at its second appearance and runs as a replay from then on: the first portions
    # (5 times), the second portions off a key-block boundary (4 times; the trial whose second portions start at 128 has
    # the same counts but starts on boundaries, another shape, seen once), the mixed step (5), the decode step (15).
    assert len(engine._graphs) == 4
    # (a float32 engine's attention has no key blocks: there the odd trial's second portions are the same shape as the others')
    assert engine.graph_replays == (4 + 3 + 4 + 14 if engine.portion_multiple > 1 else 4 + 4 + 4 + 14)
    assert engine.raise_device_errors() is None and checked == len(trials) * 22


XL2_LONG = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_layer": 2, "n_embd": 1600, "n_head": 25,
            "n_inner": 6400, "vocab_size": 50257, "n_positions": 2048, "layer_norm_epsilon": 1e-5,
            "activation_function": "gelu_new"}


@pytest.fixture(scope="module")
def xl_long(tmp_path_factory):
    folder = make_model(tmp_path_factory.mktemp("xl_long") / "m", XL2_LONG, seed=8, dtype="bfloat16", sharpen=2.0)
    config, w = read_folder(folder)
    w = {k: v.cuda() for k, v in w.items()}
    g = torch.Generator().manual_seed(12)
    n_decode = 4
    lengths = [1, 2, 7, 8, 9, 15, 16, 17, 31, 33, 63, 64, 65, 100, 127, 128, 129, 200, 255, 256, 257, 300, 383, 384,
               400, 450, 500, 511, 512, 513, 600, 640, 700, 767, 768, 769, 800, 850, 900, 1000, 1023, 1024, 1025, 1100,
               1200, 1279, 1280, 1281, 1300, 1400, 1500, 1535, 1536, 1537, 1600, 1700, 1800, 1900, 2000, 2040, 3, 5, 50, 77]
    assert len(lengths) == 64
    tokens = [torch.randint(0, 50257, (n + n_decode,), generator=g).tolist() for n in lengths]
    want, moved = [], 0.0
    for n, seq in zip(lengths, tokens):
        rows = list(range(n - 1, n + n_decode))
        exact = logits_of(config, w, seq, rows=rows)
        rounded = logits_of(config, w, seq, rounded=torch.bfloat16, rows=rows)
        moved = max(moved, (rounded - exact).abs().max().item())
        want.append(exact.float().cpu())
    del w
    torch.cuda.empty_cache()
    return folder, lengths, tokens, want, 3.0 * moved + 2e-3, n_decode


@pytest.mark.parametrize("use_graph", [False, True])
@pytest.mark.parametrize("page_size", [8, 16])
def test_decode_of_sixty_four_requests(xl_long, page_size, use_graph):
    """64 requests of 1 to 2,040 tokens decoded together in bfloat16: with pages of 8 tokens a block table is 256 pages
    wide, twice what one block of the page-streaming attention kernel holds. Every decoded position of every request
    is held against the plain implementation run on that request alone."""
    from damendaemon_b200.engine import Engine, StepEntry
    folder, lengths, tokens, want, tol, n_decode = xl_long
    kv = sum((n + n_decode + page_size - 1) // page_size * page_size for n in lengths)
    engine = Engine(folder, dtype="bfloat16", kv_tokens=kv, page_size=page_size, max_requests=64, use_graph=use_graph)
    for group in engine.cache.groups:
        group.arena.fill_(float("nan"))
    batch, budget = [], 0
    order = sorted(range(64), key=lambda r: (r * 37) % 64)          # prompts enter in a scrambled order
    def flush():
        out = engine.step([StepEntry(r, tokens[r][:lengths[r]], [lengths[r] - 1]) for r in batch]).cpu()
        for i, r in enumerate(batch):
            err = (out[i] - want[r][0]).abs().max().item()
            assert err < tol, f"prompt of request {r} ({lengths[r]} tokens) differs by {err:.3e} (allowed {tol:.1e})"
    for r in order:
        if budget + lengths[r] > 4096:
            flush()
            batch, budget = [], 0
        batch.append(r)
        budget += lengths[r]
    flush()
    for step in range(n_decode):
        out = engine.step([StepEntry(r, [tokens[r][lengths[r] + step]], [0]) for r in range(64)]).cpu()
        for r in range(64):
            err = (out[r] - want[r][1 + step]).abs().max().item()
            assert err < tol, f"request {r} ({lengths[r]} tokens), decoded token {step}: differs by {err:.3e} (allowed {tol:.1e})"
    if use_graph:
        assert engine.graph_replays >= n_decode - 2
    for r in range(64):
        engine.finish(r)
    engine.cache.check()
    assert engine.cache.used_tokens == 0
    assert engine.raise_device_errors() is None
