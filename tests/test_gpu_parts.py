"""Each part alone against the plain function it implements, and a toy mixer with state of its own
that is registered, built and stepped without touching the framework's files."""
import json
from dataclasses import dataclass
from types import SimpleNamespace

import pytest
import torch

import plain_gpt2 as plain
from damendaemon_b200.cache import CacheManager, RequestState
from damendaemon_b200.parts import (AttentionSpec, DenseFeedForwardSpec, EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, NormSpec, PositionSpec,
                                    RunEntry, Runtime, TensorDecl, register_mixer)
from damendaemon_b200.parts.interfaces import Mixer
from damendaemon_b200.registry import Architecture, register_architecture

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
TOL = {torch.float32: 2e-5, torch.bfloat16: 3e-2}


def runtime(dtype):
    return Runtime(dtype=dtype, device=DEV)


def context_for(cache, requests, dtype):
    """A StepContext for whole sequences [(request, n_tokens)], built by hand."""
    from damendaemon_b200.engine.context import StepContext
    ids, pos, ent, slots, starts, tables = [], [], [], [], [0], {g.name: [] for g in cache.groups}
    for i, (r, n) in enumerate(requests):
        p0 = cache.length.get(r, 0) if r in cache.slot_of else 0
        if r not in cache.slot_of:
            cache.admit(r)
        cache.extend([(r, p0 + n)])
        pos += list(range(p0, p0 + n)); ent += [i] * n; ids += [0] * n
        slots.append(cache.slot_of[r]); starts.append(starts[-1] + n)
        for g in cache.groups:
            tables[g.name].append(torch.from_numpy(g.table_array[cache.slot_of[r]].copy()))
        cache.advance(r, p0 + n)
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return StepContext(n_tokens=len(ids), n_entries=len(requests), n_wanted=0, token_ids=t(ids), positions=t(pos),
                       token_entry=t(ent), want_rows=t([]), entry_slot=t(slots), entry_start=t(starts), entry_pos0=t([0] * len(requests)),
                       block_tables={k: torch.stack(v).to(DEV) for k, v in tables.items()},
                       host={"lengths": [n for _, n in requests], "slots": slots}, runtime=runtime(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layernorm_part(dtype):
    from damendaemon_b200.parts.norms import LayerNorm
    g = torch.Generator().manual_seed(0)
    x = torch.randn(11, 72, generator=g) * 2 + 1
    w = {"n.weight": torch.randn(72, generator=g), "n.bias": torch.randn(72, generator=g)}
    spec = NormSpec("layernorm", 72, 3e-4, "n.weight", "n.bias")
    assert [d.name for d in LayerNorm.tensor_decls(spec)] == ["n.weight", "n.bias"]
    part = LayerNorm(spec, {k: v.to(DEV) for k, v in w.items()}, runtime(dtype))
    want = plain.layer_norm(x.double(), w["n.weight"].double(), w["n.bias"].double(), 3e-4)
    assert (part.forward(x.to(DEV)).double().cpu() - want).abs().max() < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("activation", ["gelu_new", "gelu"])
def test_dense_feed_forward_part(dtype, activation):
    from damendaemon_b200.parts.feed_forward import DenseFeedForward
    g = torch.Generator().manual_seed(1)
    width, inner, n = 72, 200, 13
    raw = {"h.0.mlp.c_fc.weight": torch.randn(width, inner, generator=g) * 0.1, "h.0.mlp.c_fc.bias": torch.randn(inner, generator=g) * 0.1,
           "h.0.mlp.c_proj.weight": torch.randn(inner, width, generator=g) * 0.1, "h.0.mlp.c_proj.bias": torch.randn(width, generator=g) * 0.1}
    raw = {k: (v.to(dtype).float() if v.dim() == 2 else v) for k, v in raw.items()}     # what the engine dtype can hold
    spec = DenseFeedForwardSpec("dense", width, inner, activation, "h.0.mlp.c_fc.weight", "h.0.mlp.c_fc.bias",
                                "h.0.mlp.c_proj.weight", "h.0.mlp.c_proj.bias", stored_in_out=True)
    shapes = {d.name: d.shape for d in DenseFeedForward.tensor_decls(spec)}
    assert shapes["h.0.mlp.c_fc.weight"] == (width, inner)
    placed = {k: (v.t().contiguous().to(dtype) if v.dim() == 2 else v).to(DEV) for k, v in raw.items()}
    part = DenseFeedForward(spec, placed, runtime(dtype))
    y = torch.randn(n, width, generator=g).to(dtype)
    residual = torch.randn(n, width, generator=g)
    want = residual.double() + plain.mlp_block(y.double(), {k: v.double() for k, v in raw.items()}, "h.0.", activation)
    got = part.forward(y.to(DEV), residual.to(DEV).clone(), None)
    assert got.dtype == torch.float32 and (got.double().cpu() - want).abs().max() < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_part_and_learned_positions(dtype):
    from damendaemon_b200 import kernels
    from damendaemon_b200.parts.attention import Attention
    from damendaemon_b200.parts.positions import LearnedPositions
    g = torch.Generator().manual_seed(2)
    width, heads, n = 96, 3, 21
    raw = {"h.0.attn.c_attn.weight": torch.randn(width, 3 * width, generator=g) * 0.3, "h.0.attn.c_attn.bias": torch.randn(3 * width, generator=g) * 0.1,
           "h.0.attn.c_proj.weight": torch.randn(width, width, generator=g) * 0.1, "h.0.attn.c_proj.bias": torch.randn(width, generator=g) * 0.1}
    raw = {k: (v.to(dtype).float() if v.dim() == 2 else v) for k, v in raw.items()}
    spec = AttentionSpec("attention", width, heads, heads, 32, 0.11, None, "h.0.attn.c_attn.weight", "h.0.attn.c_attn.bias",
                         "h.0.attn.c_proj.weight", "h.0.attn.c_proj.bias", stored_in_out=True)
    placed = {k: (v.t().contiguous().to(dtype) if v.dim() == 2 else v).to(DEV) for k, v in raw.items()}
    part = Attention(spec, placed, runtime(dtype))
    cache = CacheManager([Attention.cache_needs(spec)], 64, 8, 2, 64)
    cache.allocate(DEV, dtype)
    cache.groups[0].arena.fill_(float("nan"))
    ctx = context_for(cache, [("a", n)], dtype)
    y = torch.randn(n, width, generator=g).to(dtype)
    residual = torch.randn(n, width, generator=g)
    positions = LearnedPositions(PositionSpec("learned", 64, width, "wpe"), {"wpe": torch.zeros(64, width, device=DEV, dtype=dtype)}, runtime(dtype))
    got = part.forward(y.to(DEV), residual.to(DEV).clone(), ctx, cache.layer_view(0), positions)
    want = residual.double() + plain.attention_block(y.double(), {k: v.double() for k, v in raw.items()}, "h.0.", heads, 0.11)
    # bfloat16 rounds the projected q, k, v and the attended values: the bound is relative to their size (~6 here)
    bound = TOL[dtype] if dtype == torch.float32 else 3 * 2.0 ** -8 * float(want.abs().max())
    assert (got.double().cpu() - want).abs().max() < bound
    # learned positions: the table is what the embedding kernel adds
    table = torch.randn(64, width, generator=g).to(dtype).to(DEV)
    tokens = torch.randn(50, width, generator=g).to(dtype).to(DEV)
    lp = LearnedPositions(PositionSpec("learned", 64, width, "wpe"), {"wpe": table}, runtime(dtype))
    ids = torch.tensor([4, 9, 9], dtype=torch.int32, device=DEV)
    pos = torch.tensor([0, 7, 63], dtype=torch.int32, device=DEV)
    x = kernels.embed(ids, pos, tokens, lp.embedding_table())
    assert torch.equal(x.cpu(), tokens[ids.long()].float().cpu() + table[pos.long()].float().cpu())


# ---------------------------------------------------------------------------------------------------
# A toy mixer with state of its own: out[t] = gain * (state + sum of y[0..t]); the state is the sum so far.

@dataclass(frozen=True)
class ToyStateSpec:
    kind: str
    width: int
    gain: str


class ToyStateMixer(Mixer):
    graph_safe = False        # it plans on the host (a loop over entries)

    def __init__(self, spec, weights, runtime):
        self.spec, self.gain = spec, weights[spec.gain]

    @staticmethod
    def tensor_decls(spec):
        return [TensorDecl(spec.gain, (spec.width,), "vector")]

    @staticmethod
    def cache_needs(spec):
        return [RequestState((spec.width,), "float32")]

    def forward(self, y, residual, ctx, cache, position):
        start = 0
        for n, slot in zip(ctx.host["lengths"], ctx.host["slots"]):
            running = cache.state[slot] + torch.cumsum(y[start:start + n].float(), 0)
            cache.state[slot] = running[-1]
            residual[start:start + n] += running * self.gain
            start += n
        return residual


@dataclass(frozen=True)
class ToyConfig:
    width: int
    vocab: int
    positions: int
    order: str = "twice"

    def to_dict(self):
        return {"architectures": ["ToyStateLM"], "width": self.width, "vocab": self.vocab, "positions": self.positions,
                "order": self.order}


RUN_ORDERS = {"twice": (RunEntry(0), RunEntry(1), RunEntry(1)),
              "borrow": (RunEntry(0), RunEntry(1), RunEntry(1, cache_of=1))}


def toy_spec(c):
    def norm(name):
        return NormSpec("layernorm", c.width, 1e-5, name + ".weight", name + ".bias")
    ff = lambda i: DenseFeedForwardSpec("dense", c.width, 2 * c.width, "gelu_new", f"l{i}.up.weight", f"l{i}.up.bias",
                                        f"l{i}.down.weight", f"l{i}.down.bias")
    layers = (
        LayerSpec("pre_norm", ToyStateSpec("toy_state", c.width, "l0.gain"), ff(0), (norm("l0.n1"), norm("l0.n2"))),
        LayerSpec("pre_norm", AttentionSpec("attention", c.width, 2, 1, c.width // 2, (c.width // 2) ** -0.5, None,
                                            "l1.qkv.weight", None, "l1.out.weight", None), ff(1), (norm("l1.n1"), norm("l1.n2"))),
    )
    # layer 1 runs twice: the order of layers is data. "twice": each run has its own cache;
    # "borrow": the second run reads the keys and values of the first and writes none
    return ModelSpec("ToyStateLM", c.vocab, c.width, c.positions, EmbeddingSpec("tokens", c.vocab, c.width, "embed.weight"),
                     PositionSpec("learned", c.positions, c.width, "pos.weight"), layers, RUN_ORDERS[c.order],
                     HeadSpec("linear", c.vocab, c.width, norm("final"), "embed.weight", tied=True))


def toy_tensors(c, seed, dtype=torch.float32):
    from damendaemon_b200.parts import tensor_decls
    g = torch.Generator().manual_seed(seed)
    out = {}
    for d in tensor_decls(toy_spec(c)):
        t = torch.randn(d.shape, generator=g) * (0.2 if len(d.shape) == 2 else 0.1)
        if d.name.endswith("n1.weight") or d.name.endswith("n2.weight") or d.name == "final.weight":
            t = t + 1
        out[d.name] = t.to(dtype) if len(d.shape) == 2 else t
    return out


def toy_plain(c, w, ids):
    """The same model with ordinary tensor arithmetic, whole sequence."""
    w = {k: v.double() for k, v in w.items()}
    ids = torch.as_tensor(ids)
    x = w["embed.weight"][ids] + w["pos.weight"][torch.arange(len(ids))]
    ln = lambda x, n: plain.layer_norm(x, w[n + ".weight"], w[n + ".bias"], 1e-5)
    ff = lambda x, i: plain.gelu_new(x @ w[f"l{i}.up.weight"].t() + w[f"l{i}.up.bias"]) @ w[f"l{i}.down.weight"].t() + w[f"l{i}.down.bias"]
    x = x + torch.cumsum(ln(x, "l0.n1"), 0) * w["l0.gain"]
    x = x + ff(ln(x, "l0.n2"), 0)
    d = c.width // 2
    for run in range(2):
        qkv = ln(x, "l1.n1") @ w["l1.qkv.weight"].t()
        q = qkv[:, :2 * d].reshape(-1, 2, d)
        if run == 0 or c.order == "twice":
            k, v = qkv[:, 2 * d:3 * d].reshape(-1, 1, d), qkv[:, 3 * d:].reshape(-1, 1, d)
        o = plain.causal_attention(q, k.expand(-1, 2, -1), v.expand(-1, 2, -1), d ** -0.5).reshape(len(ids), 2 * d)
        x = x + o @ w["l1.out.weight"].t()
        x = x + ff(ln(x, "l1.n2"), 1)
    return ln(x, "final") @ w["embed.weight"].t()


@pytest.mark.parametrize("order", ["twice", "borrow"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_registers_builds_and_steps(dtype, order):
    from damendaemon_b200.engine import Engine, StepEntry
    register_mixer("toy_state", ToyStateMixer, replace=True)
    register_architecture(Architecture("ToyStateLM", lambda raw: ToyConfig(raw["width"], raw["vocab"], raw["positions"], raw.get("order", "twice")),
                                       toy_spec, toy_tensors), replace=True)
    c = ToyConfig(48, 211, 64, order)
    tensors = toy_tensors(c, 3, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    engine = Engine(config=c.to_dict(), tensors=tensors, dtype=dtype, kv_tokens=128, page_size=8, max_requests=3, use_graph=True)
    assert not engine.use_graph                         # the toy mixer plans on the host
    from damendaemon_b200.parts import cache_needs
    assert [[type(x).__name__ for x in n] for n in cache_needs(engine.spec)] == \
        [["RequestState"], ["PagedKeyValues"], ["PagedKeyValues"] if order == "twice" else []]
    assert engine.cache.groups[0].arena.shape[0] == (2 if order == "twice" else 1)
    assert engine.cache.state[0].shape == (3, 48)
    g = torch.Generator().manual_seed(4)
    a, b = (torch.randint(0, 211, (n,), generator=g).tolist() for n in (40, 23))
    want = {"a": toy_plain(c, tensors, a).float(), "b": toy_plain(c, tensors, b).float()}
    tol = 1e-4 if dtype == "float32" else 6e-2
    # a in portions, b joins later, the state carries across steps and slots do not mix
    got_a = [engine.step([StepEntry("a", a[:7], list(range(7)))])]
    both = engine.step([StepEntry("a", a[7:30], list(range(23))), StepEntry("b", b[:10], list(range(10)))])
    got_a.append(both[:23]); got_b = [both[23:]]
    for t in a[30:]:
        got_a.append(engine.step([StepEntry("a", [t], [0])]))
    got_b.append(engine.step([StepEntry("b", b[10:], list(range(13)))], end=["a", "b"]))
    assert (torch.cat(got_a).cpu() - want["a"]).abs().max() < tol
    assert (torch.cat(got_b).cpu() - want["b"]).abs().max() < tol
    # a finished request's slot starts from zero state again
    again = engine.step([StepEntry("c", b, list(range(23)))])
    assert (again.cpu() - want["b"]).abs().max() < tol


def test_bfloat16_width_that_is_no_multiple_of_8():
    """A reduction width that TMA cannot take (100 = 4 mod 8) falls to the CUDA-core GEMM, never to a wrong result."""
    from damendaemon_b200.parts.linear import linear
    g = torch.Generator().manual_seed(9)
    a = torch.randn(5, 100, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(36, 100, generator=g).to(torch.bfloat16).to(DEV)
    out = linear(runtime(torch.bfloat16), a, w, out_dtype=torch.float32)
    assert (out.double() - a.double() @ w.double().t()).abs().max() < 1e-3
