"""Chains of small products and norms in one persistent kernel (csrc/decode_chain.cu) against float64 formulas of
the same bfloat16 operands, at other sizes than the engine's, and against the separate kernels they stand for."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def K():
    from damendaemon_b200 import kernels
    kernels.library("tensor")
    kernels.chain_barrier(DEV)
    return kernels


def bf16(t):
    return t.to(torch.bfloat16)


def gelu_new(u):
    return 0.5 * u * (1 + torch.tanh(math.sqrt(2 / math.pi) * (u + 0.044715 * u ** 3)))


def layer_norm(x, gamma, beta, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * gamma + beta


@pytest.mark.parametrize("M,N,Kd", [(1, 8, 32), (3, 40, 96), (8, 1600, 1600), (5, 4800, 1600), (8, 1600, 6400), (7, 6400, 1600),
                                    (2, 2368, 3104), (8, 152, 12288)])
def test_one_product_with_every_epilogue(K, M, N, Kd):
    g = torch.Generator().manual_seed(M * 1000 + N)
    a = bf16(torch.randn(M, Kd, generator=g)).to(DEV)
    w = bf16(torch.randn(N, Kd, generator=g) / math.sqrt(Kd)).to(DEV)
    bias, res = torch.randn(N, generator=g).to(DEV), torch.randn(M, N, generator=g).to(DEV)
    base = a.double() @ w.double().t()
    before = K.chains_launched
    with K.chain():
        plain = K.gemm_tcgen05(a, w, out_dtype=torch.float32)
        act = K.gemm_tcgen05(a, w, bias, activation="gelu_new")
        erf = K.gemm_tcgen05(a, w, bias, activation="gelu", out_dtype=torch.float32)
        stream = res.clone()
        K.gemm_tcgen05(a, w, bias, residual=stream, out_dtype=torch.float32, out=stream)
    assert K.chains_launched == before + 1, "four independent products are four phases of one kernel"
    assert K.read_error_flag(DEV) == 0
    tol = 2e-4 * math.sqrt(Kd / 64)
    assert (plain.double() - base).abs().max() < tol
    want = gelu_new(base + bias.double())
    assert act.dtype == torch.bfloat16 and (act.double() - want).abs().max() < 2.0 ** -8 * float(want.abs().max()) + 1e-3
    want = 0.5 * (base + bias.double()) * (1 + torch.erf((base + bias.double()) / math.sqrt(2)))
    assert (erf.double() - want).abs().max() < 2 * tol
    assert (stream.double() - (base + bias.double() + res.double())).abs().max() < 2 * tol


@pytest.mark.parametrize("M", [1, 4, 8])
@pytest.mark.parametrize("width,inner,heads_width", [(1600, 6400, 4800), (192, 416, 576), (2080, 96, 64)])
def test_a_layer_as_one_chain(K, M, width, inner, heads_width):
    """Output projection + residual, norm, up projection + gelu, down projection + residual, the next norm and the next
    projection: six operations, four phases, one kernel; against float64 with the same roundings at the hand-overs.
    Run three times over: the barrier's words must come back to where they were."""
    g = torch.Generator().manual_seed(width + M)
    rnd = lambda *shape, scale=1.0: (torch.randn(*shape, generator=g) * scale)
    attended = bf16(rnd(M, width)).to(DEV)
    w_proj, w_up = bf16(rnd(width, width, scale=width ** -0.5)).to(DEV), bf16(rnd(inner, width, scale=width ** -0.5)).to(DEV)
    w_down, w_qkv = bf16(rnd(width, inner, scale=inner ** -0.5)).to(DEV), bf16(rnd(heads_width, width, scale=width ** -0.5)).to(DEV)
    b_proj, b_up, b_down, b_qkv = (rnd(n, scale=0.1).to(DEV) for n in (width, inner, width, heads_width))
    g2, be2, g1, be1 = (1 + rnd(width, scale=0.1)).to(DEV), rnd(width, scale=0.1).to(DEV), (1 + rnd(width, scale=0.1)).to(DEV), rnd(width, scale=0.1).to(DEV)
    x0 = rnd(M, width, scale=2.0).to(DEV)
    d = lambda t: t.double()
    x1 = d(x0) + d(attended) @ d(w_proj).t() + d(b_proj)
    y2 = d(bf16(layer_norm(x1, d(g2), d(be2), 1e-5)))
    hidden = d(bf16(gelu_new(y2 @ d(w_up).t() + d(b_up))))
    x2 = x1 + hidden @ d(w_down).t() + d(b_down)
    y1 = d(bf16(layer_norm(x2, d(g1), d(be1), 1e-6)))
    qkv = y1 @ d(w_qkv).t() + d(b_qkv)
    for _ in range(3):
        x = x0.clone()
        before = K.chains_launched
        with K.chain():
            K.gemm_tcgen05(attended, w_proj, b_proj, residual=x, out_dtype=torch.float32, out=x)
            n2 = K.layernorm(x, g2, be2, 1e-5, torch.bfloat16)
            h = K.gemm_tcgen05(n2, w_up, b_up, activation="gelu_new")
            K.gemm_tcgen05(h, w_down, b_down, residual=x, out_dtype=torch.float32, out=x)
            n1 = K.layernorm(x, g1, be1, 1e-6, torch.bfloat16)
            got = K.gemm_tcgen05(n1, w_qkv, b_qkv)
        assert K.chains_launched == before + 1
        assert K.read_error_flag(DEV) == 0
        scale = float(qkv.abs().max())
        assert (d(x) - x2).abs().max() < 2.0 ** -7 * float(x2.abs().max()), "residual stream"
        assert (d(n2) - y2).abs().max() < 2.0 ** -6 * float(y2.abs().max()), "the first norm's rows, as left for other readers"
        assert (d(n1) - y1).abs().max() < 2.0 ** -6 * float(y1.abs().max())
        assert (d(got) - qkv).abs().max() < 2.0 ** -6 * scale + 1e-2
    assert K.chain_barrier(DEV)[0].item() == 0


def test_chain_equals_the_separate_kernels_and_steps_aside_for_what_it_does_not_take(K):
    """A norm whose reader is no product, a product whose sizes the chain does not take (N no multiple of 8, K no
    multiple of 32), and another kernel in the middle: everything runs, in order, and gives what the separate kernels
    give."""
    g = torch.Generator().manual_seed(4)
    x = torch.randn(6, 96, generator=g).to(DEV)
    gamma, beta = (1 + 0.1 * torch.randn(96, generator=g)).to(DEV), (0.1 * torch.randn(96, generator=g)).to(DEV)
    w_a = bf16(torch.randn(100, 96, generator=g) * 0.1).to(DEV)        # N = 100: not taken
    w_b = bf16(torch.randn(64, 96, generator=g) * 0.1).to(DEV)
    w_c = bf16(torch.randn(96, 104, generator=g) * 0.1).to(DEV)        # K = 104: not taken
    w_d = bf16(torch.randn(104, 64, generator=g) * 0.1).to(DEV)

    def run():
        y = K.layernorm(x, gamma, beta, 1e-5, torch.bfloat16)
        a = K.gemm_tcgen05(y, w_a, out_dtype=torch.float32)
        b = K.gemm_tcgen05(y, w_b)
        z = K.layernorm(x, gamma, None, 1e-5, torch.bfloat16)         # nobody in the chain reads it
        d = K.gemm_tcgen05(b, w_d)
        c = K.gemm_tcgen05(d, w_c, out_dtype=torch.float32)
        ids = K.sample(c)                                              # another kernel: the chain runs before it
        return y, a, b, z, d, c, ids
    want = run()
    with K.chain():
        got = run()
    for i, (u, v) in enumerate(zip(got, want)):
        assert (u.double() - v.double()).abs().max() <= 2.0 ** -7 * float(v.double().abs().max()) + 1e-6, f"result {i}"
    assert torch.equal(got[-1], want[-1])
    assert K.read_error_flag(DEV) == 0


def test_refusals(K):
    a = torch.zeros(9, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 64, dtype=torch.bfloat16, device=DEV)
    assert not K.chain_takes(9, 8, 64) and not K.chain_takes(8, 12, 64) and not K.chain_takes(8, 8, 48)
    assert not K.chain_takes(8, 8, 12320) and K.chain_takes(8, 8, 12288)
    with K.chain():
        out = K.gemm_tcgen05(a, w)          # nine rows: the ordinary kernel takes it
    assert out.shape == (9, 8) and float(out.abs().max()) == 0.0
