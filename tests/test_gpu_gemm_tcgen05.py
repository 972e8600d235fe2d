"""The tcgen05/TMA GEMM alone against a float64 product of the same bfloat16 operands."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def K():
    from damendaemon_b200 import kernels
    kernels.library("tensor")
    return kernels


def operands(M, N, Kd, seed=0):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(M, Kd, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, Kd, generator=g) / math.sqrt(Kd)).to(torch.bfloat16).to(DEV)
    return a, w, torch.randn(N, generator=g).to(DEV), torch.randn(M, N, generator=g).to(DEV)


# (tokens, features, reduction): tile edges, k tails, widths and vocabularies that are no power of two
SHAPES = [(1, 128, 64), (5, 200, 96), (16, 130, 320), (17, 1000, 96), (33, 96, 64), (64, 4800, 1600), (100, 1600, 6400),
          (129, 515, 200), (300, 257, 1608), (8, 50257, 1600), (2048, 1600, 1600)]


@pytest.mark.parametrize("shape", SHAPES)
def test_plain_product(K, shape):
    M, N, Kd = shape
    a, w, bias, res = operands(M, N, Kd)
    out = K.gemm_tcgen05(a, w, out_dtype=torch.float32)
    assert K.read_error_flag(DEV) == 0
    ref = a.double() @ w.double().t()
    err = (out.double() - ref).abs().max().item()
    assert err < 2e-4 * math.sqrt(Kd / 64), f"{shape}: {err}"          # float32 accumulation of exact bf16 products


@pytest.mark.parametrize("shape", [(7, 300, 192), (64, 1600, 6400), (200, 6400, 1600), (1, 4800, 1600)])
def test_epilogues(K, shape):
    M, N, Kd = shape
    a, w, bias, res = operands(M, N, Kd, seed=1)
    base = a.double() @ w.double().t() + bias.double()
    gelu_new = 0.5 * base * (1 + torch.tanh(math.sqrt(2 / math.pi) * (base + 0.044715 * base ** 3)))
    gelu_erf = 0.5 * base * (1 + torch.erf(base / math.sqrt(2)))
    rel = lambda ref: 2.0 ** -8 * float(ref.abs().max()) + 1e-3
    out = K.gemm_tcgen05(a, w, bias)
    assert out.dtype == torch.bfloat16 and (out.double() - base).abs().max() < rel(base)
    assert (K.gemm_tcgen05(a, w, bias, activation="gelu_new").double() - gelu_new).abs().max() < rel(gelu_new)
    assert (K.gemm_tcgen05(a, w, bias, activation="gelu").double() - gelu_erf).abs().max() < rel(gelu_erf)
    stream = res.clone()
    K.gemm_tcgen05(a, w, bias, residual=stream, out_dtype=torch.float32, out=stream)
    assert (stream.double() - (base + res.double())).abs().max() < 5e-4 * math.sqrt(Kd / 64)
    assert K.read_error_flag(DEV) == 0


@pytest.mark.parametrize("splits", [1, 2, 5, 13])
@pytest.mark.parametrize("tile", [16, 32, 64])
def test_forced_splits_and_tiles(K, splits, tile):
    a, w, bias, res = operands(40 if tile < 64 else 150, 700, 1600, seed=2)
    ref = a.double() @ w.double().t() + bias.double()
    out = K.gemm_tcgen05(a, w, bias, out_dtype=torch.float32, splits=splits, token_tile=tile)
    again = K.gemm_tcgen05(a, w, bias, out_dtype=torch.float32, splits=splits, token_tile=tile)
    assert K.read_error_flag(DEV) == 0
    assert (out.double() - ref).abs().max() < 1e-3
    assert torch.equal(out, again), "split-K sums in a fixed order: two runs are bit-equal"


@pytest.mark.parametrize("splits", [2, 3, 5, 8, 12, 16])
@pytest.mark.parametrize("tokens,tile,cluster", [(1, 16, 1), (8, 16, 1), (13, 16, 1), (30, 32, 1), (64, 64, 1), (40, 16, 1),
                                                 (64, 16, 1), (50, 32, 1), (1, 16, 3), (6, 16, 3), (16, 16, 3), (35, 16, 3)])
def test_cluster_split(K, splits, tokens, tile, cluster):
    """K split inside a thread-block cluster of up to 16 blocks, partial tiles reduced over distributed shared memory
    (16 bytes a store, only the pieces that hold a token); cluster 3: the rings of 10 stages (with 2 splits a block
    has more k-blocks than stages). Token counts that end anywhere in a piece of four and in a tile."""
    a, w, bias, res = operands(tokens, 700, 1600, seed=4)
    ref = a.double() @ w.double().t() + bias.double()
    out = K.gemm_tcgen05(a, w, bias, out_dtype=torch.float32, splits=splits, token_tile=tile, cluster=cluster)
    again = K.gemm_tcgen05(a, w, bias, out_dtype=torch.float32, splits=splits, token_tile=tile, cluster=cluster)
    assert K.read_error_flag(DEV) == 0
    assert (out.double() - ref).abs().max() < 1e-3
    assert torch.equal(out, again), "the partial tiles are added in rank order: two runs are bit-equal"
    stream = res.clone()
    K.gemm_tcgen05(a, w, bias, residual=stream, out_dtype=torch.float32, out=stream, splits=splits, token_tile=tile, cluster=cluster)
    assert (stream.double() - (ref + res.double())).abs().max() < 1e-3
    gelu = K.gemm_tcgen05(a, w, bias, activation="gelu_new", splits=splits, token_tile=tile, cluster=cluster)
    u = ref
    want = 0.5 * u * (1 + torch.tanh(math.sqrt(2 / math.pi) * (u + 0.044715 * u ** 3)))
    assert (gelu.double() - want).abs().max() < 2.0 ** -8 * float(want.abs().max()) + 1e-3


@pytest.mark.parametrize("tile", [128, 192, 256])
@pytest.mark.parametrize("shape", [(300, 520, 200), (129, 257, 1608), (65, 50257, 64), (700, 1600, 320)])
def test_token_lane_tiles(K, tile, shape):
    """Tiles of 128 tokens x tile features (one SM): rows moved in 16-byte pieces where every row start allows it,
    element by element at a ragged last chunk (520 = 32 x 16 + 8), with rows that are not 16-byte aligned (257
    floats), a bias or an output that starts off a 16-byte boundary, and an output inside a wider buffer."""
    M, N, Kd = shape
    a, w, bias, res = operands(M, N, Kd, seed=7)
    ref = a.double() @ w.double().t() + bias.double()
    tol = 5e-4 * math.sqrt(Kd / 64)
    out = K.gemm_tcgen05(a, w, bias, out_dtype=torch.float32, splits=1, token_tile=tile, cluster=0)
    assert (out.double() - ref).abs().max() < tol
    shifted = torch.zeros(N + 1, device=DEV)
    shifted[1:] = bias
    assert torch.equal(out, K.gemm_tcgen05(a, w, shifted[1:], out_dtype=torch.float32, splits=1, token_tile=tile, cluster=0))
    wide = torch.full((M, N + 24), 7.0, device=DEV)
    K.gemm_tcgen05(a, w, bias, out_dtype=torch.float32, out=wide[:, 8:8 + N], splits=1, token_tile=tile, cluster=0)
    assert torch.equal(wide[:, 8:8 + N], out) and bool((wide[:, :8] == 7).all()) and bool((wide[:, 8 + N:] == 7).all())
    odd = torch.full((M, N + 3), 7.0, device=DEV)
    K.gemm_tcgen05(a, w, bias, out_dtype=torch.float32, out=odd[:, 1:1 + N], splits=1, token_tile=tile, cluster=0)
    assert torch.equal(odd[:, 1:1 + N], out) and bool((odd[:, :1] == 7).all()) and bool((odd[:, 1 + N:] == 7).all())
    stream = res.clone()
    K.gemm_tcgen05(a, w, bias, residual=stream, out_dtype=torch.float32, out=stream, splits=1, token_tile=tile, cluster=0)
    assert (stream.double() - (ref + res.double())).abs().max() < tol
    half = K.gemm_tcgen05(a, w, bias, splits=1, token_tile=tile, cluster=0)
    assert half.dtype == torch.bfloat16 and (half.double() - ref).abs().max() < 2.0 ** -8 * float(ref.abs().max()) + 1e-3
    half_wide = torch.full((M, N + 24), 7.0, device=DEV, dtype=torch.bfloat16)
    K.gemm_tcgen05(a, w, bias, out=half_wide[:, 8:8 + N], splits=1, token_tile=tile, cluster=0)
    assert torch.equal(half_wide[:, 8:8 + N], half) and bool((half_wide[:, :8] == 7).all()) and bool((half_wide[:, 8 + N:] == 7).all())
    gelu = K.gemm_tcgen05(a, w, bias, activation="gelu_new", splits=1, token_tile=tile, cluster=0)
    want = 0.5 * ref * (1 + torch.tanh(math.sqrt(2 / math.pi) * (ref + 0.044715 * ref ** 3)))
    assert (gelu.double() - want).abs().max() < 2.0 ** -7 * float(want.abs().max()) + 1e-3
    erf = K.gemm_tcgen05(a, w, bias, activation="gelu", out_dtype=torch.float32, splits=1, token_tile=tile, cluster=0)
    assert (erf.double() - 0.5 * ref * (1 + torch.erf(ref / math.sqrt(2)))).abs().max() < tol
    assert K.read_error_flag(DEV) == 0
    if Kd >= 128:
        with pytest.raises(K.KernelError, match="no K split"):
            K.gemm_tcgen05(a, w, bias, splits=2, token_tile=tile, cluster=0)


@pytest.mark.parametrize("tile", [128, 192, 256])
@pytest.mark.parametrize("shape", [(300, 257, 1608), (2048, 1600, 1600), (1000, 4800, 320), (130, 520, 64)])
def test_two_sms_per_tile(K, tile, shape):
    """tcgen05 cta_group::2: a cluster of two blocks on one tile of 256 tokens, every epilogue."""
    M, N, Kd = shape
    a, w, bias, res = operands(M, N, Kd, seed=6)
    ref = a.double() @ w.double().t() + bias.double()
    out = K.gemm_tcgen05(a, w, bias, out_dtype=torch.float32, splits=1, token_tile=tile, cluster=2)
    assert K.read_error_flag(DEV) == 0
    assert (out.double() - ref).abs().max() < 5e-4 * math.sqrt(Kd / 64)
    assert torch.equal(out, K.gemm_tcgen05(a, w, bias, out_dtype=torch.float32, splits=1, token_tile=128, cluster=0))
    stream = res.clone()
    K.gemm_tcgen05(a, w, bias, residual=stream, out_dtype=torch.float32, out=stream, splits=1, token_tile=tile, cluster=2)
    assert (stream.double() - (ref + res.double())).abs().max() < 5e-4 * math.sqrt(Kd / 64)
    half = K.gemm_tcgen05(a, w, bias, activation="gelu_new", splits=1, token_tile=tile, cluster=2)
    want = 0.5 * ref * (1 + torch.tanh(math.sqrt(2 / math.pi) * (ref + 0.044715 * ref ** 3)))
    assert (half.double() - want).abs().max() < 2.0 ** -7 * float(want.abs().max()) + 1e-3
    assert K.read_error_flag(DEV) == 0


def test_strided_views_and_refusals(K):
    a, w, bias, res = operands(20, 256, 128, seed=3)
    wide = torch.zeros(20, 128 + 64, dtype=torch.bfloat16, device=DEV)
    wide[:, 64:] = a
    out = K.gemm_tcgen05(wide[:, 64:], w, out_dtype=torch.float32)
    assert torch.equal(out, K.gemm_tcgen05(a, w, out_dtype=torch.float32))
    with pytest.raises(K.KernelError, match="multiples of 8"):
        K.gemm_tcgen05(a[:, :100].contiguous(), w[:, :100].contiguous())
    with pytest.raises(K.KernelError, match="bfloat16"):
        K.gemm_tcgen05(a.float(), w.float())


def test_a_wait_that_runs_out_is_reported_and_the_device_goes_on(K):
    """A barrier at which nobody arrives, waited on through the function every pipeline of the library waits with,
    under a limit of 2 ms: the wait gives up, the kernel returns, bit 8 stands in the error word, a second waiting warp
    leaves through the block's abort flag well before its own limit, and a product right after it is correct."""
    assert K.read_error_flag(DEV) == 0
    limit = 2_000_000
    first, second = K.wait_probe(limit, DEV)
    torch.cuda.synchronize()
    assert K.read_error_flag(DEV) == 8
    assert limit <= first < 50 * limit, f"the first warp gave up after {first} ns"
    assert 0 < second < 5 * limit, f"the second warp left after {second} ns, not with the block's abort flag"
    assert K.read_error_flag(DEV) == 0          # reading cleared it
    a, w, bias, res = operands(8, 1600, 1600, seed=3)
    out = K.gemm_tcgen05(a, w, out_dtype=torch.float32)
    assert (out.double() - a.double() @ w.double().t()).abs().max().item() < 2e-4 * math.sqrt(1600 / 64)
    assert K.read_error_flag(DEV) == 0
    with pytest.raises(K.KernelError):
        K.wait_probe(2_000_000_000, DEV)        # limits beyond a second are refused
