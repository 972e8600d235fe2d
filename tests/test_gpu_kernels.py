"""Each CUDA-core kernel alone against a plain float64 reference, at sizes the engine's tiny
models do not use (widths and vocabularies that are no power of two, grouped heads, windows)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def K():
    from damendaemon_b200 import kernels
    kernels.library("core")
    return kernels


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(K, dtype):
    g = torch.Generator().manual_seed(0)
    wte = torch.randn(301, 80, generator=g).to(dtype).to(DEV)
    wpe = torch.randn(77, 80, generator=g).to(dtype).to(DEV)
    ids = torch.randint(0, 301, (50,), generator=g, dtype=torch.int32).to(DEV)
    pos = torch.randint(0, 77, (50,), generator=g, dtype=torch.int32).to(DEV)
    out = K.embed(ids, pos, wte, wpe)
    ref = wte[ids.long()].float() + wpe[pos.long()].float()
    assert out.dtype == torch.float32 and torch.equal(out, ref)
    assert torch.equal(K.embed(ids, pos, wte, None), wte[ids.long()].float())
    assert K.read_error_flag(DEV) == 0
    bad = ids.clone(); bad[3] = 301
    K.embed(bad, pos, wte, wpe)
    assert K.read_error_flag(DEV) == 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [100, 1600])
def test_layernorm(K, dtype, width):
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(9, width, generator=g) * 3 + 5).to(DEV)       # a large mean shows a one-pass variance
    gamma, beta = torch.randn(width, generator=g).to(DEV), torch.randn(width, generator=g).to(DEV)
    eps = 1e-6
    x64 = x.double()
    ref = (x64 - x64.mean(-1, keepdim=True)) / torch.sqrt(x64.var(-1, unbiased=False, keepdim=True) + eps) * gamma.double() + beta.double()
    out = K.layernorm(x, gamma, beta, eps, dtype)
    assert out.dtype == dtype
    assert (out.double() - ref).abs().max() < (1e-5 if dtype == torch.float32 else 4e-2)
    rows = torch.tensor([7, 2, 2], dtype=torch.int32, device=DEV)
    picked = K.layernorm(x, gamma, beta, eps, dtype, row_index=rows)
    assert torch.equal(picked, out[rows.long()])
    nobeta = K.layernorm(x, gamma, None, eps, torch.float32)
    assert (nobeta.double() - (ref - beta.double())).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(37, 53, 45), (1, 130, 96), (70, 64, 320), (13, 200, 100), (30, 3300, 136), (40, 1600, 1600),
                                   (150, 200, 72), (300, 130, 1600)])
def test_gemm_simt(K, dtype, shape):
    M, N, Kd = shape
    g = torch.Generator().manual_seed(2)
    a = torch.randn(M, Kd, generator=g).to(dtype).to(DEV)
    w = torch.randn(N, Kd, generator=g).to(dtype).to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    res = torch.randn(M, N, generator=g).to(DEV)
    base = a.double() @ w.double().t()
    # bfloat16 results are rounded to 8 bits of mantissa: the bound is relative to the value
    t = 1e-4 if dtype == torch.float32 else 2.0 ** -8 * float(base.abs().max()) + 1e-3
    # float32 results: 1,600 float32 additions in a row at values up to a hundred need a bound that goes with the value
    # (64 units in the last place of a float32)
    t32 = 1e-4 if Kd <= 320 else 2.0 ** -18 * float(base.abs().max())
    if dtype == torch.float32:
        t = t32
    out = K.gemm_simt(a, w)
    assert out.dtype == dtype and (out.double() - base).abs().max() < t
    u = base + bias.double()
    gelu_new = 0.5 * u * (1 + torch.tanh(math.sqrt(2 / math.pi) * (u + 0.044715 * u ** 3)))
    gelu_erf = 0.5 * u * (1 + torch.erf(u / math.sqrt(2)))
    assert (K.gemm_simt(a, w, bias, activation="gelu_new").double() - gelu_new).abs().max() < t
    assert (K.gemm_simt(a, w, bias, activation="gelu").double() - gelu_erf).abs().max() < t
    stream = res.clone()
    got = K.gemm_simt(a, w, bias, residual=stream, out_dtype=torch.float32, out=stream)
    assert got.data_ptr() == stream.data_ptr()
    assert (stream.double() - (u + res.double())).abs().max() < t32
    # a row's result does not depend on the other rows of the batch
    alone = K.gemm_simt(a[3:4].contiguous() if M > 3 else a, w, bias)
    whole = K.gemm_simt(a, w, bias)
    assert torch.equal(alone[0], whole[3 if M > 3 else 0])
    # ... nor on the kernel that the number of rows selects (up to 8, 16, 32 and 64 rows stream the weights once; more
    # rows run in tiles of 128 x 128; operands that are not 16-byte aligned in tiles of 64 x 64): the same bits
    for m in (2, 8, 9, 16, 17, 32, 33, 64, 65, 129):
        if m < M:
            assert torch.equal(K.gemm_simt(a[:m], w, bias), whole[:m]), f"{m} rows alone differ from the same rows among {M}"


def paged_case(K, dtype, n_heads, kv_heads, d, page, lengths, new, window, n_splits, seed=0, poison=True, spike=None,
               store=True):
    """Requests with `lengths` tokens of which the last `new` are this step's queries."""
    g = torch.Generator().manual_seed(seed)
    max_blocks = (max(lengths) + page - 1) // page + 1
    n_pages = sum((L + page - 1) // page for L in lengths) + 5
    perm = torch.randperm(n_pages, generator=g).tolist()
    cache = torch.full((n_pages, 2, kv_heads, page, d), float("nan") if poison else 0.0).to(dtype).to(DEV)
    table = torch.full((len(lengths), max_blocks), -1, dtype=torch.int32)
    qs, ks, vs, ent, pos = [], [], [], [], []
    refs = []
    scale = d ** -0.5
    for e, (L, n) in enumerate(zip(lengths, new)):
        q = torch.randn(L, n_heads, d, generator=g)
        k = torch.randn(L, kv_heads, d, generator=g)
        v = torch.randn(L, kv_heads, d, generator=g)
        if spike is not None and L > spike + 1:
            # one far key stands out for the last query
            k[spike] *= 0; k[spike, :, 0] = 30.0
            q[L - 1] *= 0; q[L - 1, :, 0] = 30.0
        q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
        for b in range((L + page - 1) // page):
            table[e, b] = perm.pop()
        # earlier tokens are already in the cache
        for j in range(L - n):
            pg = table[e, j // page]
            cache[pg, 0, :, j % page] = k[j].to(DEV)
            cache[pg, 1, :, j % page] = v[j].to(DEV)
        qs.append(q[L - n:]); ks.append(k[L - n:]); vs.append(v[L - n:])
        ent += [e] * n; pos += list(range(L - n, L))
        rep = n_heads // kv_heads
        kk, vv = k.double().repeat_interleave(rep, 1), v.double().repeat_interleave(rep, 1)
        s = torch.einsum("ihd,jhd->hij", q.double(), kk) * scale
        i, j = torch.arange(L)[:, None], torch.arange(L)[None, :]
        vis = j <= i
        if window:
            vis = vis & (j > i - window)
        s = s.masked_fill(~vis, float("-inf"))
        refs.append(torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), vv)[L - n:].reshape(n, n_heads * d))
    q = torch.cat(qs).reshape(-1, n_heads * d).to(DEV)
    k = torch.cat(ks).reshape(-1, kv_heads * d).to(DEV)
    v = torch.cat(vs).reshape(-1, kv_heads * d).to(DEV)
    # the three live side by side in one buffer, as after a fused QKV projection
    packed = torch.cat([q, k, v], 1).contiguous()
    qv, kv_, vv_ = packed[:, :n_heads * d], packed[:, n_heads * d:(n_heads + kv_heads) * d], packed[:, (n_heads + kv_heads) * d:]
    ent = torch.tensor(ent, dtype=torch.int32, device=DEV)
    pos = torch.tensor(pos, dtype=torch.int32, device=DEV)
    table = table.to(DEV)
    if store:
        K.kv_store(kv_, vv_, ent, pos, table, cache)
    return dict(q=qv, cache=cache, ent=ent, pos=pos, table=table, ref=torch.cat(refs), scale=scale, packed=packed)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,d,page", [(6, 2, 48, 8), (5, 5, 16, 16), (3, 1, 128, 4), (2, 2, 200, 16)])
@pytest.mark.parametrize("window", [None, 7])
def test_attention_rows_mixed(K, dtype, heads, kv_heads, d, page, window):
    c = paged_case(K, dtype, heads, kv_heads, d, page, lengths=[37, 1, 90, 64], new=[37, 1, 2, 1], window=window, n_splits=1)
    out = K.attention_rows(c["q"], c["cache"], c["ent"], c["pos"], c["table"], heads, c["scale"], window)
    assert K.read_error_flag(DEV) == 0
    assert not torch.isnan(out.float()).any(), "a key outside the live range was read"
    assert (out.double().cpu() - c["ref"]).abs().max() < tol(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_splits", [2, 5, 32])
def test_attention_rows_split_decode(K, dtype, n_splits):
    c = paged_case(K, dtype, 4, 2, 64, 16, lengths=[300, 33, 1, 700], new=[1, 1, 1, 1], window=None, n_splits=n_splits,
                   spike=5)
    out = K.attention_rows(c["q"], c["cache"], c["ent"], c["pos"], c["table"], 4, c["scale"], None, n_splits=n_splits)
    assert K.read_error_flag(DEV) == 0
    assert (out.double().cpu() - c["ref"]).abs().max() < tol(dtype)
    one = K.attention_rows(c["q"], c["cache"], c["ent"], c["pos"], c["table"], 4, c["scale"], None, n_splits=1)
    assert (out.float() - one.float()).abs().max() < tol(dtype)


@pytest.mark.parametrize("d,heads,page", [(64, 5, 16), (128, 3, 8), (64, 25, 16)])
@pytest.mark.parametrize("n_splits", [1, 3, 8])
@pytest.mark.parametrize("window", [None, 100])
def test_attention_decode_bf16(K, d, heads, page, n_splits, window):
    """The bfloat16 decode kernel: contexts from 1 to 1000 keys, a far key that stands out, fragmented pages."""
    K.library("tensor")
    assert K.attention_decode_supported(heads, heads, d, torch.bfloat16)
    assert not K.attention_decode_supported(heads, 1, d, torch.bfloat16) or heads == 1
    assert not K.attention_decode_supported(heads, heads, 48, torch.bfloat16)
    c = paged_case(K, torch.bfloat16, heads, heads, d, page, lengths=[300, 33, 1, 1000, 129], new=[1, 1, 1, 1, 1],
                   window=window, n_splits=n_splits, spike=5 if window is None else 250)
    out = K.attention_decode(c["q"], c["cache"], c["ent"], c["pos"], c["table"], heads, c["scale"], window, n_splits=n_splits)
    again = K.attention_decode(c["q"], c["cache"], c["ent"], c["pos"], c["table"], heads, c["scale"], window, n_splits=n_splits)
    assert K.read_error_flag(DEV) == 0
    assert not torch.isnan(out.float()).any(), "a key outside the live range was read"
    assert (out.double().cpu() - c["ref"]).abs().max() < tol(torch.bfloat16)
    assert torch.equal(out, again), "the split counters were not left at zero"
    # fused cache write: wipe the newest key and value from the pages, hand them over beside q
    packed = c["packed"]
    hd = heads * d
    wiped = c["cache"].clone()
    for e, (L, n) in enumerate(zip([300, 33, 1, 1000, 129], [1] * 5)):
        pg = int(c["table"][e, (L - 1) // page])
        wiped[pg, :, :, (L - 1) % page] = float("nan")
    fused = K.attention_decode(packed[:, :hd], wiped, c["ent"], c["pos"], c["table"], heads, c["scale"], window,
                               n_splits=n_splits, k_new=packed[:, hd:2 * hd], v_new=packed[:, 2 * hd:])
    assert K.read_error_flag(DEV) == 0
    assert torch.equal(fused, out)
    same = (wiped == c["cache"]) | (torch.isnan(wiped.float()) & torch.isnan(c["cache"].float()))
    assert bool(same.all()), "the fused kernel did not write the new key and value into the cache"


@pytest.mark.parametrize("heads,page", [(5, 16), (25, 16), (17, 32), (3, 64), (2, 128), (33, 16)])
@pytest.mark.parametrize("n_splits", [1, 2, 3, 8, 11])
@pytest.mark.parametrize("window", [None, 100])
def test_attention_decode_pages(K, heads, page, n_splits, window):
    """The page-streaming decode kernel (TMA boxes of a group of heads): contexts from 1 to 1000 keys that end anywhere
    in a page, a far key, fragmented pages, a poisoned cache, head counts that fill one, two or three groups unevenly,
    more splits than some requests have pages; then the fused cache write."""
    K.library("tensor")
    assert K.attention_decode_pages_supported(heads, heads, 64, page, torch.bfloat16)
    assert not K.attention_decode_pages_supported(heads, heads, 128, page, torch.bfloat16)
    assert not K.attention_decode_pages_supported(heads, heads, 64, 8, torch.bfloat16)
    assert not K.attention_decode_pages_supported(heads, 1, 64, page, torch.bfloat16) or heads == 1
    lengths = [300, 33, 1, 1000, 129, 512]
    c = paged_case(K, torch.bfloat16, heads, heads, 64, page, lengths=lengths, new=[1] * 6,
                   window=window, n_splits=n_splits, spike=5 if window is None else 250)
    run = lambda q, cache, **kw: K.attention_decode(q, cache, c["ent"], c["pos"], c["table"], heads, c["scale"], window,
                                                    n_splits=n_splits, kernel="pages", **kw)
    out = run(c["q"], c["cache"])
    again = run(c["q"], c["cache"])
    assert K.read_error_flag(DEV) == 0
    assert not torch.isnan(out.float()).any(), "a key outside the live range was read"
    assert (out.double().cpu() - c["ref"]).abs().max() < tol(torch.bfloat16)
    assert torch.equal(out, again), "the split counters were not left at zero"
    packed = c["packed"]
    hd = heads * 64
    wiped = c["cache"].clone()
    for e, L in enumerate(lengths):
        pg = int(c["table"][e, (L - 1) // page])
        wiped[pg, :, :, (L - 1) % page] = float("nan")
    fused = run(packed[:, :hd], wiped, k_new=packed[:, hd:2 * hd], v_new=packed[:, 2 * hd:])
    assert K.read_error_flag(DEV) == 0
    assert torch.equal(fused, out)
    same = (wiped == c["cache"]) | (torch.isnan(wiped.float()) & torch.isnan(c["cache"].float()))
    assert bool(same.all()), "the fused kernel did not write the new key and value into the cache"
    assert 1 <= K.attention_decode_pages_splits(8, heads, page, 1000, DEV) <= (1000 + page - 1) // page


@pytest.mark.parametrize("heads,page", [(25, 16), (8, 64), (20, 32)])
@pytest.mark.parametrize("n_splits", [3, 8])
@pytest.mark.parametrize("window", [None, 100])
def test_attention_decode_pages_deals_its_splits(K, heads, page, n_splits, window):
    """More blocks in the grid than can be resident: the kernel deals the key splits out from all tokens' positions,
    long contexts get several, short ones one, and the blocks beyond a token's count leave. Twenty tokens with
    contexts from 1 to 1000 keys, without an entry index (token t is entry t), then the fused cache write."""
    K.library("tensor")
    lengths = [1000, 3, 17, 640, 1, 255, 256, 257, 511, 90, 1000, 33, 800, 64, 128, 5, 700, 16, 15, 999]
    c = paged_case(K, torch.bfloat16, heads, heads, 64, page, lengths=lengths, new=[1] * len(lengths),
                   window=window, n_splits=n_splits, spike=5 if window is None else 250)
    run = lambda q, cache, **kw: K.attention_decode(q, cache, None, c["pos"], c["table"], heads, c["scale"], window,
                                                    n_splits=n_splits, kernel="pages", **kw)
    out = run(c["q"], c["cache"])
    again = run(c["q"], c["cache"])
    assert K.read_error_flag(DEV) == 0
    assert not torch.isnan(out.float()).any(), "a key outside the live range was read"
    assert (out.double().cpu() - c["ref"]).abs().max() < tol(torch.bfloat16)
    assert torch.equal(out, again), "the split counters were not left at zero"
    packed = c["packed"]
    hd = heads * 64
    wiped = c["cache"].clone()
    for e, L in enumerate(lengths):
        wiped[int(c["table"][e, (L - 1) // page]), :, :, (L - 1) % page] = float("nan")
    fused = run(packed[:, :hd], wiped, k_new=packed[:, hd:2 * hd], v_new=packed[:, 2 * hd:])
    assert K.read_error_flag(DEV) == 0
    assert torch.equal(fused, out)
    same = (wiped == c["cache"]) | (torch.isnan(wiped.float()) & torch.isnan(c["cache"].float()))
    assert bool(same.all()), "the fused kernel did not write the new key and value into the cache"


@pytest.mark.parametrize("d,heads,kv_heads,page", [(64, 5, 5, 16), (128, 4, 2, 8), (64, 6, 1, 32)])
@pytest.mark.parametrize("window", [None, 70])
def test_attention_prefill_bf16(K, d, heads, kv_heads, page, window):
    """The tensor-core kernel: whole prompts, a portion that continues 300 cached keys, single tokens, a far key."""
    K.library("tensor")
    assert K.attention_prefill_supported(heads, kv_heads, d, torch.bfloat16)
    assert not K.attention_prefill_supported(heads, kv_heads, 48, torch.bfloat16)
    lengths, new = [150, 1, 365, 64, 700, 65], [150, 1, 65, 64, 1, 3]
    c = paged_case(K, torch.bfloat16, heads, kv_heads, d, page, lengths=lengths, new=new, window=window, n_splits=1,
                   spike=3 if window is None else None)
    starts = [0]
    for n in new:
        starts.append(starts[-1] + n)
    entry_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
    entry_pos0 = torch.tensor([L - n for L, n in zip(lengths, new)], dtype=torch.int32, device=DEV)
    out = K.attention_prefill(c["q"], c["cache"], entry_start, entry_pos0, c["table"], heads, c["scale"], window)
    assert K.read_error_flag(DEV) == 0
    assert not torch.isnan(out.float()).any(), "a key outside the live range was read"
    assert (out.double().cpu() - c["ref"]).abs().max() < tol(torch.bfloat16)
    rows = K.attention_rows(c["q"], c["cache"], c["ent"], c["pos"], c["table"], heads, c["scale"], window)
    assert (out.float() - rows.float()).abs().max() < tol(torch.bfloat16)


@pytest.mark.parametrize("heads,kv_heads,page", [(5, 5, 16), (6, 1, 32), (4, 2, 8), (3, 3, 128), (2, 1, 64)])
@pytest.mark.parametrize("window", [None, 70, 300])
def test_attention_prefill_tcgen05(K, heads, kv_heads, page, window):
    """The tcgen05 kernel (tiles of 128 queries, TMA boxes per cache page, accumulators in TMEM): whole prompts
    that end inside a page, a portion that continues cached keys, single tokens, more key blocks than the ring has
    stages, a far key, a poisoned cache around the live keys."""
    K.library("tensor")
    assert K.attention_prefill_tcgen05_supported(heads, kv_heads, 64, page, torch.bfloat16)
    assert not K.attention_prefill_tcgen05_supported(heads, kv_heads, 128, page, torch.bfloat16)
    assert not K.attention_prefill_tcgen05_supported(heads, kv_heads, 64, 48, torch.bfloat16)
    lengths, new = [150, 1, 365, 64, 1300, 65, 900, 129], [150, 1, 65, 64, 1300, 3, 130, 128]
    c = paged_case(K, torch.bfloat16, heads, kv_heads, 64, page, lengths=lengths, new=new, window=window, n_splits=1,
                   spike=3 if window is None else None)
    starts = [0]
    for n in new:
        starts.append(starts[-1] + n)
    entry_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
    entry_pos0 = torch.tensor([L - n for L, n in zip(lengths, new)], dtype=torch.int32, device=DEV)
    out = K.attention_prefill(c["q"], c["cache"], entry_start, entry_pos0, c["table"], heads, c["scale"], window, kernel="tcgen05")
    assert K.read_error_flag(DEV) == 0
    assert not torch.isnan(out.float()).any(), "a key outside the live range was read"
    assert (out.double().cpu() - c["ref"]).abs().max() < tol(torch.bfloat16)
    rows = K.attention_rows(c["q"], c["cache"], c["ent"], c["pos"], c["table"], heads, c["scale"], window)
    assert (out.float() - rows.float()).abs().max() < tol(torch.bfloat16)
    # with this step's keys and values at hand as rows beside the queries, whole key blocks of the step are read from
    # there instead of page by page: the same values, so the same result bit for bit
    hd, kd = heads * 64, kv_heads * 64
    packed = c["packed"]
    direct = K.attention_prefill(packed[:, :hd], c["cache"], entry_start, entry_pos0, c["table"], heads, c["scale"], window,
                                 kernel="tcgen05", k_new=packed[:, hd:hd + kd], v_new=packed[:, hd + kd:])
    assert K.read_error_flag(DEV) == 0
    assert torch.equal(direct, out)


@pytest.mark.parametrize("heads,kv_heads,page", [(5, 5, 16), (6, 2, 128), (4, 1, 8)])
@pytest.mark.parametrize("window", [None, 200])
def test_attention_prefill_tcgen05_writes_the_cache(K, heads, kv_heads, page, window):
    """With store_new the kernel puts the step's keys and values into the pages itself: the same result, and the
    same live cache rows bit for bit, as after kv_store. Every portion starts at a multiple of 128 keys, ends anywhere."""
    K.library("tensor")
    lengths, new = [150, 128 + 3, 256 + 300, 1, 384 + 129, 640], [150, 3, 300, 1, 129, 256]
    kw = dict(lengths=lengths, new=new, window=window, n_splits=1, spike=3 if window is None else None)
    c = paged_case(K, torch.bfloat16, heads, kv_heads, 64, page, store=False, **kw)
    stored = paged_case(K, torch.bfloat16, heads, kv_heads, 64, page, **kw)
    assert not torch.equal(c["cache"].view(torch.int16), stored["cache"].view(torch.int16))
    starts = [0]
    for n in new:
        starts.append(starts[-1] + n)
    entry_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
    entry_pos0 = torch.tensor([L - n for L, n in zip(lengths, new)], dtype=torch.int32, device=DEV)
    hd, kd = heads * 64, kv_heads * 64
    packed = c["packed"]
    out = K.attention_prefill(packed[:, :hd], c["cache"], entry_start, entry_pos0, c["table"], heads, c["scale"], window,
                              kernel="tcgen05", k_new=packed[:, hd:hd + kd], v_new=packed[:, hd + kd:], store_new=True)
    assert K.read_error_flag(DEV) == 0
    assert (out.double().cpu() - c["ref"]).abs().max() < tol(torch.bfloat16)
    # slot by slot up to each request's length; what lies beyond in a request's last page is never read
    live = torch.zeros(c["cache"].shape[0], page, dtype=torch.bool)
    for e, L in enumerate(lengths):
        for pos in range(L):
            live[int(c["table"][e, pos // page]), pos % page] = True
    live = live.to(DEV)[:, None, None, :, None]
    ours, theirs = c["cache"].view(torch.int16), stored["cache"].view(torch.int16)
    assert torch.equal(torch.where(live, ours, 0), torch.where(live, theirs, 0))
    untouched = ~live.flatten(1).any(1)                      # pages of no request
    assert torch.equal(ours[untouched], theirs[untouched])
    # a portion that starts inside a key block is refused on the device: error bit 2 and nothing written
    before = c["cache"].clone()
    K.attention_prefill(packed[:, :hd], c["cache"], entry_start, entry_pos0 + 1, c["table"], heads, c["scale"], window,
                        kernel="tcgen05", k_new=packed[:, hd:hd + kd], v_new=packed[:, hd + kd:], store_new=True)
    assert K.read_error_flag(DEV) & 2
    assert torch.equal(c["cache"].view(torch.int16), before.view(torch.int16))
    with pytest.raises(K.KernelError, match="store_new"):
        K.attention_prefill(packed[:, :hd], c["cache"], entry_start, entry_pos0, c["table"], heads, c["scale"], window,
                            kernel="tcgen05", store_new=True)


def test_attention_rejects_bad_sizes(K):
    cache = torch.zeros(4, 2, 2, 16, 20, device=DEV)
    q = torch.zeros(1, 40, device=DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(K.KernelError, match="head size"):
        K.attention_rows(q, cache, z, z, torch.zeros(1, 2, dtype=torch.int32, device=DEV), 2, 1.0)
    with pytest.raises(K.KernelError, match="no CPU fallback"):
        K.layernorm(torch.zeros(2, 8), torch.zeros(8), None, 1e-5, torch.float32)


def test_attention_missing_page_sets_flag(K):
    c = paged_case(K, torch.float32, 2, 2, 16, 8, lengths=[20], new=[1], window=None, n_splits=1, poison=False)
    c["table"][0, 1] = -1
    K.attention_rows(c["q"], c["cache"], c["ent"], c["pos"], c["table"], 2, c["scale"])
    assert K.read_error_flag(DEV) == 4


def test_sampling(K):
    import sys
    from plain_gpt2 import sample_token
    g = torch.Generator().manual_seed(5)
    V = 1003
    logits = (torch.randn(6, V, generator=g) * 3)
    logits[1, 17] = logits[1, 400] = 50.0           # a tie: the first index wins
    logits[2, 5] = float("nan")
    logits[3, :] = float("-inf")
    logits[4, 9] = float("inf")
    dev = logits.to(DEV)
    greedy = K.sample(dev).cpu().tolist()
    assert greedy[0] == int(logits[0].argmax()) and greedy[1] == 17 and greedy[2:5] == [-1, -1, -1]
    assert greedy[5] == int(logits[5].argmax())
    rows = torch.randn(64, V, generator=g) * 2
    temps = torch.tensor([0.0, 0.8, 1.0, 1.7] * 16)
    us = torch.rand(64, generator=g, dtype=torch.float64)
    us[1], us[2] = 0.0, 1.0 - 2 ** -53
    got = K.sample(rows.to(DEV), temps.to(DEV), us.to(DEV)).cpu().tolist()
    for r in range(64):
        want = sample_token(rows[r], float(temps[r]), float(us[r]))
        if got[r] != want:
            # only a draw within rounding of a boundary of the CDF may differ, and then by one neighbour
            z = torch.softmax(rows[r].double() / float(temps[r]), 0).cumsum(0)
            assert abs(got[r] - want) == 1 and (z[min(got[r], want)] - float(us[r])).abs() < 1e-6
    # a padded row stride is honoured
    wide = torch.zeros(3, V + 13); wide[:, :V] = rows[:3]; wide[:, V:] = 100.0
    assert K.sample(wide.to(DEV)[:, :V]).cpu().tolist() == [int(rows[i].argmax()) for i in range(3)]


def test_early_launch_can_be_switched_for_a_stretch_of_launches(K):
    """kernels.pdl_scope: programmatic dependent launch off (or on) inside, what was in force before afterwards, also
    when scopes nest or an exception passes through; results do not depend on it."""
    K.library("core")
    x = torch.randn(9, 64, device=DEV)
    w = torch.randn(40, 64, device=DEV)
    assert K._pdl is True
    with K.pdl_scope(False):
        assert K._pdl is False
        quiet = K.gemm_simt(x, w)
        with K.pdl_scope(True):
            assert K._pdl is True
        assert K._pdl is False
    assert K._pdl is True
    with pytest.raises(ValueError):
        with K.pdl_scope(False):
            raise ValueError("passes through")
    assert K._pdl is True
    assert torch.equal(quiet, K.gemm_simt(x, w))
