// Decode attention that streams whole cache pages with TMA, for bfloat16 caches with head size 64, as many
// key/value heads as heads, and pages of 16, 32, 64 or 128 tokens.
//
// In the cache a page holds the keys of all heads side by side and then the values ([page][K|V][head][slot][64]):
// the keys of G neighbouring heads are one run of G x page_size rows of 128 bytes. A block owns (token, group of
// G <= 8 heads, split of the token's pages); thread 0 asks TMA for one box of G x page_size rows of keys and one
// of values per page, as many pages ahead as the ring holds, so a block moves its bytes in pieces of tens of KB with two instructions
// each (copying the same bytes 16 at a time, one key row per 8 lanes, the memory system delivered 4.5 TB/s;
// in boxes of this size it delivers 5.4). The 128-byte swizzle of the tensor map is the layout ldmatrix wants.
// Each of the 8 warps owns one head of the group for all pages, so nothing is merged inside the block:
// scores and P.V on mma.sync m16n8k16 with the single query in row 0 (see attention_decode.cu), running maximum
// and sum in float32, base 2 (damendaemon/kernels.py:147-178; split merge by log-sum-exp kernels.py:190-210).
//
// With k_new/v_new the step's own key and value replace the cache row of the token's position in shared memory
// and are written to the cache by the warp that owns the head. Rows of the last page beyond the position are
// zeroed in shared memory (values) or masked by index (scores), so stale cache contents never reach the result.
// n_splits is the most splits a token's pages may be cut into (the grid's third dimension); when the grid then holds
// more blocks than can be resident at once, the kernel gives each token its share of them, by its number of pages
// among all tokens' pages (see the kernel), and the blocks beyond a token's count leave at once.
// Every wait on a barrier is bounded (error bit 8).
#include "common.cuh"
#include "tcgen05.cuh"
#include <math_constants.h>

namespace {
constexpr int D = 64, TILE = 16, WARPS = 8, THREADS = WARPS * 32, HEADS_PER_WARP = 1, MAX_GROUP = WARPS * HEADS_PER_WARP;
constexpr int MAX_BLOCK_PAGES = 128;          // pages a block may own (their ids live in shared memory); 1 << 7 below
constexpr int MAX_STAGES = 6;

struct Params {
    const __nv_bfloat16* q;
    const __nv_bfloat16* k_new;
    const __nv_bfloat16* v_new;
    __nv_bfloat16* cache;
    const int* tok_entry;
    const int* tok_pos;
    const int* block_table;
    __nv_bfloat16* out;
    float* part_o;
    float* part_ml;
    int* counters;
    int* error_flag;
    int q_stride, out_stride, max_blocks, H, G, P, n_pages, window, stages;
    int n_tokens, log2_P;
    int deal;                    // 1: more blocks in the grid than can be resident, so the splits are dealt out (see the kernel)
    float inv_block_budget;      // 1 / blocks that can be resident at once: the key splits are dealt out against them
    float scale_log2e;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t* r) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t* r) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// The same product when only row 0 of A is not zero: rows 8..15 of the result are zero whatever B holds, so their two
// accumulators are fed with zeros and dropped instead of being kept in registers from tile to tile.
__device__ __forceinline__ void mma_bf16_row0(float& c0, float& c1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    float d2, d3;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%10,%10};"
                 : "+f"(c0), "+f"(c1), "=f"(d2), "=f"(d3)
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(0.f));
    asm volatile("" ::"f"(d2), "f"(d3));      // the two dead accumulators count as used
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// byte offset of 16-byte chunk c of key row r in a tile of 128-byte rows under the 128-byte swizzle
__device__ __forceinline__ uint32_t tile_off(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

__global__ void __launch_bounds__(THREADS, 2)
attention_decode_pages_kernel(const __grid_constant__ CUtensorMap map_kv, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int box_bytes = p.G * p.P * 128;                 // keys (or values) of the group's heads in one page
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + (size_t)p.stages * 2 * box_bytes);
    int* page_ids = reinterpret_cast<int*>(full + MAX_STAGES);
    __shared__ int abort_flag, sh_last;
    dd_launch_dependents();

    // Positions, entries and the block table are this step's inputs, not an earlier kernel's results: they are read
    // while the kernel before this one is still running.
    // The grid holds the most splits a token may need (gridDim.z, the slowest index, so that the splits every token
    // has are launched first); how many a token gets is decided here, from all tokens' positions, so that blocks do
    // about equal work whatever the contexts are: the step's pages x head groups are dealt out over the blocks that
    // can be resident at once, a token takes its share rounded to the nearest count, and the blocks beyond it leave.
    // (One split per token with contexts spread over 1..1000 made the kernel as long as its longest token: 61 us for
    // 64 tokens x 20 heads against 44 us with the long ones cut in three; with equal contexts nothing changes.)
    const int split = blockIdx.z, g = blockIdx.y, t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int quad = lane >> 2, t4 = lane & 3;
    // (page sizes are powers of two, and the block budget's reciprocal comes from the host: a chain of integer
    // divisions here, a hundred cycles each, stood between the positions and the first page request)
    const int span = p.max_blocks << p.log2_P;              // positions the block table can describe
    auto pages_of = [&](int position, int* first) {
        position = min(max(position, 0), span - 1);
        const int from = p.window > 0 ? max(0, position - p.window + 1) : 0;
        if (first) *first = from >> p.log2_P;
        return (position >> p.log2_P) - (from >> p.log2_P) + 1;
    };
    // every warp adds up the pages of all tokens for itself (a load per lane and five shuffles for up to 32 tokens):
    // no barrier and no shared memory stand between the positions and the first page request
    const int pos = p.tok_pos[t];
    int total_pages = 0;
    if (p.deal) {
        for (int i = lane; i < p.n_tokens; i += 32) total_pages += pages_of(p.tok_pos[i], nullptr);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) total_pages += __shfl_xor_sync(0xffffffffu, total_pages, o);
    }
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    int first_page = 0;
    const int my_pages = pages_of(pos, &first_page);
    const int last_page = first_page + my_pages - 1;
    // pages a block should take: all pages x groups over the blocks that can be resident (every block of a token does
    // the same arithmetic on the same numbers, so they agree whatever the rounding)
    int n_splits = gridDim.z;               // few tokens: every token may have all the splits, the blocks fit anyway
    if (p.deal) {
        const float share = fmaxf(1.f, ceilf((float)total_pages * (float)gridDim.y * p.inv_block_budget));
        n_splits = max(1, (int)(((float)my_pages + 0.5f * share) / share));
        n_splits = max(n_splits, (my_pages + MAX_BLOCK_PAGES - 1) >> 7);
        n_splits = min(n_splits, (int)gridDim.z);
        if (split >= n_splits) return;
    }
    const int per = (my_pages + n_splits - 1) / n_splits;                // pages per split, rounded up
    const int page0 = first_page + split * per;
    const int n_mine = max(0, min(last_page + 1, page0 + per) - page0);
    // without tok_entry token t is entry t (a step of single tokens in entry order): one trip to L2 less before the pages
    const int* bt = p.block_table + (size_t)(p.tok_entry ? p.tok_entry[t] : t) * p.max_blocks;
    for (int i = threadIdx.x; i < n_mine; i += THREADS) {
        const int blk = page0 + i;
        int page = blk < p.max_blocks ? bt[blk] : -1;
        if (page < 0 || page >= p.n_pages) {
            atomicOr(p.error_flag, 4);
            page = -1;
        }
        page_ids[i] = page;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) tc::mbar_init(&full[s], 1);
        abort_flag = 0;
        tc::fence_barrier_init();
        tc::fence_proxy_async();
        tc::prefetch_tensormap(&map_kv);
    }
    __syncthreads();

    const int head0 = g * p.G;                              // first head of the group
    const int group_heads = min(p.G, p.H - head0);
    auto load_page = [&](int i) {                           // thread 0: page i of this block into stage i % stages
        const int s = i % p.stages, page = page_ids[i];
        uint8_t* dst = tiles + (size_t)s * 2 * box_bytes;
        if (page < 0) {                                     // a missing page (error bit set): nothing to wait for
            tc::mbar_arrive(&full[s]);
            return;
        }
        tc::mbar_expect_tx(&full[s], 2 * box_bytes);
        tc::tma_load_2d(dst, &map_kv, 0, ((page * 2 + 0) * p.H + head0) * p.P, &full[s]);
        tc::tma_load_2d(dst + box_bytes, &map_kv, 0, ((page * 2 + 1) * p.H + head0) * p.P, &full[s]);
    };
    // With k_new/v_new given the pages hold earlier steps' keys and values only (this step's own row is patched in
    // below), so the first stages are requested while the projection that produces the queries is still running.
    // Without them the step's row is in the cache already, written by some kernel of this step: then the wait comes first.
    if (threadIdx.x == 0 && p.k_new != nullptr)
        for (int i = 0; i < min(n_mine, p.stages); ++i) load_page(i);
    dd_grid_wait();              // the queries and this step's keys and values are the kernel before this one's work
    if (threadIdx.x == 0 && p.k_new == nullptr)
        for (int i = 0; i < min(n_mine, p.stages); ++i) load_page(i);

    // the queries of this warp's heads as A operands: row 0 of a 16-row tile, every other row zero
    uint32_t qf[HEADS_PER_WARP][D / 16][2];
    float m[HEADS_PER_WARP], l[HEADS_PER_WARP], o[HEADS_PER_WARP][D / 8][2];
#pragma unroll
    for (int u = 0; u < HEADS_PER_WARP; ++u) {
        const int hl = warp + u * WARPS;
        const __nv_bfloat16* qp = p.q + (size_t)t * p.q_stride + (size_t)(head0 + min(hl, group_heads - 1)) * D;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            qf[u][ks][0] = quad == 0 ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 2 * t4) : 0u;
            qf[u][ks][1] = quad == 0 ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8 + 2 * t4) : 0u;
        }
        m[u] = -CUDART_INF_F;
        l[u] = 0.f;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) o[u][j][0] = o[u][j][1] = 0.f;
    }

    const size_t head_plane = (size_t)p.P * D, page_stride = 2 * (size_t)p.H * head_plane;
    for (int i = 0; i < n_mine; ++i) {
        const int s = i % p.stages;
        // all threads leave together if the wait ran out for any of them
        if (!__syncthreads_and(tc::mbar_wait(&full[s], (i / p.stages) & 1, &abort_flag) ? 1 : 0)) break;
        const int page = page_ids[i];
        const int key0 = (page0 + i) * p.P;                 // first key of the page
        uint8_t* k_box = tiles + (size_t)s * 2 * box_bytes;
        uint8_t* v_box = k_box + box_bytes;
        if (page >= 0) {
#pragma unroll
            for (int u = 0; u < HEADS_PER_WARP; ++u) {
                const int hl = warp + u * WARPS;
                if (hl >= group_heads) continue;
                uint8_t* kh = k_box + (size_t)hl * p.P * 128;
                uint8_t* vh = v_box + (size_t)hl * p.P * 128;
                if (key0 + p.P > pos) {
                    // the page of the token's own position: its new key and value, and zeros for the unwritten slots
                    const int slot = pos - key0;
                    if (p.k_new != nullptr && lane < 16) {
                        const int c = lane & 7;
                        const __nv_bfloat16* src = (lane < 8 ? p.k_new : p.v_new) + (size_t)t * p.q_stride + (size_t)(head0 + hl) * D + c * 8;
                        const uint4 v = *reinterpret_cast<const uint4*>(src);
                        *reinterpret_cast<uint4*>((lane < 8 ? kh : vh) + tile_off(slot, c)) = v;
                        __nv_bfloat16* dst = p.cache + (size_t)page * page_stride + (size_t)(head0 + hl) * head_plane + (size_t)slot * D + c * 8;
                        *reinterpret_cast<uint4*>(lane < 8 ? dst : dst + (size_t)p.H * head_plane) = v;
                    }
                    for (int r = slot + 1 + (lane >> 3); r < p.P; r += 4)
                        *reinterpret_cast<uint4*>(vh + tile_off(r, lane & 7)) = make_uint4(0, 0, 0, 0);
                    __syncwarp();
                }
                for (int tt = 0; tt < p.P / TILE; ++tt) {
                    const int base = key0 + tt * TILE;
                    if (base > pos || base + TILE <= lo) continue;          // no live key in this tile
                    const uint8_t* kt = kh + tt * TILE * 128;
                    const uint8_t* vt = vh + tt * TILE * 128;
                    // scores of 16 keys against the query (row 0)
                    float sc[2][2];
                    sc[0][0] = sc[0][1] = sc[1][0] = sc[1][1] = 0.f;
                    const int mi = lane >> 3;
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks) {
                        uint32_t b[4];
                        ldmatrix_x4(smem_addr(kt + tile_off((mi >> 1) * 8 + (lane & 7), 2 * ks + (mi & 1))), b);
                        mma_bf16_row0(sc[0][0], sc[0][1], qf[u][ks][0], qf[u][ks][1], b[0], b[1]);
                        mma_bf16_row0(sc[1][0], sc[1][1], qf[u][ks][0], qf[u][ks][1], b[2], b[3]);
                    }
                    // row 0 lives in lanes 0..3 (elements 0 and 1 of each 8-key tile); the other rows are idle
                    float mx = -CUDART_INF_F;
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int key = base + nt * 8 + 2 * t4 + e;
                            const float v = (key <= pos && key >= lo) ? sc[nt][e] * p.scale_log2e : -CUDART_INF_F;
                            sc[nt][e] = v;
                            mx = fmaxf(mx, v);
                        }
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                    const float m_new = fmaxf(m[u], mx);               // the tile holds at least one live key
                    const float corr = exp2f(m[u] - m_new);
                    m[u] = m_new;
                    l[u] *= corr;
                    uint32_t pf[2];
                    {
                        const float p00 = exp2f(sc[0][0] - m_new), p01 = exp2f(sc[0][1] - m_new);
                        const float p10 = exp2f(sc[1][0] - m_new), p11 = exp2f(sc[1][1] - m_new);
                        l[u] += (p00 + p01) + (p10 + p11);
                        pf[0] = quad == 0 ? pack_bf16(p00, p01) : 0u;
                        pf[1] = quad == 0 ? pack_bf16(p10, p11) : 0u;
                    }
#pragma unroll
                    for (int j = 0; j < D / 8; ++j) { o[u][j][0] *= corr; o[u][j][1] *= corr; }
#pragma unroll
                    for (int dp = 0; dp < D / 16; ++dp) {
                        uint32_t b[4];
                        ldmatrix_x4_trans(smem_addr(vt + tile_off((mi & 1) * 8 + (lane & 7), 2 * dp + (mi >> 1))), b);
                        mma_bf16_row0(o[u][2 * dp][0], o[u][2 * dp][1], pf[0], pf[1], b[0], b[1]);
                        mma_bf16_row0(o[u][2 * dp + 1][0], o[u][2 * dp + 1][1], pf[0], pf[1], b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();                                    // every warp is done with the stage
        if (threadIdx.x == 0 && i + p.stages < n_mine) load_page(i + p.stages);
    }

    // row 0: lanes 0..3 hold dims 8j + 2*t4 + {0,1}; their sums of l differ by the keys each saw
#pragma unroll
    for (int u = 0; u < HEADS_PER_WARP; ++u) {
        const int hl = warp + u * WARPS;
        float lu = l[u];
        lu += __shfl_xor_sync(0xffffffffu, lu, 1);
        lu += __shfl_xor_sync(0xffffffffu, lu, 2);
        if (hl >= group_heads || quad != 0) continue;
        const int h = head0 + hl;
        if (n_splits == 1) {
            const float inv = lu > 0.f ? 1.f / lu : 0.f;
            __nv_bfloat16* dst = p.out + (size_t)t * p.out_stride + (size_t)h * D + 2 * t4;
#pragma unroll
            for (int j = 0; j < D / 8; ++j) *reinterpret_cast<uint32_t*>(dst + j * 8) = pack_bf16(o[u][j][0] * inv, o[u][j][1] * inv);
        } else {
            const size_t item = ((size_t)t * p.H + h) * gridDim.z + split;     // the scratch is laid out for the most splits
            float* dst = p.part_o + item * D + 2 * t4;
#pragma unroll
            for (int j = 0; j < D / 8; ++j) *reinterpret_cast<float2*>(dst + j * 8) = make_float2(o[u][j][0], o[u][j][1]);
            if (t4 == 0) { p.part_ml[2 * item] = m[u]; p.part_ml[2 * item + 1] = lu; }
        }
    }
    if (threadIdx.x == 0 && abort_flag) atomicOr(p.error_flag, 8);
    if (n_splits == 1) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int prev = atomicAdd(&p.counters[t * gridDim.y + g], 1);
        sh_last = prev == n_splits - 1;
    }
    __syncthreads();
    if (!sh_last) return;
    __threadfence();
    // The block that finished last merges the group's heads: a thread per output dimension, the partial maxima, sums
    // and outputs of eight splits requested together and merged with a running maximum.
    for (int idx = threadIdx.x; idx < group_heads * D; idx += THREADS) {
        const int h = head0 + idx / D, d = idx % D;
        const size_t first = ((size_t)t * p.H + h) * gridDim.z;
        float Mx = -CUDART_INF_F, Lx = 0.f, acc = 0.f;
        for (int sp0 = 0; sp0 < n_splits; sp0 += 8) {
            float mm[8], ll[8], oo[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const bool live = sp0 + u < n_splits;
                const size_t it = first + sp0 + (live ? u : 0);
                mm[u] = live ? __ldcg(p.part_ml + 2 * it) : -CUDART_INF_F;
                ll[u] = live ? __ldcg(p.part_ml + 2 * it + 1) : 0.f;
                oo[u] = live ? __ldcg(p.part_o + it * D + d) : 0.f;
            }
            float cm = Mx;
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (ll[u] > 0.f) cm = fmaxf(cm, mm[u]);
            if (cm == -CUDART_INF_F) continue;            // nothing live so far
            const float keep = Mx == -CUDART_INF_F ? 0.f : exp2f(Mx - cm);
            acc *= keep;
            Lx *= keep;
            Mx = cm;
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (ll[u] > 0.f) {
                    const float w = exp2f(mm[u] - Mx);
                    Lx += ll[u] * w;
                    acc += oo[u] * w;
                }
        }
        p.out[(size_t)t * p.out_stride + (size_t)h * D + d] = __float2bfloat16_rn(Lx > 0.f ? acc / Lx : 0.f);
    }
    if (threadIdx.x == 0) p.counters[t * gridDim.y + g] = 0;
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(sym);
    }
    return fn;
}

// heads per block: as many as two per warp and 256 box rows allow, spread evenly over the groups
void grouping(int n_heads, int page_size, int* group, int* n_groups) {
    const int most = MAX_GROUP < 256 / page_size ? MAX_GROUP : 256 / page_size;
    *n_groups = dd_ceil_div(n_heads, most);
    *group = dd_ceil_div(n_heads, *n_groups);
}
}  // namespace

// 1 if dd_attention_decode_pages takes the problem.
DD_API int dd_attention_decode_pages_supported(int n_heads, int n_kv_heads, int head_dim, int page_size, int dtype) {
    return dtype == DD_BF16 && n_heads == n_kv_heads && n_heads > 0 && head_dim == D &&
           (page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128);
}

// The most key splits a token of dd_attention_decode_pages may need when the longest context is `context` keys (the
// kernel's n_splits argument: the grid is laid out for it; how many splits each token really gets the kernel decides
// from all tokens' positions). At most eight, which merge in one trip to L2 (measured at 8 tokens x 25 heads x 768
// keys: 8 splits, all blocks resident, 13 us; a second wave of blocks 18 us).
DD_API int dd_attention_decode_pages_splits(int n_tokens, int n_heads, int page_size, int context, int sm_count) {
    int group = 0, n_groups = 0;
    grouping(n_heads, page_size, &group, &n_groups);
    const int pages = dd_ceil_div(context < 1 ? 1 : context, page_size);
    // A token gets pages / (all pages x groups / resident blocks) splits: with equal contexts that is resident blocks
    // / (tokens x groups); a token 2.5 times as long as the average gets 2.5 times as many, and the grid allows for
    // that much. More would only add blocks that leave at once, and while those wait for a place the next kernel
    // cannot start its prologue (64 tokens, 8 splits allowed, 1 taken: 58 us against 56).
    int splits = dd_ceil_div(5ll * 2 * sm_count, 2ll * (n_tokens < 1 ? 1 : n_tokens) * n_groups);
    // at most eight, which merge in one trip to L2, unless the context is so long that more splits still leave a block 16
    // pages (one token of 16,384 keys x 25 heads: 118 us in 8 splits, 32 blocks in all)
    const int most = pages / 16 > 8 ? pages / 16 : 8;
    if (splits > most) splits = most;
    if (splits > pages) splits = pages;
    if (splits < dd_ceil_div(pages, MAX_BLOCK_PAGES)) splits = dd_ceil_div(pages, MAX_BLOCK_PAGES);
    return splits < 1 ? 1 : splits;
}

// The arguments of dd_attention_decode (attention_decode.cu); max_blocks / n_splits may not exceed 128 pages.
DD_API int dd_attention_decode_pages(const void* q, int q_stride, const void* k_new, const void* v_new, void* cache,
                                     const int* tok_entry, const int* tok_pos, const int* block_table, int max_blocks,
                                     void* out, int out_stride, float* part_o, float* part_ml, int* counters, int n_tokens,
                                     int n_heads, int n_kv_heads, int head_dim, int page_size, int n_pages, int window,
                                     float scale, int n_splits, int* error_flag, void* stream) {
    if (n_tokens <= 0) return 0;
    if (!dd_attention_decode_pages_supported(n_heads, n_kv_heads, head_dim, page_size, DD_BF16))
        return dd_fail("dd_attention_decode_pages: needs heads == key/value heads, head size 64 and pages of 16, 32, 64 or 128 "
                       "tokens (got %d, %d, %d, %d)", n_heads, n_kv_heads, head_dim, page_size);
    if (n_splits < 1 || n_splits > 65535 || (n_splits > 1 && (!part_o || !part_ml || !counters)))
        return dd_fail("dd_attention_decode_pages: n_splits=%d needs scratch and counters", n_splits);
    if (dd_ceil_div(max_blocks, n_splits) > MAX_BLOCK_PAGES)
        return dd_fail("dd_attention_decode_pages: %d pages in %d splits are more than %d pages per block", max_blocks, n_splits, MAX_BLOCK_PAGES);
    if (q_stride % 8 || out_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)cache & 15) || ((uintptr_t)out & 3))
        return dd_fail("dd_attention_decode_pages: rows must be 16-byte aligned");
    if (n_tokens > 65535) return dd_fail("dd_attention_decode_pages: too many tokens");
    if ((k_new == nullptr) != (v_new == nullptr) || ((uintptr_t)k_new & 15) || ((uintptr_t)v_new & 15))
        return dd_fail("dd_attention_decode_pages: k_new and v_new come together, 16-byte aligned");
    EncodeTiled enc = encode_fn();
    if (!enc) return dd_fail("dd_attention_decode_pages: cuTensorMapEncodeTiled is not available from this driver");
    Params p;
    int n_groups = 0;
    grouping(n_heads, page_size, &p.G, &n_groups);
    const int box_rows = p.G * page_size, box_bytes = box_rows * 128;
    p.stages = (106 * 1024) / (2 * box_bytes);            // two blocks per SM
    int blocks_per_sm = 2;
    if (p.stages < 2) {                                               // large pages: one block per SM
        p.stages = (210 * 1024) / (2 * box_bytes);
        blocks_per_sm = 1;
    }
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 148;
    }
    p.inv_block_budget = 1.0f / (float)(blocks_per_sm * sm_count);
    p.deal = (long long)n_tokens * n_groups * n_splits > (long long)blocks_per_sm * sm_count;
    p.log2_P = page_size == 16 ? 4 : (page_size == 32 ? 5 : (page_size == 64 ? 6 : 7));
    if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
    if (p.stages < 2) return dd_fail("dd_attention_decode_pages: a page of %d heads x %d tokens does not fit twice into shared memory", p.G, page_size);
    const int smem = p.stages * 2 * box_bytes + 1024 + MAX_STAGES * 8 + MAX_BLOCK_PAGES * 4;
    static int configured = 0;
    if (configured < smem) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_pages_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return dd_fail("dd_attention_decode_pages: shared memory of %d bytes refused: %s", smem, cudaGetErrorString(e));
        configured = smem;
    }
    CUtensorMap map;
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)n_pages * 2 * n_heads * page_size};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {(cuuint32_t)D, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, cache, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return dd_fail("dd_attention_decode_pages: cannot describe the cache to TMA (driver error %d)", (int)r);
    p.q = (const __nv_bfloat16*)q; p.k_new = (const __nv_bfloat16*)k_new; p.v_new = (const __nv_bfloat16*)v_new;
    p.cache = (__nv_bfloat16*)cache; p.tok_entry = tok_entry; p.tok_pos = tok_pos; p.block_table = block_table;
    p.out = (__nv_bfloat16*)out; p.part_o = part_o; p.part_ml = part_ml; p.counters = counters; p.error_flag = error_flag;
    p.q_stride = q_stride; p.out_stride = out_stride; p.max_blocks = max_blocks; p.H = n_heads; p.P = page_size;
    p.n_pages = n_pages; p.window = window; p.scale_log2e = scale * 1.4426950408889634f;
    p.n_tokens = n_tokens;
    dd_launch(attention_decode_pages_kernel, dim3(n_tokens, n_groups, n_splits), dim3(THREADS), (size_t)smem, (cudaStream_t)stream, map, p);
    return dd_check_launch("dd_attention_decode_pages");
}
