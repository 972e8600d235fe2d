// Decode attention for bfloat16 caches: one query token per (token, head), keys cut into splits so
// that a small batch still fills the GPU, the split results merged by the block that finishes last.
//
// A block of 4 warps owns (split, head, token). Every warp runs its own ring of cp.async stages in
// shared memory (16 keys of K and V per stage, three stages deep: 48 KB per block, so four blocks
// and their 16 warps share an SM). A key row of D bf16 is fetched by D/8 neighbouring lanes, 16
// bytes each, into a row-major tile whose 16-byte chunks are swizzled by the key index, so that
// ldmatrix reads it without bank conflicts. Scores and the weighted value sum run on the tensor
// cores (mma.sync m16n8k16, float32 accumulate) with the single query in row 0 of the 16-row
// operand: fifteen rows are idle, but a 16-key stage costs about 55 warp instructions instead of the
// 175 that unpacking bf16 and scalar FMAs cost, and it is instruction issue, not tensor throughput,
// that limits this kernel beside the memory system. Running maximum, sum and the softmax are
// float32 in the base-2 domain.
//
// With k_new/v_new given, the step's own key and value (position = the token's position) are taken
// from there instead of the cache and written to the cache page by the one warp that meets them:
// the separate cache-write kernel is not needed on a decode step.
//
// The general kernel (attention_rows.cu) remains the reference for every size this one does not
// take (grouped heads, head sizes other than 64 and 128, float32 caches).
#include "common.cuh"
#include <math_constants.h>

namespace {
constexpr int WARPS = 4;
constexpr int TILE = 16;            // keys per stage (one k-step of the P.V product)
constexpr int STAGES = 3;           // ring depth per warp

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t* r) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t* r) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// byte offset of 16-byte chunk c of key row r in a [16][D] tile, chunks swizzled by the row
template <int D> __device__ __forceinline__ uint32_t tile_off(int r, int c) {
    return (uint32_t)(r * D * 2 + ((c ^ (r & 7)) << 4));
}

// Debugging aid (dd_attention_decode_stamps): 16 time stamps (ns) per block, written by its first thread: 0 start,
// 1 inputs ready, 2 first copies issued, 3.. the first eight tiles begin, 11 last tile done, 12 block's result
// written, 13 splits merged (only in the block that merges).
__device__ unsigned long long* g_stamps = nullptr;
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define STAMP(i)                                                                                                      \
    do {                                                                                                              \
        if (g_stamps && threadIdx.x == 0)                                                                             \
            g_stamps[(((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 + (i)] = now_ns(); \
    } while (0)

template <int D>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* k_new,
                        const __nv_bfloat16* v_new, __nv_bfloat16* cache,
                        const int* __restrict__ tok_entry, const int* __restrict__ tok_pos,
                        const int* __restrict__ block_table, int max_blocks, __nv_bfloat16* __restrict__ out,
                        int out_stride, float* __restrict__ part_o, float* __restrict__ part_ml,
                        int* __restrict__ counters, int H, int P, int n_pages, int window, float scale_log2e,
                        int* __restrict__ error_flag) {
    constexpr int C = D / 8;            // 16-byte chunks (and lanes) per key row
    constexpr int KPL = 32 / C;         // keys per copy instruction of a warp
    constexpr int STEPS = TILE / KPL;   // copy instructions of K (and of V) per lane and stage
    constexpr int KS = D / 16;          // k-steps of q.k over the head dimension
    constexpr int TILE_BYTES = TILE * D * 2;
    extern __shared__ __align__(128) uint8_t ring[];     // [WARPS][STAGES][K tile, V tile]
    __shared__ float sh_o[WARPS][D];
    __shared__ float sh_ml[WARPS][2];
    __shared__ int sh_last;
    STAMP(0);
    dd_launch_dependents();

    // Positions, entries and the block table are this step's inputs, not an earlier kernel's results: they are read,
    // and the table lines of this block's keys brought into L1, while the kernel before this one is still running.
    const int split = blockIdx.x, n_splits = gridDim.x, h = blockIdx.y, t = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = lane % C, kg = lane / C;
    const int g = lane >> 2, t4 = lane & 3;
    const int pos = tok_pos[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int hi = pos + 1;
    int per = (hi - lo + n_splits - 1) / n_splits;
    per = (per + TILE - 1) / TILE * TILE;
    const int k0 = lo + split * per;
    const int k1 = min(hi, k0 + per);
    const int* bt = block_table + (size_t)(tok_entry ? tok_entry[t] : t) * max_blocks;     // no tok_entry: token t is entry t
    for (int blk = k0 / P + (int)threadIdx.x * 32; blk < max_blocks && blk * P < k1 + 32 * P; blk += WARPS * 32 * 32)
        asm volatile("prefetch.global.L1 [%0];" ::"l"(bt + min(blk, max_blocks - 1)));
    const size_t head_plane = (size_t)P * D;
    const size_t page_stride = 2 * (size_t)H * head_plane;       // key/value heads = heads here
    const size_t k_off = (size_t)h * head_plane + c * 8;
    const size_t v_off = k_off + (size_t)H * head_plane;
    uint8_t* my_ring = ring + (size_t)warp * STAGES * 2 * TILE_BYTES;

    // tiles of this warp: base = k0 + (warp + i * WARPS) * TILE
    const int first_key = k0 + warp * TILE;
    const int n_tiles = first_key < k1 ? (k1 - first_key + WARPS * TILE - 1) / (WARPS * TILE) : 0;
    // The cache pages of the rows this lane copies in tile i, looked up apart from the copies: the copies are
    // ordered (asm volatile), and with a table read in front of each, a tile cost four trips to L2 in a row,
    // about 1 us, which bounded the whole kernel. The next tile's pages are requested a tile ahead.
    auto lookup = [&](int i, int* pages) {
        const int base = first_key + i * WARPS * TILE;
#pragma unroll
        for (int s = 0; s < STEPS; ++s) {
            const int key = base + s * KPL + kg;
            const int blk = key / P;
            pages[s] = (key < k1 && blk < max_blocks) ? bt[blk] : -1;
        }
    };
    auto issue = [&](int i, const int* pages) {
        uint8_t* kt = my_ring + (i % STAGES) * 2 * TILE_BYTES;
        uint8_t* vt = kt + TILE_BYTES;
        const int base = first_key + i * WARPS * TILE;
#pragma unroll
        for (int s = 0; s < STEPS; ++s) {
            const int row = s * KPL + kg;
            const int key = base + row;
            const uint32_t off = tile_off<D>(row, c);
            const int page = pages[s];
            bool ok = key < k1;
            if (ok && (page < 0 || page >= n_pages)) {
                atomicOr(error_flag, k_new != nullptr && key == pos ? 2 : 4);
                ok = false;
            }
            if (ok && k_new != nullptr && key == pos) {
                // this step's own key and value: from the projection's output, and into the cache
                const __nv_bfloat16* ks = k_new + (size_t)t * q_stride + (size_t)h * D + c * 8;
                const __nv_bfloat16* vs = v_new + (size_t)t * q_stride + (size_t)h * D + c * 8;
                cp_async16(kt + off, ks);
                cp_async16(vt + off, vs);
                const size_t dst = (size_t)page * page_stride + (size_t)(key % P) * D;
                *reinterpret_cast<uint4*>(cache + dst + k_off) = *reinterpret_cast<const uint4*>(ks);
                *reinterpret_cast<uint4*>(cache + dst + v_off) = *reinterpret_cast<const uint4*>(vs);
                continue;
            }
            if (ok) {
                const size_t src = (size_t)page * page_stride + (size_t)(key % P) * D;
                cp_async16(kt + off, cache + src + k_off);
                cp_async16(vt + off, cache + src + v_off);
            } else {            // keys beyond the range are masked by their index; their rows must still be finite
                *reinterpret_cast<uint4*>(kt + off) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vt + off) = make_uint4(0, 0, 0, 0);
            }
        }
    };

    float m = -CUDART_INF_F, l = 0.f, o[C][4];
#pragma unroll
    for (int i = 0; i < C; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    int pages[STAGES][STEPS];          // of the tiles about to be issued; the loop below is unrolled over its slots
#pragma unroll
    for (int i = 0; i < STAGES; ++i) lookup(i, pages[i]);
    // The first tiles are requested while the projection that produces the query is still running: with k_new/v_new
    // given, everything before the token's own position was written by earlier steps. Only the tile with that position
    // takes its row from k_new/v_new and has to wait, and with it every tile after it (copy groups complete in order).
    // Without k_new/v_new the row of this step is in the cache already, written by some kernel of this step: then
    // nothing is read before the wait.
    int issued = 0;
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) {
        const bool early = issued == i && k_new != nullptr && first_key + i * WARPS * TILE + TILE <= pos;
        if (early) {
            if (i < n_tiles) issue(i, pages[i]);
            cp_commit();
            issued = i + 1;
        }
    }
    dd_grid_wait();
    STAMP(1);

    // the query as the A operand: row 0 of a 16-row tile, every other row zero
    uint32_t qf[KS][4];
    {
        const __nv_bfloat16* qp = q + (size_t)t * q_stride + (size_t)h * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qf[ks][0] = g == 0 ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 2 * t4) : 0u;
            qf[ks][1] = 0u;
            qf[ks][2] = g == 0 ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8 + 2 * t4) : 0u;
            qf[ks][3] = 0u;
        }
    }
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) {
        if (i < issued) continue;
        if (i < n_tiles) issue(i, pages[i]);
        cp_commit();
    }
    STAMP(2);
    for (int i = 0; i < n_tiles; ++i) {
        if (i < 8) STAMP(3 + i);
        if (i + STAGES - 1 < n_tiles) issue(i + STAGES - 1, pages[STAGES - 1]);
        // slide: the next tile to issue is i + STAGES, its pages come while this tile is computed
#pragma unroll
        for (int s = 0; s < STEPS; ++s) pages[STAGES - 1][s] = -1;
        if (i + STAGES < n_tiles) lookup(i + STAGES, pages[STAGES - 1]);
        cp_commit();
        cp_wait<STAGES - 1>();
        __syncwarp();                                   // other lanes' copies and zero fills are visible
        const uint8_t* kt = my_ring + (i % STAGES) * 2 * TILE_BYTES;
        const uint8_t* vt = kt + TILE_BYTES;
        const int base = first_key + i * WARPS * TILE;
        // scores of 16 keys against the query (row 0)
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
        const int mi = lane >> 3;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t b[4];
            ldmatrix_x4(smem_addr(kt + tile_off<D>((mi >> 1) * 8 + (lane & 7), 2 * ks + (mi & 1))), b);
            mma_bf16(s[0], qf[ks], b[0], b[1]);
            mma_bf16(s[1], qf[ks], b[2], b[3]);
        }
        // row 0 lives in lanes 0..3 (elements 0 and 1 of each 8-key tile); the other rows are idle
        float mx = -CUDART_INF_F;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = base + nt * 8 + 2 * t4 + e;
                const float v = key < k1 ? s[nt][e] * scale_log2e : -CUDART_INF_F;
                s[nt][e] = v;
                mx = fmaxf(mx, v);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m, mx);               // every tile holds at least one live key
        const float corr = exp2f(m - m_new);
        m = m_new;
        l *= corr;
        uint32_t pf[4];
        {
            const float p00 = exp2f(s[0][0] - m_new), p01 = exp2f(s[0][1] - m_new);
            const float p10 = exp2f(s[1][0] - m_new), p11 = exp2f(s[1][1] - m_new);
            l += (p00 + p01) + (p10 + p11);
            pf[0] = g == 0 ? pack_bf16(p00, p01) : 0u;
            pf[1] = 0u;
            pf[2] = g == 0 ? pack_bf16(p10, p11) : 0u;
            pf[3] = 0u;
        }
#pragma unroll
        for (int j = 0; j < C; ++j) { o[j][0] *= corr; o[j][1] *= corr; }
#pragma unroll
        for (int dp = 0; dp < C / 2; ++dp) {
            uint32_t b[4];
            ldmatrix_x4_trans(smem_addr(vt + tile_off<D>((mi & 1) * 8 + (lane & 7), 2 * dp + (mi >> 1))), b);
            mma_bf16(o[2 * dp], pf, b[0], b[1]);
            mma_bf16(o[2 * dp + 1], pf, b[2], b[3]);
        }
        __syncwarp();                                   // the stage may be refilled
    }
    cp_wait<0>();
    STAMP(11);
    // row 0: lanes 0..3 hold dims 8j + 2*t4 + {0,1}; their sums of l differ by the keys each saw
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (g == 0) {
#pragma unroll
        for (int j = 0; j < C; ++j) {
            sh_o[warp][j * 8 + 2 * t4] = o[j][0];
            sh_o[warp][j * 8 + 2 * t4 + 1] = o[j][1];
        }
        if (t4 == 0) { sh_ml[warp][0] = m; sh_ml[warp][1] = l; }
    }
    __syncthreads();
    // combine the warps: thread d owns output dimension d
    const size_t item = ((size_t)t * H + h) * n_splits + split;
    float M = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, sh_ml[w][0]);
    float L = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) L += sh_ml[w][1] > 0.f ? sh_ml[w][1] * exp2f(sh_ml[w][0] - M) : 0.f;
    for (int d = threadIdx.x; d < D; d += WARPS * 32) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) acc += sh_ml[w][1] > 0.f ? sh_o[w][d] * exp2f(sh_ml[w][0] - M) : 0.f;
        if (n_splits == 1) out[(size_t)t * out_stride + (size_t)h * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        else part_o[item * D + d] = acc;
    }
    STAMP(12);
    if (n_splits == 1) return;
    if (threadIdx.x == 0) { part_ml[2 * item] = M; part_ml[2 * item + 1] = L; }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int prev = atomicAdd(&counters[t * H + h], 1);
        sh_last = prev == n_splits - 1;
    }
    __syncthreads();
    if (!sh_last) return;
    __threadfence();
    // Thread d merges output dimension d. The partial maxima, sums and outputs of eight splits are requested
    // together and merged with a running maximum, so the tail costs one trip to L2 per eight splits.
    const size_t first = ((size_t)t * H + h) * n_splits;
    for (int d = threadIdx.x; d < D; d += WARPS * 32) {
        float Mx = -CUDART_INF_F, Lx = 0.f, acc = 0.f;
        for (int sp0 = 0; sp0 < n_splits; sp0 += 8) {
            float mm[8], ll[8], oo[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const bool live = sp0 + u < n_splits;
                const size_t it = first + sp0 + (live ? u : 0);
                mm[u] = live ? __ldcg(part_ml + 2 * it) : -CUDART_INF_F;
                ll[u] = live ? __ldcg(part_ml + 2 * it + 1) : 0.f;
                oo[u] = live ? __ldcg(part_o + it * D + d) : 0.f;
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
        out[(size_t)t * out_stride + (size_t)h * D + d] = __float2bfloat16_rn(Lx > 0.f ? acc / Lx : 0.f);
    }
    if (threadIdx.x == 0) counters[t * H + h] = 0;
    STAMP(13);
}
}  // namespace

// A device buffer of 16 stamps per block of the following launches; null switches the stamps off.
DD_API void dd_attention_decode_stamps(unsigned long long* buffer) { cudaMemcpyToSymbol(g_stamps, &buffer, sizeof(buffer)); }

// Returns 1 if dd_attention_decode takes this problem, else 0 (use dd_attention_rows).
DD_API int dd_attention_decode_supported(int n_heads, int n_kv_heads, int head_dim, int dtype) {
    return dtype == DD_BF16 && n_heads == n_kv_heads && (head_dim == 64 || head_dim == 128);
}

// One query per token. q/out: rows of q_stride/out_stride bf16, head h at h*head_dim. k_new/v_new: null, or
// this step's keys and values as rows of q_stride bf16 (the fused projection's output), which are then
// used for each token's own position and written to the cache here. part_o: float32
// [n_tokens*heads*n_splits*head_dim], part_ml: float32 [n_tokens*heads*n_splits*2], counters: int32
// [n_tokens*heads], zero before the first launch (the kernel leaves them zero); all three only when n_splits > 1.
DD_API int dd_attention_decode(const void* q, int q_stride, const void* k_new, const void* v_new, void* cache,
                               const int* tok_entry, const int* tok_pos,
                               const int* block_table, int max_blocks, void* out, int out_stride, float* part_o,
                               float* part_ml, int* counters, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                               int page_size, int n_pages, int window, float scale, int n_splits, int* error_flag,
                               void* stream) {
    if (n_tokens <= 0) return 0;
    if (!dd_attention_decode_supported(n_heads, n_kv_heads, head_dim, DD_BF16))
        return dd_fail("dd_attention_decode: needs heads == key/value heads and head size 64 or 128 (got %d, %d, %d)",
                       n_heads, n_kv_heads, head_dim);
    if (n_splits < 1 || n_splits > 65535 || (n_splits > 1 && (!part_o || !part_ml || !counters)))
        return dd_fail("dd_attention_decode: n_splits=%d needs scratch and counters", n_splits);
    if (q_stride % 8 || out_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)cache & 15))
        return dd_fail("dd_attention_decode: rows must be 16-byte aligned");
    if (n_heads > 65535 || n_tokens > 65535) return dd_fail("dd_attention_decode: too many heads or tokens");
    if ((k_new == nullptr) != (v_new == nullptr) || ((uintptr_t)k_new & 15) || ((uintptr_t)v_new & 15))
        return dd_fail("dd_attention_decode: k_new and v_new come together, 16-byte aligned");
    dim3 grid(n_splits, n_heads, n_tokens);
    const float scale_log2e = scale * 1.4426950408889634f;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t RING = (size_t)WARPS * STAGES * 2 * TILE * head_dim * 2;
    static bool configured = false;
    if (!configured) {
        const int ring64 = WARPS * STAGES * 2 * TILE * 64 * 2, ring128 = WARPS * STAGES * 2 * TILE * 128 * 2;
        cudaError_t e1 = cudaFuncSetAttribute(attention_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, ring64);
        cudaError_t e2 = cudaFuncSetAttribute(attention_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, ring128);
        if (e1 != cudaSuccess || e2 != cudaSuccess) return dd_fail("dd_attention_decode: shared memory of %d bytes refused", ring128);
        configured = true;
    }
    if (head_dim == 64)
        dd_launch(attention_decode_kernel<64>, dim3(grid), dim3(WARPS * 32), RING, s, (const __nv_bfloat16*)q, q_stride,
            (const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new, (__nv_bfloat16*)cache,
            tok_entry, tok_pos, block_table, max_blocks, (__nv_bfloat16*)out, out_stride, part_o, part_ml, counters,
            n_heads, page_size, n_pages, window, scale_log2e, error_flag);
    else
        dd_launch(attention_decode_kernel<128>, dim3(grid), dim3(WARPS * 32), RING, s, (const __nv_bfloat16*)q, q_stride,
            (const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new, (__nv_bfloat16*)cache,
            tok_entry, tok_pos, block_table, max_blocks, (__nv_bfloat16*)out, out_stride, part_o, part_ml, counters,
            n_heads, page_size, n_pages, window, scale_log2e, error_flag);
    return dd_check_launch("dd_attention_decode");
}
