// Prompt-portion attention for bfloat16 caches on the tensor cores (mma.sync m16n8k16,
// float32 accumulate): a block of 4 warps owns 64 consecutive query tokens of one request and
// one head, walks the request's keys in tiles of 64 straight out of the cache pages (cp.async,
// double buffered, 16-byte-chunk swizzle in shared memory) and keeps a running maximum and sum
// per query row, so earlier portions of the prompt are read exactly like this step's tokens.
// Scores, softmax and the weighted value sum are float32 (damendaemon/kernels.py:147-178 for the
// mask and the stable softmax; damendaemon/qwen2.py:754-770 for the offset-aware causal rule).
// Takes head sizes 64 and 128 with any number of heads and key/value groups; the general
// kernel (attention_rows.cu) serves every other size and is its reference in the tests.
#include "common.cuh"
#include <math_constants.h>

namespace {
constexpr int BQ = 64, BKV = 64, THREADS = 128;

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
// byte offset of 16-byte chunk c of row r in a tile whose rows are D bf16, chunks swizzled by the row
template <int D> __device__ __forceinline__ uint32_t tile_off(int r, int c) {
    return (uint32_t)(r * D * 2 + ((c ^ (r & 7)) << 4));
}

template <int D>
__global__ void __launch_bounds__(THREADS)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ cache,
                         const int* __restrict__ entry_start, const int* __restrict__ entry_pos0, int n_entries,
                         const int* __restrict__ block_table, int max_blocks, __nv_bfloat16* __restrict__ out,
                         int out_stride, int H, int KH, int P, int n_pages, int window, float scale_log2e,
                         int* __restrict__ error_flag) {
    constexpr int NC = D / 8;                 // 16-byte chunks per row
    constexpr int KS = D / 16;                // k-steps over the head dimension
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + BQ * D * 2;            // [2][BKV][D]
    uint8_t* sV = sK + 2 * BKV * D * 2;       // [2][BKV][D]
    dd_launch_dependents();
    dd_grid_wait();

    // which 64-row tile of which entry is this block's?
    int e = 0, tile = blockIdx.x, len = 0;
    for (; e < n_entries; ++e) {
        len = entry_start[e + 1] - entry_start[e];
        const int nt = (len + BQ - 1) / BQ;
        if (tile < nt) break;
        tile -= nt;
    }
    if (e == n_entries) return;
    const int h = blockIdx.y, kh = h / (H / KH);
    const int q0 = tile * BQ;
    const int rows = min(BQ, len - q0);
    const int row0 = entry_start[e] + q0;
    const int pos_first = entry_pos0[e] + q0, pos_last = pos_first + rows - 1;
    const int kv_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int* bt = block_table + (size_t)e * max_blocks;
    const size_t head_plane = (size_t)P * D, page_stride = 2 * (size_t)KH * head_plane;
    const __nv_bfloat16* k_base = cache + (size_t)kh * head_plane;
    const __nv_bfloat16* v_base = k_base + (size_t)KH * head_plane;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;

    // Q tile -> shared memory (rows beyond the tile are zero)
    for (int idx = tid; idx < BQ * NC; idx += THREADS) {
        const int r = idx / NC, c = idx % NC;
        uint8_t* dst = sQ + tile_off<D>(r, c);
        if (r < rows) cp_async16(dst, q + (size_t)(row0 + r) * q_stride + (size_t)h * D + c * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    auto load_kv = [&](int kb, int buf) {
        for (int idx = tid; idx < BKV * NC; idx += THREADS) {
            const int r = idx / NC, c = idx % NC;
            const int key = kb + r;
            uint8_t* dk = sK + buf * BKV * D * 2 + tile_off<D>(r, c);
            uint8_t* dv = sV + buf * BKV * D * 2 + tile_off<D>(r, c);
            int page = -1;
            if (key >= kv_lo && key <= pos_last) {
                const int blk = key / P;
                page = blk < max_blocks ? bt[blk] : -1;
                if (page < 0 || page >= n_pages) {
                    if (c == 0) atomicOr(error_flag, 4);
                    page = -1;
                }
            }
            if (page >= 0) {
                const size_t off = (size_t)page * page_stride + (size_t)(key % P) * D + c * 8;
                cp_async16(dk, k_base + off);
                cp_async16(dv, v_base + off);
            } else {                      // masked or missing keys must be zeros: 0 * stale NaN would spoil the sum
                *reinterpret_cast<uint4*>(dk) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(dv) = make_uint4(0, 0, 0, 0);
            }
        }
    };
    const int kb_first = kv_lo / BKV * BKV;
    const int n_tiles = (pos_last - kb_first) / BKV + 1;
    load_kv(kb_first, 0);
    cp_commit();

    float o[NC][4], m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < NC; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    uint32_t qf[KS][4];
    const int qpos[2] = {pos_first + warp * 16 + g, pos_first + warp * 16 + g + 8};
    int qlo[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) qlo[i] = window > 0 ? max(0, qpos[i] - window + 1) : 0;

    for (int j = 0; j < n_tiles; ++j) {
        const int kb = kb_first + j * BKV, buf = j & 1;
        if (j + 1 < n_tiles) load_kv(kb + BKV, buf ^ 1);
        cp_commit();
        cp_wait<1>();
        __syncthreads();
        if (j == 0) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int mi = lane >> 3;
                ldmatrix_x4(smem_addr(sQ + tile_off<D>(warp * 16 + (mi & 1) * 8 + (lane & 7), 2 * ks + (mi >> 1))), qf[ks]);
            }
        }
        const uint8_t* tk = sK + buf * BKV * D * 2;
        const uint8_t* tv = sV + buf * BKV * D * 2;
        // S = Q K^T for 16 query rows x 64 keys
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {             // pairs of 8-key tiles
                uint32_t b[4];
                const int mi = lane >> 3;
                ldmatrix_x4(smem_addr(tk + tile_off<D>(np * 16 + (mi >> 1) * 8 + (lane & 7), 2 * ks + (mi & 1))), b);
                mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
                mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
            }
        }
        // scale, mask, running maximum
        const bool need_mask = (kb + BKV - 1 > pos_first + warp * 16) || window > 0 || kb < kv_lo;
        float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int key = kb + nt * 8 + 2 * t4 + (i & 1);
                const int r = i >> 1;
                float v = s[nt][i] * scale_log2e;
                if (need_mask && (key > qpos[r] || key < qlo[r])) v = -CUDART_INF_F;
                s[nt][i] = v;
                mx[r] = fmaxf(mx[r], v);
            }
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m[r], mx[r]);
            corr[r] = m_new == -CUDART_INF_F ? 1.f : exp2f(m[r] - m_new);
            m[r] = m_new;
            l[r] *= corr[r];
        }
        const float msub[2] = {m[0] == -CUDART_INF_F ? 0.f : m[0], m[1] == -CUDART_INF_F ? 0.f : m[1]};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float p = exp2f(s[nt][i] - msub[i >> 1]);
                s[nt][i] = p;
                l[i >> 1] += p;
            }
        }
#pragma unroll
        for (int i = 0; i < NC; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < NC / 2; ++dp) {
                uint32_t b[4];
                const int mi = lane >> 3;
                ldmatrix_x4_trans(smem_addr(tv + tile_off<D>(kk * 16 + (mi & 1) * 8 + (lane & 7), 2 * dp + (mi >> 1))), b);
                mma_bf16(o[2 * dp], a, b[0], b[1]);
                mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();       // everyone is done with this buffer before it is filled again
    }
    cp_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + g + r * 8;
        if (row >= rows) continue;
        const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
        __nv_bfloat16* dst = out + (size_t)(row0 + row) * out_stride + (size_t)h * D + 2 * t4;
#pragma unroll
        for (int i = 0; i < NC; ++i)
            *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
    }
}

template <int D>
int launch(const void* q, int q_stride, const void* cache, const int* entry_start, const int* entry_pos0, int n_entries,
           int n_tokens, const int* block_table, int max_blocks, void* out, int out_stride, int H, int KH, int P,
           int n_pages, int window, float scale, int* error_flag, cudaStream_t s) {
    constexpr int SMEM = (BQ + 4 * BKV) * D * 2;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return dd_fail("dd_attention_prefill: shared memory refused: %s", cudaGetErrorString(e));
        configured = true;
    }
    // an upper bound of the number of 64-row tiles; blocks beyond the real count return at once
    dim3 grid(dd_ceil_div(n_tokens, BQ) + n_entries, H);
    dd_launch(attention_prefill_kernel<D>, dim3(grid), dim3(THREADS), SMEM, s, (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)cache,
        entry_start, entry_pos0, n_entries, block_table, max_blocks, (__nv_bfloat16*)out, out_stride, H, KH, P, n_pages,
        window, scale * 1.4426950408889634f, error_flag);
    return dd_check_launch("dd_attention_prefill");
}
}  // namespace

DD_API int dd_attention_prefill_supported(int n_heads, int n_kv_heads, int head_dim, int dtype) {
    return dtype == DD_BF16 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 && (head_dim == 64 || head_dim == 128);
}

// Entries are runs of consecutive tokens of one request: entry e holds flattened tokens
// entry_start[e] .. entry_start[e+1]-1 at positions entry_pos0[e] ... ; block_table row e is its pages.
DD_API int dd_attention_prefill(const void* q, int q_stride, const void* cache, const int* entry_start,
                                const int* entry_pos0, int n_entries, int n_tokens, const int* block_table,
                                int max_blocks, void* out, int out_stride, int n_heads, int n_kv_heads, int head_dim,
                                int page_size, int n_pages, int window, float scale, int* error_flag, void* stream) {
    if (n_tokens <= 0 || n_entries <= 0) return 0;
    if (!dd_attention_prefill_supported(n_heads, n_kv_heads, head_dim, DD_BF16))
        return dd_fail("dd_attention_prefill: needs head size 64 or 128 and heads a multiple of key/value heads (got %d, %d, %d)",
                       n_heads, n_kv_heads, head_dim);
    if (q_stride % 8 || out_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)cache & 15) || ((uintptr_t)out & 3))
        return dd_fail("dd_attention_prefill: rows must be 16-byte aligned");
    if (n_heads > 65535) return dd_fail("dd_attention_prefill: too many heads");
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 64)
        return launch<64>(q, q_stride, cache, entry_start, entry_pos0, n_entries, n_tokens, block_table, max_blocks, out,
                          out_stride, n_heads, n_kv_heads, page_size, n_pages, window, scale, error_flag, s);
    return launch<128>(q, q_stride, cache, entry_start, entry_pos0, n_entries, n_tokens, block_table, max_blocks, out,
                       out_stride, n_heads, n_kv_heads, page_size, n_pages, window, scale, error_flag, s);
}
