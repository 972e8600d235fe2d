// Decode attention for bfloat16 caches: one query token per (token, head), keys cut into splits so
// that a small batch still fills the GPU, the split results merged by the block that finishes last.
//
// A block of 4 warps owns (split, head, token). A key row of D bf16 is read by D/8 neighbouring
// lanes, 16 bytes each, so one load instruction of a warp fetches 32/(D/8) consecutive keys (512
// contiguous bytes of a page); eight such loads of K and eight of V are in flight per lane before
// anything is consumed. Scores, running maximum, sum and the weighted value sum are float32 in the
// base-2 domain (q is pre-multiplied by scale * log2 e), as in the general kernel
// (attention_rows.cu), which remains the reference for every size this one does not take
// (grouped heads, head sizes other than 64 and 128, float32 caches).
#include "common.cuh"
#include <math_constants.h>

namespace {
constexpr int WARPS = 4;
constexpr int STEPS = 8;            // loads of K (and of V) in flight per lane

__device__ __forceinline__ void unpack8(const uint4& v, float* out) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <int D>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ cache,
                        const int* __restrict__ tok_entry, const int* __restrict__ tok_pos,
                        const int* __restrict__ block_table, int max_blocks, __nv_bfloat16* __restrict__ out,
                        int out_stride, float* __restrict__ part_o, float* __restrict__ part_ml,
                        int* __restrict__ counters, int H, int P, int n_pages, int window, float scale_log2e,
                        int* __restrict__ error_flag) {
    constexpr int C = D / 8;            // lanes per key row
    constexpr int KPL = 32 / C;         // keys per load instruction of a warp
    constexpr int TILE = KPL * STEPS;   // keys per warp iteration
    __shared__ float sh_o[WARPS][D];
    __shared__ float sh_ml[WARPS][2];
    __shared__ int sh_last;
    dd_launch_dependents();
    dd_grid_wait();

    const int split = blockIdx.x, n_splits = gridDim.x, h = blockIdx.y, t = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = lane % C, kg = lane / C;
    const int pos = tok_pos[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int hi = pos + 1;
    int per = (hi - lo + n_splits - 1) / n_splits;
    per = (per + TILE - 1) / TILE * TILE;
    const int k0 = lo + split * per;
    const int k1 = min(hi, k0 + per);

    float qv[8];
    {
        const uint4 raw = *reinterpret_cast<const uint4*>(q + (size_t)t * q_stride + (size_t)h * D + c * 8);
        unpack8(raw, qv);
#pragma unroll
        for (int i = 0; i < 8; ++i) qv[i] *= scale_log2e;
    }
    const int* bt = block_table + (size_t)tok_entry[t] * max_blocks;
    const size_t head_plane = (size_t)P * D;
    const size_t page_stride = 2 * (size_t)H * head_plane;       // key/value heads = heads here
    const __nv_bfloat16* k_base = cache + (size_t)h * head_plane + c * 8;
    const __nv_bfloat16* v_base = k_base + (size_t)H * head_plane;

    float m = -CUDART_INF_F, l = 0.f, o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = 0.f;

    for (int base = k0 + warp * TILE; base < k1; base += WARPS * TILE) {
        uint4 kr[STEPS], vr[STEPS];
        bool valid[STEPS];
#pragma unroll
        for (int i = 0; i < STEPS; ++i) {
            const int key = base + i * KPL + kg;
            valid[i] = key < k1;
            kr[i] = make_uint4(0, 0, 0, 0);
            vr[i] = make_uint4(0, 0, 0, 0);
            if (valid[i]) {
                const int blk = key / P;
                const int page = blk < max_blocks ? bt[blk] : -1;
                if (page < 0 || page >= n_pages) {
                    atomicOr(error_flag, 4);
                    valid[i] = false;
                } else {
                    const size_t off = (size_t)page * page_stride + (size_t)(key % P) * D;
                    kr[i] = *reinterpret_cast<const uint4*>(k_base + off);
                    vr[i] = *reinterpret_cast<const uint4*>(v_base + off);
                }
            }
        }
        float s[STEPS];
        float tile_max = -CUDART_INF_F;
#pragma unroll
        for (int i = 0; i < STEPS; ++i) {
            float kf[8];
            unpack8(kr[i], kf);
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc = fmaf(qv[j], kf[j], acc);
#pragma unroll
            for (int off = 1; off < C; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            s[i] = valid[i] ? acc : -CUDART_INF_F;
            tile_max = fmaxf(tile_max, s[i]);
        }
#pragma unroll
        for (int off = C; off < 32; off <<= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, off));
        if (tile_max == -CUDART_INF_F) continue;
        const float m_new = fmaxf(m, tile_max);
        const float corr = exp2f(m - m_new);
        l *= corr;
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] *= corr;
        m = m_new;
#pragma unroll
        for (int i = 0; i < STEPS; ++i) {
            const float p = exp2f(s[i] - m_new);       // 0 for masked keys
            l += p;
            float vf[8];
            unpack8(vr[i], vf);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = fmaf(p, vf[j], o[j]);
        }
    }
    // lanes with the same c hold different keys: add them up (l is the same in the C lanes of a key)
#pragma unroll
    for (int off = C; off < 32; off <<= 1) {
        l += __shfl_xor_sync(0xffffffffu, l, off);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += __shfl_xor_sync(0xffffffffu, o[j], off);
    }
    if (kg == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) sh_o[warp][c * 8 + j] = o[j];
        if (c == 0) { sh_ml[warp][0] = m; sh_ml[warp][1] = l; }
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
    const size_t first = ((size_t)t * H + h) * n_splits;
    float Mx = -CUDART_INF_F;
    for (int sp = 0; sp < n_splits; ++sp) Mx = fmaxf(Mx, __ldcg(part_ml + 2 * (first + sp)));
    float Lx = 0.f;
    for (int sp = 0; sp < n_splits; ++sp) {
        const float ls = __ldcg(part_ml + 2 * (first + sp) + 1);
        if (ls > 0.f) Lx += ls * exp2f(__ldcg(part_ml + 2 * (first + sp)) - Mx);
    }
    for (int d = threadIdx.x; d < D; d += WARPS * 32) {
        float acc = 0.f;
        for (int sp = 0; sp < n_splits; ++sp) {
            const float ls = __ldcg(part_ml + 2 * (first + sp) + 1);
            if (ls > 0.f) acc += __ldcg(part_o + (first + sp) * D + d) * exp2f(__ldcg(part_ml + 2 * (first + sp)) - Mx);
        }
        out[(size_t)t * out_stride + (size_t)h * D + d] = __float2bfloat16_rn(Lx > 0.f ? acc / Lx : 0.f);
    }
    if (threadIdx.x == 0) counters[t * H + h] = 0;
}
}  // namespace

// Returns 1 if dd_attention_decode takes this problem, else 0 (use dd_attention_rows).
DD_API int dd_attention_decode_supported(int n_heads, int n_kv_heads, int head_dim, int dtype) {
    return dtype == DD_BF16 && n_heads == n_kv_heads && (head_dim == 64 || head_dim == 128);
}

// One query per token. q/out: rows of q_stride/out_stride bf16, head h at h*head_dim. part_o: float32
// [n_tokens*heads*n_splits*head_dim], part_ml: float32 [n_tokens*heads*n_splits*2], counters: int32
// [n_tokens*heads], zero before the first launch (the kernel leaves them zero); all three only when n_splits > 1.
DD_API int dd_attention_decode(const void* q, int q_stride, const void* cache, const int* tok_entry, const int* tok_pos,
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
    dim3 grid(n_splits, n_heads, n_tokens);
    const float scale_log2e = scale * 1.4426950408889634f;
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 64)
        dd_launch(attention_decode_kernel<64>, dim3(grid), dim3(WARPS * 32), 0, s, (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)cache,
            tok_entry, tok_pos, block_table, max_blocks, (__nv_bfloat16*)out, out_stride, part_o, part_ml, counters,
            n_heads, page_size, n_pages, window, scale_log2e, error_flag);
    else
        dd_launch(attention_decode_kernel<128>, dim3(grid), dim3(WARPS * 32), 0, s, (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)cache,
            tok_entry, tok_pos, block_table, max_blocks, (__nv_bfloat16*)out, out_stride, part_o, part_ml, counters,
            n_heads, page_size, n_pages, window, scale_log2e, error_flag);
    return dd_check_launch("dd_attention_decode");
}
