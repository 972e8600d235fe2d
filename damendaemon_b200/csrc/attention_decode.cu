// Decode attention for bfloat16 caches: one query token per (token, head), keys cut into splits so
// that a small batch still fills the GPU, the split results merged by the block that finishes last.
//
// A block of 4 warps owns (split, head, token). A key row of D bf16 is fetched by D/8 neighbouring
// lanes, 16 bytes each, so one copy instruction of a warp moves 32/(D/8) consecutive keys (512
// contiguous bytes of a page). Every warp runs its own ring of cp.async stages in shared memory
// (16 keys of K and V per stage, three stages deep: 48 KB per block, so four blocks and their 16
// warps share an SM; with fewer, larger stages the arithmetic's dependency chains were left
// uncovered and the kernel ran at two thirds of this speed); a lane reads back exactly the chunks
// it copied itself, which needs no synchronisation beyond cp.async.wait_group. Scores, running maximum, sum and the
// weighted value sum are float32 in the base-2 domain (q is pre-multiplied by scale * log2 e).
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
constexpr int STEPS = 4;            // copy instructions of K (and of V) per lane and stage
constexpr int STAGES = 3;           // ring depth per warp

__device__ __forceinline__ void unpack8(const uint4& v, float* out) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int D>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* k_new,
                        const __nv_bfloat16* v_new, __nv_bfloat16* cache,
                        const int* __restrict__ tok_entry, const int* __restrict__ tok_pos,
                        const int* __restrict__ block_table, int max_blocks, __nv_bfloat16* __restrict__ out,
                        int out_stride, float* __restrict__ part_o, float* __restrict__ part_ml,
                        int* __restrict__ counters, int H, int P, int n_pages, int window, float scale_log2e,
                        int* __restrict__ error_flag) {
    constexpr int C = D / 8;            // lanes per key row
    constexpr int KPL = 32 / C;         // keys per copy instruction of a warp
    constexpr int TILE = KPL * STEPS;   // keys per stage
    constexpr int STAGE_U4 = 2 * STEPS * 32;      // uint4 per stage: K then V
    extern __shared__ uint4 ring[];     // [WARPS][STAGES][STAGE_U4]
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
    const size_t k_off = (size_t)h * head_plane + c * 8;
    const size_t v_off = k_off + (size_t)H * head_plane;
    uint4* my_ring = ring + (size_t)warp * STAGES * STAGE_U4;
    unsigned valid_bits[STAGES];        // per stage: bit i = step i of this lane holds a live key

    // tiles of this warp: base = k0 + (warp + i * WARPS) * TILE
    const int first_key = k0 + warp * TILE;
    const int n_tiles = first_key < k1 ? (k1 - first_key + WARPS * TILE - 1) / (WARPS * TILE) : 0;
    auto issue = [&](int i) {
        const int stage = i % STAGES;
        uint4* dst = my_ring + stage * STAGE_U4;
        const int base = first_key + i * WARPS * TILE;
        unsigned bits = 0;
#pragma unroll
        for (int s = 0; s < STEPS; ++s) {
            const int key = base + s * KPL + kg;
            bool ok = key < k1;
            if (ok && k_new != nullptr && key == pos) {
                // this step's own key and value: from the projection's output, and into the cache
                const __nv_bfloat16* ks = k_new + (size_t)t * q_stride + (size_t)h * D + c * 8;
                const __nv_bfloat16* vs = v_new + (size_t)t * q_stride + (size_t)h * D + c * 8;
                cp_async16(dst + s * 32 + lane, ks);
                cp_async16(dst + STEPS * 32 + s * 32 + lane, vs);
                const int blk = key / P;
                const int page = blk < max_blocks ? bt[blk] : -1;
                if (page < 0 || page >= n_pages) atomicOr(error_flag, 2);
                else {
                    const size_t off = (size_t)page * page_stride + (size_t)(key % P) * D;
                    *reinterpret_cast<uint4*>(cache + off + k_off) = *reinterpret_cast<const uint4*>(ks);
                    *reinterpret_cast<uint4*>(cache + off + v_off) = *reinterpret_cast<const uint4*>(vs);
                }
                bits |= 1u << s;
                continue;
            }
            if (ok) {
                const int blk = key / P;
                const int page = blk < max_blocks ? bt[blk] : -1;
                if (page < 0 || page >= n_pages) {
                    atomicOr(error_flag, 4);
                    ok = false;
                } else {
                    const size_t off = (size_t)page * page_stride + (size_t)(key % P) * D;
                    cp_async16(dst + s * 32 + lane, cache + off + k_off);
                    cp_async16(dst + STEPS * 32 + s * 32 + lane, cache + off + v_off);
                    bits |= 1u << s;
                }
            }
            if (!ok) dst[STEPS * 32 + s * 32 + lane] = make_uint4(0, 0, 0, 0);   // a masked value must be zero, not stale
        }
        valid_bits[stage] = bits;
    };

    float m = -CUDART_INF_F, l = 0.f, o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = 0.f;
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) {
        if (i < n_tiles) issue(i);
        cp_commit();
    }
    for (int i = 0; i < n_tiles; ++i) {
        if (i + STAGES - 1 < n_tiles) issue(i + STAGES - 1);
        cp_commit();
        cp_wait<STAGES - 1>();
        const int stage = i % STAGES;
        const uint4* src = my_ring + stage * STAGE_U4;
        unsigned bits = 0;
#pragma unroll
        for (int st = 0; st < STAGES; ++st) bits = st == stage ? valid_bits[st] : bits;
        float s[STEPS];
        float tile_max = -CUDART_INF_F;
#pragma unroll
        for (int i2 = 0; i2 < STEPS; ++i2) {
            float kf[8];
            unpack8(src[i2 * 32 + lane], kf);
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc = fmaf(qv[j], kf[j], acc);
#pragma unroll
            for (int off = 1; off < C; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            s[i2] = ((bits >> i2) & 1u) ? acc : -CUDART_INF_F;
            tile_max = fmaxf(tile_max, s[i2]);
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
        for (int i2 = 0; i2 < STEPS; ++i2) {
            const float p = exp2f(s[i2] - m_new);       // 0 for masked keys
            l += p;
            float vf[8];
            unpack8(src[STEPS * 32 + i2 * 32 + lane], vf);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = fmaf(p, vf[j], o[j]);
        }
    }
    cp_wait<0>();
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
    constexpr size_t RING = (size_t)WARPS * STAGES * 2 * STEPS * 32 * sizeof(uint4);
    static bool configured = false;
    if (!configured) {
        cudaError_t e1 = cudaFuncSetAttribute(attention_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RING);
        cudaError_t e2 = cudaFuncSetAttribute(attention_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RING);
        if (e1 != cudaSuccess || e2 != cudaSuccess) return dd_fail("dd_attention_decode: shared memory of %zu bytes refused", RING);
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
