// Causal attention over the paged cache, one warp per (token, head, key split).
// This is the general kernel: any number of heads and key/value groups, head sizes
// in steps of 8 up to 256, an optional window, portions of prompts and single
// decoded tokens in the same launch. Scores, the running maximum, the softmax sum
// and the weighted value sum are float32 whatever the storage type
// (damendaemon/kernels.py:133-210: scale d^-0.5, mask key <= position, exp(s - max),
// partial results merged by their log-sum-exp).
//
// Query token t at position p of entry e sees keys lo..p, lo = max(0, p - window + 1)
// with a window, else 0. Key j lives in page block_table[e][j / page_size] of the
// layer's cache [n_pages, 2, kv_heads, page_size, head_dim]. With n_splits > 1 the
// key range is cut in n_splits pieces whose (max, sum, unnormalised output) go to
// scratch and dd_attention_merge combines them.
#include "common.cuh"
#include <math_constants.h>

namespace {
constexpr int WARPS = 4;

template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
    __device__ static float exp(float x) { return expf(x); }
};
template <> struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void load(const __nv_bfloat16* p, float* out) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ static float exp(float x) { return __expf(x); }
};

template <typename T, int DPL>
__global__ void __launch_bounds__(WARPS * 32)
attention_rows_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ cache,
                      const int* __restrict__ tok_entry, const int* __restrict__ tok_pos,
                      const int* __restrict__ block_table, int max_blocks,
                      T* __restrict__ out, int out_stride, float* __restrict__ part_o, float* __restrict__ part_ml,
                      int n_tokens, int H, int KH, int d, int P, int n_pages, int window, float scale,
                      int n_splits, int* __restrict__ error_flag) {
    extern __shared__ float q_smem[];
    dd_launch_dependents();
    dd_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * H * n_splits) return;
    const int split = (int)(item % n_splits);
    const int h = (int)((item / n_splits) % H);
    const int t = (int)(item / ((long long)n_splits * H));
    const int pos = tok_pos[t];
    const int kh = h / (H / KH);
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int hi = pos + 1;
    int per = (hi - lo + n_splits - 1) / n_splits;
    per = (per + 31) / 32 * 32;
    const int k0 = lo + split * per;
    const int k1 = min(hi, k0 + per);

    float* qs = q_smem + warp * d;
    const T* qp = q + (size_t)t * q_stride + (size_t)h * d;
    for (int c = lane; c < d; c += 32) qs[c] = dd_to_f32(qp[c]) * scale;
    __syncwarp();

    const int* bt = block_table + (size_t)tok_entry[t] * max_blocks;
    const size_t head_plane = (size_t)P * d;
    float m = -CUDART_INF_F, l = 0.f, o[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) o[i] = 0.f;

    for (int base = k0; base < k1; base += 32) {
        const int key = base + lane;
        bool valid = key < k1;
        int page = 0;
        if (valid) {
            const int blk = key / P;
            page = blk < max_blocks ? bt[blk] : -1;
            if (page < 0 || page >= n_pages) {
                atomicOr(error_flag, 4);
                valid = false;
                page = 0;
            }
        }
        float sc = -CUDART_INF_F;
        if (valid) {
            const T* kp = cache + ((size_t)page * 2 * KH + kh) * head_plane + (size_t)(key % P) * d;
            float acc = 0.f;
#pragma unroll 4
            for (int c = 0; c < d; c += Vec<T>::N) {      // (unrolled: the next pieces are on their way while this one is added)
                float kv[Vec<T>::N];
                Vec<T>::load(kp + c, kv);
#pragma unroll
                for (int i = 0; i < Vec<T>::N; ++i) acc = fmaf(qs[c + i], kv[i], acc);
            }
            sc = acc;
        }
        const float cm = dd_warp_max(sc);
        if (cm == -CUDART_INF_F) continue;
        const float m_new = fmaxf(m, cm);
        const float corr = Vec<T>::exp(m - m_new);
        const float p = valid ? Vec<T>::exp(sc - m_new) : 0.f;
        l = l * corr + dd_warp_sum(p);
#pragma unroll
        for (int i = 0; i < DPL; ++i) o[i] *= corr;
        m = m_new;
        const int n_valid = min(32, k1 - base);
        // The value rows of eight keys are requested together and then added in key order (one row at a time, each
        // load waited for before the next was asked, a tile of 32 keys cost 32 trips to memory).
        for (int j0 = 0; j0 < n_valid; j0 += 8) {
            float pj[8], vv[8][DPL];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int j = min(j0 + u, n_valid - 1);     // past the last key: its row again, never added
                pj[u] = __shfl_sync(0xffffffffu, p, j);
                const int pg = __shfl_sync(0xffffffffu, page, j);
                const T* vp = cache + ((size_t)pg * 2 * KH + KH + kh) * head_plane + (size_t)((base + j) % P) * d;
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    const int c = lane + 32 * i;
                    vv[u][i] = c < d ? dd_to_f32(vp[c]) : 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (j0 + u >= n_valid) break;
#pragma unroll
                for (int i = 0; i < DPL; ++i) o[i] = fmaf(pj[u], vv[u][i], o[i]);
            }
        }
    }
    if (n_splits == 1) {
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        T* op = out + (size_t)t * out_stride + (size_t)h * d;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int c = lane + 32 * i;
            if (c < d) op[c] = dd_from_f32<T>(o[i] * inv);
        }
    } else {
        float* po = part_o + (size_t)item * d;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int c = lane + 32 * i;
            if (c < d) po[c] = o[i];
        }
        if (lane == 0) {
            part_ml[2 * item] = m;
            part_ml[2 * item + 1] = l;
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                       T* __restrict__ out, int out_stride, int n_tokens, int H, int d, int n_splits) {
    dd_launch_dependents();
    dd_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * WARPS + warp;   // (token, head)
    if (row >= (long long)n_tokens * H) return;
    const float* ml = part_ml + (size_t)row * n_splits * 2;
    const int t = (int)(row / H), h = (int)(row % H);
    T* op = out + (size_t)t * out_stride + (size_t)h * d;
    if (n_splits <= 32) {
        // Lane s fetches split s's maximum and sum; the merge then runs over the splits in order with values passed
        // between lanes, and the partial outputs of eight splits are requested together: the same additions in the same
        // order as the plain loops below, without a trip to memory for every term (14 -> 3 us for 200 rows x 9 splits).
        const float my_m = lane < n_splits ? ml[2 * lane] : -CUDART_INF_F;
        const float my_l = lane < n_splits ? ml[2 * lane + 1] : 0.f;
        float m = -CUDART_INF_F;
        for (int s = 0; s < n_splits; ++s) m = fmaxf(m, __shfl_sync(0xffffffffu, my_m, s));
        const float my_w = my_l > 0.f ? expf(my_m - m) : 0.f;
        float l = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ls = __shfl_sync(0xffffffffu, my_l, s), ws = __shfl_sync(0xffffffffu, my_w, s);
            if (ls > 0.f) l += ls * ws;
        }
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        for (int c0 = 0; c0 < d; c0 += 32) {
            const int c = c0 + lane;
            float acc = 0.f;
            for (int s0 = 0; s0 < n_splits; s0 += 8) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    v[u] = (s0 + u < n_splits && c < d) ? part_o[((size_t)row * n_splits + s0 + u) * d + c] : 0.f;
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int s = min(s0 + u, n_splits - 1);
                    const float ls = __shfl_sync(0xffffffffu, my_l, s), ws = __shfl_sync(0xffffffffu, my_w, s);
                    if (s0 + u < n_splits && ls > 0.f) acc += v[u] * ws;
                }
            }
            if (c < d) op[c] = dd_from_f32<T>(acc * inv);
        }
        return;
    }
    float m = -CUDART_INF_F;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, ml[2 * s]);
    float l = 0.f;
    for (int s = 0; s < n_splits; ++s)
        if (ml[2 * s + 1] > 0.f) l += ml[2 * s + 1] * expf(ml[2 * s] - m);
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    for (int c = lane; c < d; c += 32) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s)
            if (ml[2 * s + 1] > 0.f) acc += part_o[((size_t)row * n_splits + s) * d + c] * expf(ml[2 * s] - m);
        op[c] = dd_from_f32<T>(acc * inv);
    }
}

template <typename T>
int launch_rows(const void* q, int q_stride, const void* cache, const int* tok_entry, const int* tok_pos,
                const int* block_table, int max_blocks, void* out, int out_stride, float* part_o, float* part_ml,
                int n_tokens, int H, int KH, int d, int P, int n_pages, int window, float scale, int n_splits,
                int* error_flag, cudaStream_t s) {
    const long long items = (long long)n_tokens * H * n_splits;
    if ((items + WARPS - 1) / WARPS > 0x7fffffffLL)
        return dd_fail("dd_attention_rows: %d tokens x %d heads x %d splits are more work items than one launch takes",
                       n_tokens, H, n_splits);
    const int grid = dd_ceil_div(items, WARPS);
    const size_t smem = (size_t)WARPS * d * sizeof(float);
#define DD_ROWS(DPL)                                                                                        \
    dd_launch(attention_rows_kernel<T, DPL>, dim3(grid), dim3(WARPS * 32), smem, s, (const T*)q, q_stride, (const T*)cache,    \
        tok_entry, tok_pos, block_table, max_blocks, (T*)out, out_stride, part_o, part_ml, n_tokens, H, KH, \
        d, P, n_pages, window, scale, n_splits, error_flag)
    if (d <= 32) DD_ROWS(1);
    else if (d <= 64) DD_ROWS(2);
    else if (d <= 128) DD_ROWS(4);
    else DD_ROWS(8);
#undef DD_ROWS
    if (int e = dd_check_launch("dd_attention_rows")) return e;
    if (n_splits > 1) {
        dd_launch(attention_merge_kernel<T>, dim3(dd_ceil_div((long long)n_tokens * H, WARPS)), dim3(WARPS * 32), 0, s, 
            part_o, part_ml, (T*)out, out_stride, n_tokens, H, d, n_splits);
        return dd_check_launch("dd_attention_merge");
    }
    return 0;
}
}  // namespace

// q: [n_tokens] rows of q_stride elements, head h at offset h*head_dim. out likewise.
// part_o: float32 [n_tokens*H*n_splits*head_dim], part_ml: float32 [n_tokens*H*n_splits*2]
// (scratch, used only when n_splits > 1). error_flag bit 2 (value 4): a page index
// outside the pool was met and skipped.
DD_API int dd_attention_rows(const void* q, int q_stride, const void* cache, const int* tok_entry,
                             const int* tok_pos, const int* block_table, int max_blocks, void* out, int out_stride,
                             float* part_o, float* part_ml, int n_tokens, int n_heads, int n_kv_heads,
                             int head_dim, int page_size, int n_pages, int window, float scale, int n_splits,
                             int dtype, int* error_flag, void* stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim <= 0 || head_dim > 256 || head_dim % 8)
        return dd_fail("dd_attention_rows: head size %d is not supported (a multiple of 8, at most 256)", head_dim);
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads)
        return dd_fail("dd_attention_rows: %d heads cannot share %d key/value heads", n_heads, n_kv_heads);
    if (n_splits < 1 || (n_splits > 1 && (!part_o || !part_ml)))
        return dd_fail("dd_attention_rows: n_splits=%d needs scratch", n_splits);
    if (q_stride % 8 || out_stride % 8) return dd_fail("dd_attention_rows: row strides must be multiples of 8");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DD_F32)
        return launch_rows<float>(q, q_stride, cache, tok_entry, tok_pos, block_table, max_blocks, out, out_stride,
                                  part_o, part_ml, n_tokens, n_heads, n_kv_heads, head_dim, page_size, n_pages,
                                  window, scale, n_splits, error_flag, s);
    if (dtype == DD_BF16)
        return launch_rows<__nv_bfloat16>(q, q_stride, cache, tok_entry, tok_pos, block_table, max_blocks, out,
                                          out_stride, part_o, part_ml, n_tokens, n_heads, n_kv_heads, head_dim,
                                          page_size, n_pages, window, scale, n_splits, error_flag, s);
    return dd_fail("dd_attention_rows: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------------------
// The variant for callers that cannot allocate (declared and described in no_alloc.h). The split
// scratch lives in this library's image; host code may not use the array's name as an address,
// so the device address is looked up once per device and handed to the same kernels as above.
#include "no_alloc.h"
#include <mutex>

static __device__ __align__(256) unsigned char dd_static_scratch[DD_STATIC_SCRATCH_BYTES];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_static_scratch[MAX_DEVICES] = {};
std::mutex g_static_mutex;

// The device address of dd_static_scratch on the current device, looked up on first use.
int static_scratch(float** ptr) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return dd_fail("dd_attention_rows_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= MAX_DEVICES) return dd_fail("dd_attention_rows_static: device %d is beyond %d", dev, MAX_DEVICES);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_scratch[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, dd_static_scratch);
        if (e != cudaSuccess || !p)
            return dd_fail("dd_attention_rows_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_static_scratch[dev] = static_cast<float*>(p);
    }
    *ptr = g_static_scratch[dev];
    return 0;
}
}  // namespace

DD_API int dd_attention_rows_static(const void* q, int q_stride, const void* cache, const int* tok_entry,
                                    const int* tok_pos, const int* block_table, int max_blocks, void* out,
                                    int out_stride, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                    int page_size, int n_pages, int window, float scale, int n_splits, int dtype,
                                    int* error_flag, void* stream) {
    if (n_tokens <= 0) return 0;
    if (n_splits < 1) return dd_fail("dd_attention_rows_static: n_splits=%d", n_splits);
    float* part_o = nullptr;
    float* part_ml = nullptr;
    if (n_splits > 1) {
        if (n_heads <= 0 || head_dim <= 0) return dd_fail("dd_attention_rows_static: bad sizes");
        const unsigned long long items = (unsigned long long)n_tokens * n_heads * n_splits;
        const unsigned long long need = items * (unsigned long long)(head_dim + 2) * sizeof(float);
        if (need > DD_STATIC_SCRATCH_BYTES)
            return dd_fail("dd_attention_rows_static: %d tokens x %d heads x %d splits x head size %d need %llu bytes of "
                           "scratch; the built-in scratch holds %u (use dd_attention_rows with your own buffers, or fewer splits)",
                           n_tokens, n_heads, n_splits, head_dim, need, DD_STATIC_SCRATCH_BYTES);
        float* base = nullptr;
        if (int e = static_scratch(&base)) return e;
        part_o = base;                                   // [items, head_dim]
        part_ml = base + items * head_dim;               // [items, 2]
    }
    return dd_attention_rows(q, q_stride, cache, tok_entry, tok_pos, block_table, max_blocks, out, out_stride, part_o,
                             part_ml, n_tokens, n_heads, n_kv_heads, head_dim, page_size, n_pages, window, scale,
                             n_splits, dtype, error_flag, stream);
}
