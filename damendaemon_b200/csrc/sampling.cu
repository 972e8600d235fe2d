// Token selection from float32 logits, one thread block per row.
//
// Greedy: the first index of the maximum; a row whose maximum is NaN, +inf or -inf
// yields -1 so that the host can fail closed (damendaemon/sampling.py:131-139,189-203).
// Sampled rows follow damendaemon/sampling.py:140-177: keep the top_k largest logits,
// softmax(logits / T) over them, keep the most probable tokens until their mass reaches
// top_p (the crossing token stays), then an inverse-CDF draw with u in [0,1) that the
// host took from the request's own random stream. Here both filters are thresholds on
// the logit found by bisection over the ordered bit patterns of float32 (tokens that tie
// with the threshold all stay), and the cumulative sum runs in token-id order.
// Exponentials are float32, running sums double.
//
// dd_adjust_logits applies repetition, frequency and presence penalties and logit bias
// to listed (row, token) pairs (damendaemon/sampling.py:86-104).
#include "common.cuh"
#include <math_constants.h>

namespace {
constexpr int THREADS = 512;

struct Best { float v; int i; };

__device__ __forceinline__ Best better(Best a, Best b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ Best block_argmax(const float* row, int V, bool* saw_nan, Best* sh, int* sh_nan) {
    Best best{-CUDART_INF_F, 0x7fffffff};
    int nan = 0;
    // A row of an odd vocabulary starts anywhere: a few single values up to the first 16-byte boundary, then four values
    // a load and four loads in flight per thread (one value a load, the scan of 50,257 logits took 11 us of a decode
    // step), then the last few.
    const int head = min(V, (int)(((16 - ((uintptr_t)row & 15)) & 15) >> 2));
    const int n4 = (V - head) >> 2;
    if ((int)threadIdx.x < head) {
        const float v = row[threadIdx.x];
        nan |= (v != v);
        best = better(best, Best{v, (int)threadIdx.x});
    }
    const float4* body = reinterpret_cast<const float4*>(row + head);
#pragma unroll 4
    for (int j = threadIdx.x; j < n4; j += THREADS) {
        const float4 v = body[j];
        const int i = head + 4 * j;
        nan |= (v.x != v.x) | (v.y != v.y) | (v.z != v.z) | (v.w != v.w);
        best = better(best, Best{v.x, i});
        best = better(best, Best{v.y, i + 1});
        best = better(best, Best{v.z, i + 2});
        best = better(best, Best{v.w, i + 3});
    }
    for (int i = head + 4 * n4 + threadIdx.x; i < V; i += THREADS) {
        const float v = row[i];
        nan |= (v != v);
        best = better(best, Best{v, i});
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
        nan |= __shfl_xor_sync(0xffffffffu, nan, o);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sh[warp] = best; sh_nan[warp] = nan; }
    __syncthreads();
    best = sh[0]; nan = sh_nan[0];
    for (int w = 1; w < THREADS / 32; ++w) { best = better(best, sh[w]); nan |= sh_nan[w]; }
    __syncthreads();
    *saw_nan = nan != 0;
    return best;
}

__device__ double block_sum_double(double v, double* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    double total = 0.0;
    for (int w = 0; w < THREADS / 32; ++w) total += sh[w];
    __syncthreads();
    return total;
}

// float32 -> uint32 that orders like the floats
__device__ __forceinline__ uint32_t ordered(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float unordered(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int ldl, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const double* __restrict__ uniform, int* __restrict__ out) {
    __shared__ Best sh_best[THREADS / 32];
    __shared__ int sh_nan[THREADS / 32];
    __shared__ double sh_d[THREADS / 32];
    __shared__ double prefix[THREADS];
    __shared__ int sh_found;
    dd_launch_dependents();
    dd_grid_wait();
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * ldl;
    const float T = temperature ? temperature[r] : 0.f;       // asked for before the scan, not after it
    bool nan;
    const Best best = block_argmax(row, V, &nan, sh_best, sh_nan);
    if (nan || !(best.v > -CUDART_INF_F) || best.v == CUDART_INF_F) {
        if (threadIdx.x == 0) out[r] = -1;
        return;
    }
    if (!(T > 0.f)) {
        if (threadIdx.x == 0) out[r] = best.i;
        return;
    }
    const float inv_t = 1.0f / T;
    float threshold = -CUDART_INF_F;                  // tokens with logit >= threshold stay
    const int k = top_k ? top_k[r] : 0;
    if (k > 0 && k < V) {
        // largest key such that at least k logits are >= it
        uint32_t lo = 0u, hi = ordered(best.v);
        while (lo < hi) {
            const uint32_t mid = lo + (uint32_t)(((unsigned long long)hi - lo + 1) >> 1);
            double cnt = 0.0;
            for (int i = threadIdx.x; i < V; i += THREADS) cnt += ordered(row[i]) >= mid ? 1.0 : 0.0;
            if (block_sum_double(cnt, sh_d) >= (double)k) lo = mid; else hi = mid - 1;
        }
        threshold = unordered(lo);
    }
    const float p = top_p ? top_p[r] : 1.f;
    if (p < 1.f) {
        double mass = 0.0;
        for (int i = threadIdx.x; i < V; i += THREADS)
            if (row[i] >= threshold) mass += (double)expf((row[i] - best.v) * inv_t);
        const double need = (double)p * block_sum_double(mass, sh_d);
        // largest key such that the tokens at or above it hold at least `need`
        uint32_t lo = ordered(threshold), hi = ordered(best.v);
        while (lo < hi) {
            const uint32_t mid = lo + (uint32_t)(((unsigned long long)hi - lo + 1) >> 1);
            double part = 0.0;
            for (int i = threadIdx.x; i < V; i += THREADS)
                if (ordered(row[i]) >= mid) part += (double)expf((row[i] - best.v) * inv_t);
            if (block_sum_double(part, sh_d) >= need) lo = mid; else hi = mid - 1;
        }
        threshold = fmaxf(threshold, unordered(lo));
    }
    // each thread owns one contiguous span, so that the cumulative order is the token order
    const int span = (V + THREADS - 1) / THREADS;
    const int begin = min(V, (int)threadIdx.x * span), end = min(V, begin + span);
    double mine = 0.0;
    for (int i = begin; i < end; ++i)
        if (row[i] >= threshold) mine += (double)expf((row[i] - best.v) * inv_t);
    const double total = block_sum_double(mine, sh_d);
    const double target = uniform[r] * total;
    prefix[threadIdx.x] = mine;
    if (threadIdx.x == 0) sh_found = 0x7fffffff;
    __syncthreads();
    if (threadIdx.x == 0) {
        double run = 0.0;
        for (int t = 0; t < THREADS; ++t) { const double v = prefix[t]; prefix[t] = run; run += v; }
    }
    __syncthreads();
    const double before = prefix[threadIdx.x];
    if (before <= target && begin < end) {
        double run = before;
        for (int i = begin; i < end; ++i) {
            if (row[i] >= threshold) {
                run += (double)expf((row[i] - best.v) * inv_t);
                if (run > target) { atomicMin(&sh_found, i); break; }
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) out[r] = sh_found == 0x7fffffff ? best.i : sh_found;
}

__global__ void adjust_kernel(float* __restrict__ logits, int ldl, int V, const int* __restrict__ item_row,
                              const int* __restrict__ item_token, const float* __restrict__ item_count,
                              const float* __restrict__ item_bias, const int* __restrict__ item_seen,
                              const float* __restrict__ repetition, const float* __restrict__ frequency,
                              const float* __restrict__ presence, int n_items) {
    dd_launch_dependents();
    dd_grid_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_items) return;
    const int r = item_row[i], t = item_token[i];
    if (t < 0 || t >= V) return;
    float x = logits[(size_t)r * ldl + t];
    if (item_seen[i] && repetition[r] != 1.f) x = x > 0.f ? x / repetition[r] : x * repetition[r];
    if (item_count[i] > 0.f) x -= item_count[i] * frequency[r] + presence[r];
    x += item_bias[i];
    logits[(size_t)r * ldl + t] = x;
}
}  // namespace

// logits [rows, V] float32 with row stride ldl; temperature [rows] float32 (null = all greedy);
// top_k [rows] int32 (null or 0 = off); top_p [rows] float32 (null or 1 = off); uniform [rows]
// float64 in [0,1) (read only where temperature > 0); out [rows] int32, -1 for a row without a
// finite maximum.
DD_API int dd_sample(const float* logits, int ldl, int rows, int V, const float* temperature, const int* top_k,
                     const float* top_p, const double* uniform, int* out, void* stream) {
    if (rows <= 0) return 0;
    if (V <= 0) return dd_fail("dd_sample: empty vocabulary");
    dd_launch(sample_kernel, dim3(rows), dim3(THREADS), 0, (cudaStream_t)stream, logits, ldl, V, temperature, top_k, top_p, uniform, out);
    return dd_check_launch("dd_sample");
}

// One item per (row, token) that needs a change; each (row, token) pair at most once.
// seen: the token is in the prompt or the output (repetition penalty applies);
// count: times the token was generated (frequency and presence penalties); bias: added last.
DD_API int dd_adjust_logits(float* logits, int ldl, int V, const int* item_row, const int* item_token,
                            const float* item_count, const float* item_bias, const int* item_seen,
                            const float* repetition, const float* frequency, const float* presence, int n_items,
                            void* stream) {
    if (n_items <= 0) return 0;
    dd_launch(adjust_kernel, dim3(dd_ceil_div(n_items, 256)), dim3(256), 0, (cudaStream_t)stream, 
        logits, ldl, V, item_row, item_token, item_count, item_bias, item_seen, repetition, frequency, presence, n_items);
    return dd_check_launch("dd_adjust_logits");
}
