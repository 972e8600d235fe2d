// Token selection from float32 logits, one thread block per row.
//
// Greedy: the first index of the maximum; a row whose maximum is NaN, +inf or -inf
// yields -1 so that the host can fail closed (damendaemon/sampling.py:131-139,189-203).
// Temperature: p = softmax(logits / T) in token order, c its cumulative sum; the
// token is the first index with c > u * c[last], u in [0,1) drawn by the host from
// the request's own random stream (damendaemon/sampling.py:166-177). Exponentials are
// float32, the running sums double, so the choice does not depend on the block shape.
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
    for (int i = threadIdx.x; i < V; i += THREADS) {
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

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int ldl, int V, const float* __restrict__ temperature,
              const double* __restrict__ uniform, int* __restrict__ out) {
    __shared__ Best sh_best[THREADS / 32];
    __shared__ int sh_nan[THREADS / 32];
    __shared__ double sh_d[THREADS / 32];
    __shared__ int sh_found;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * ldl;
    bool nan;
    const Best best = block_argmax(row, V, &nan, sh_best, sh_nan);
    if (nan || !(best.v > -CUDART_INF_F) || best.v == CUDART_INF_F) {
        if (threadIdx.x == 0) out[r] = -1;
        return;
    }
    const float T = temperature ? temperature[r] : 0.f;
    if (!(T > 0.f)) {
        if (threadIdx.x == 0) out[r] = best.i;
        return;
    }
    const float inv_t = 1.0f / T;
    // each thread owns one contiguous span, so that the cumulative order is the token order
    const int span = (V + THREADS - 1) / THREADS;
    const int begin = min(V, (int)threadIdx.x * span), end = min(V, begin + span);
    double mine = 0.0;
    for (int i = begin; i < end; ++i) mine += (double)expf((row[i] - best.v) * inv_t);
    const double total = block_sum_double(mine, sh_d);
    const double target = uniform[r] * total;
    // exclusive prefix of the spans (THREADS values; a serial pass by one warp is cheap enough)
    __shared__ double prefix[THREADS];
    prefix[threadIdx.x] = mine;
    if (threadIdx.x == 0) sh_found = V - 1;
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
            run += (double)expf((row[i] - best.v) * inv_t);
            if (run > target) { atomicMin(&sh_found, i); break; }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) out[r] = sh_found;
}
}  // namespace

// logits [rows, V] float32 with row stride ldl; temperature [rows] float32 (null = all greedy);
// uniform [rows] float64 in [0,1) (read only where temperature > 0); out [rows] int32, -1 for a
// row without a finite maximum.
DD_API int dd_sample(const float* logits, int ldl, int rows, int V, const float* temperature,
                     const double* uniform, int* out, void* stream) {
    if (rows <= 0) return 0;
    if (V <= 0) return dd_fail("dd_sample: empty vocabulary");
    sample_kernel<<<rows, THREADS, 0, (cudaStream_t)stream>>>(logits, ldl, V, temperature, uniform, out);
    return dd_check_launch("dd_sample");
}
