// LayerNorm over the float32 residual stream: y = (x - mean) / sqrt(var + eps) * gamma + beta,
// biased variance, statistics in float32 with a true two-pass variance
// (damendaemon/starcoder.py:53-55). Output in the engine dtype. An optional row
// index gathers rows first (the final norm runs only where logits are wanted).
#include "common.cuh"

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    v = dd_warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) total += scratch[w];
    return total;
}

// Rows up to THREADS * PER elements are read once and kept in registers; wider rows are re-read.
template <typename TO, int THREADS, int PER>
__global__ void __launch_bounds__(THREADS)
layernorm_kernel(const float* __restrict__ x, const int* __restrict__ row_index,
                 const float* __restrict__ gamma, const float* __restrict__ beta,
                 TO* __restrict__ out, int width, float eps) {
    __shared__ float scratch[THREADS / 32];
    dd_launch_dependents();
    dd_grid_wait();
    const int row = blockIdx.x;
    const float* in = x + (size_t)(row_index ? row_index[row] : row) * width;
    TO* o = out + (size_t)row * width;
    if (width <= THREADS * PER) {
        float v[PER];
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int c = threadIdx.x + i * THREADS;
            v[i] = c < width ? in[c] : 0.f;
            sum += v[i];
        }
        const float mean = block_sum<THREADS>(sum, scratch) / (float)width;
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int c = threadIdx.x + i * THREADS;
            const float dlt = c < width ? v[i] - mean : 0.f;
            sq += dlt * dlt;
        }
        const float rstd = 1.0f / sqrtf(block_sum<THREADS>(sq, scratch) / (float)width + eps);
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int c = threadIdx.x + i * THREADS;
            if (c < width) {
                float y = (v[i] - mean) * rstd * gamma[c];
                if (beta) y += beta[c];
                o[c] = dd_from_f32<TO>(y);
            }
        }
        return;
    }
    float sum = 0.f;
    for (int c = threadIdx.x; c < width; c += THREADS) sum += in[c];
    const float mean = block_sum<THREADS>(sum, scratch) / (float)width;
    float sq = 0.f;
    for (int c = threadIdx.x; c < width; c += THREADS) {
        const float dlt = in[c] - mean;
        sq += dlt * dlt;
    }
    const float var = block_sum<THREADS>(sq, scratch) / (float)width;
    const float rstd = 1.0f / sqrtf(var + eps);
    for (int c = threadIdx.x; c < width; c += THREADS) {
        float v = (in[c] - mean) * rstd * gamma[c];
        if (beta) v += beta[c];
        o[c] = dd_from_f32<TO>(v);
    }
}

DD_API int dd_layernorm(const float* x, const int* row_index, const float* gamma, const float* beta,
                        void* out, int rows, int width, float eps, int out_dtype, void* stream) {
    if (rows <= 0) return 0;
    if (width <= 0) return dd_fail("dd_layernorm: bad width %d", width);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == DD_F32)
        dd_launch(layernorm_kernel<float, 256, 8>, dim3(rows), dim3(256), 0, s, x, row_index, gamma, beta, (float*)out, width, eps);
    else if (out_dtype == DD_BF16)
        dd_launch(layernorm_kernel<__nv_bfloat16, 256, 8>, dim3(rows), dim3(256), 0, s, x, row_index, gamma, beta,
                                                                  (__nv_bfloat16*)out, width, eps);
    else
        return dd_fail("dd_layernorm: unknown output dtype %d", out_dtype);
    return dd_check_launch("dd_layernorm");
}
