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

// Rows whose width is a multiple of 4 and at most 128 * 4 * VPT: 128 threads, the row in registers as
// float4, 16-byte loads and packed stores. Sixteen such blocks share an SM, so thousands of rows stream.
template <typename TO> struct Pack4;
template <> struct Pack4<float> {
    __device__ static void store(float* dst, float a, float b, float c, float d) { *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d); }
};
template <> struct Pack4<__nv_bfloat16> {
    __device__ static void store(__nv_bfloat16* dst, float a, float b, float c, float d) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 v;
        v.x = *reinterpret_cast<uint32_t*>(&lo);
        v.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst) = v;
    }
};

template <typename TO, int VPT>
__global__ void __launch_bounds__(128)
layernorm_vec_kernel(const float* __restrict__ x, const int* __restrict__ row_index,
                     const float* __restrict__ gamma, const float* __restrict__ beta,
                     TO* __restrict__ out, int width, float eps) {
    __shared__ float scratch[4];
    dd_launch_dependents();
    const int row = blockIdx.x;
    const int n4 = width >> 2;
    // gamma and beta are weights: they are in registers before the kernel that produces x has finished
    float4 g[VPT], b[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * 128;
        g[i] = c < n4 ? __ldg(reinterpret_cast<const float4*>(gamma) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        b[i] = (beta && c < n4) ? __ldg(reinterpret_cast<const float4*>(beta) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    dd_grid_wait();
    const float4* in = reinterpret_cast<const float4*>(x + (size_t)(row_index ? row_index[row] : row) * width);
    float4 v[VPT];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * 128;
        v[i] = c < n4 ? in[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    const float mean = block_sum<128>(sum, scratch) / (float)width;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        if (threadIdx.x + i * 128 < n4) {
            const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
            sq += (a * a + b * b) + (c * c + d * d);
        }
    }
    const float rstd = 1.0f / sqrtf(block_sum<128>(sq, scratch) / (float)width + eps);
    TO* o = out + (size_t)row * width;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * 128;
        if (c < n4)
            Pack4<TO>::store(o + 4 * c, (v[i].x - mean) * rstd * g[i].x + b[i].x, (v[i].y - mean) * rstd * g[i].y + b[i].y,
                             (v[i].z - mean) * rstd * g[i].z + b[i].z, (v[i].w - mean) * rstd * g[i].w + b[i].w);
    }
}

DD_API int dd_layernorm(const float* x, const int* row_index, const float* gamma, const float* beta,
                        void* out, int rows, int width, float eps, int out_dtype, void* stream) {
    if (rows <= 0) return 0;
    if (width <= 0) return dd_fail("dd_layernorm: bad width %d", width);
    cudaStream_t s = (cudaStream_t)stream;
    if (width % 4 == 0 && width <= 128 * 4 * 4 && !(((uintptr_t)x | (uintptr_t)out | (uintptr_t)gamma | (uintptr_t)beta) & 15)) {
        if (out_dtype == DD_F32)
            dd_launch(layernorm_vec_kernel<float, 4>, dim3(rows), dim3(128), 0, s, x, row_index, gamma, beta, (float*)out, width, eps);
        else if (out_dtype == DD_BF16)
            dd_launch(layernorm_vec_kernel<__nv_bfloat16, 4>, dim3(rows), dim3(128), 0, s, x, row_index, gamma, beta,
                      (__nv_bfloat16*)out, width, eps);
        else
            return dd_fail("dd_layernorm: unknown output dtype %d", out_dtype);
        return dd_check_launch("dd_layernorm");
    }
    if (out_dtype == DD_F32)
        dd_launch(layernorm_kernel<float, 256, 8>, dim3(rows), dim3(256), 0, s, x, row_index, gamma, beta, (float*)out, width, eps);
    else if (out_dtype == DD_BF16)
        dd_launch(layernorm_kernel<__nv_bfloat16, 256, 8>, dim3(rows), dim3(256), 0, s, x, row_index, gamma, beta,
                                                                  (__nv_bfloat16*)out, width, eps);
    else
        return dd_fail("dd_layernorm: unknown output dtype %d", out_dtype);
    return dd_check_launch("dd_layernorm");
}
