// C[M,N] = act(A[M,K] . W[N,K]^T + bias) (+ residual): plain CUDA-core GEMM with
// float32 multiply-add and no tensor-core or reduced-precision mode. It is the
// matrix product of the true 32-bit path, and (with bfloat16 operands) the slow
// stand-in that the tensor-core kernels are checked against. Every output element
// is summed over k in ascending order by one thread, so a row's result does not
// depend on how many other rows are in the batch.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, THREADS = 256;

template <typename TI, typename TO>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(const TI* __restrict__ A, int lda, const TI* __restrict__ W, int ldw,
                 const float* __restrict__ bias, const float* residual, int ldr,
                 TO* C, int ldc, int M, int N, int K, int act) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    dd_launch_dependents();
    dd_grid_wait();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    const bool a_row = (m0 + lr) < M, w_row = (n0 + lr) < N;
    const TI* a_ptr = A + (size_t)(m0 + lr) * lda;
    const TI* w_ptr = W + (size_t)(n0 + lr) * ldw;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int kk = k0 + lk + i;
            As[lk + i][lr] = (a_row && kk < K) ? dd_to_f32(a_ptr[kk]) : 0.f;
            Ws[lk + i][lr] = (w_row && kk < K) ? dd_to_f32(w_ptr[kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 w = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            v = dd_activation(v, act);
            if (residual) v += residual[(size_t)m * ldr + n];
            C[(size_t)m * ldc + n] = dd_from_f32<TO>(v);
        }
    }
}

template <typename TI, typename TO>
int launch(const void* A, int lda, const void* W, int ldw, const float* bias, const float* residual, int ldr,
           void* C, int ldc, int M, int N, int K, int act, cudaStream_t s) {
    dim3 grid(dd_ceil_div(N, BN), dd_ceil_div(M, BM));
    if (grid.y > 65535) return dd_fail("dd_gemm_simt: too many rows (%d)", M);
    dd_launch(gemm_simt_kernel<TI, TO>, dim3(grid), dim3(THREADS), 0, s, (const TI*)A, lda, (const TI*)W, ldw, bias, residual, ldr,
                                                     (TO*)C, ldc, M, N, K, act);
    return dd_check_launch("dd_gemm_simt");
}
}  // namespace

// A [M,K] (row stride lda) and W [N,K] (row stride ldw) in in_dtype; bias [N] and
// residual [M,N] (row stride ldr, may be the output itself) float32 or null.
DD_API int dd_gemm_simt(const void* A, int lda, const void* W, int ldw, const float* bias,
                        const float* residual, int ldr, void* C, int ldc, int M, int N, int K,
                        int act, int in_dtype, int out_dtype, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return dd_fail("dd_gemm_simt: bad K=%d", K);
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == DD_F32 && out_dtype == DD_F32)
        return launch<float, float>(A, lda, W, ldw, bias, residual, ldr, C, ldc, M, N, K, act, s);
    if (in_dtype == DD_BF16 && out_dtype == DD_F32)
        return launch<__nv_bfloat16, float>(A, lda, W, ldw, bias, residual, ldr, C, ldc, M, N, K, act, s);
    if (in_dtype == DD_BF16 && out_dtype == DD_BF16)
        return launch<__nv_bfloat16, __nv_bfloat16>(A, lda, W, ldw, bias, residual, ldr, C, ldc, M, N, K, act, s);
    return dd_fail("dd_gemm_simt: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
}
