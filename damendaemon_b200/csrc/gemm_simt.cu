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

// ---- few rows (a decode step): float32 operands ----
// A block owns RB_N (32, or 16 for a narrow product, so that a hundred blocks stream it) output features for all MR
// rows of A and streams its rows of W once, in chunks of 32 k through
// a ring of cp.async stages (16-byte copies; 128 bytes of a row per chunk), so that a step of a few tokens reads
// the weights at memory speed instead of tile by tile. A thread owns one feature and MR / 4 rows; each of its
// outputs is summed over k in ascending order with fmaf from zero, exactly the arithmetic of the tiled kernel above,
// so the two give the same bits and a row's result does not depend on which of them a step's size selects.
constexpr int RB_K = 32, RB_THREADS = 128, RB_LD = RB_K + 4;   // rows padded: 16-byte aligned, float4 reads conflict-free

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool live) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = live ? 16 : 0;                       // zero-fill beyond the matrix
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

template <int MR, int RB_N, typename TO>
__global__ void __launch_bounds__(RB_THREADS)
gemm_simt_rows_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw,
                      const float* __restrict__ bias, const float* residual, int ldr,
                      TO* C, int ldc, int M, int N, int K, int act) {
    constexpr int PER = MR * RB_N / RB_THREADS;             // rows of A per thread (1 to 8)
    static_assert(PER >= 1 && MR * RB_N % RB_THREADS == 0, "a thread owns whole rows");
    constexpr int RB_STAGES = MR <= 16 ? 6 : (MR <= 32 ? 4 : 3);   // at most 41 KB of static shared memory
    __shared__ __align__(16) float Ws[RB_STAGES][RB_N][RB_LD];
    __shared__ __align__(16) float As[RB_STAGES][MR][RB_LD];
    const int n0 = blockIdx.x * RB_N;
    const int nl = threadIdx.x % RB_N, mg = threadIdx.x / RB_N;
    const int chunks = (K + RB_K - 1) / RB_K;
    // a chunk of W: RB_N rows x 8 pieces of 16 bytes, one or two per thread; of A: MR rows x 8 pieces
    auto load_w = [&](int c) {
        const int st = c % RB_STAGES, k0 = c * RB_K;
#pragma unroll
        for (int i = 0; i < RB_N * 8 / RB_THREADS; ++i) {
            const int piece = threadIdx.x + i * RB_THREADS, row = piece >> 3, kk = (piece & 7) * 4;
            const bool live = n0 + row < N && k0 + kk < K;          // K is a multiple of 4: a piece is inside or outside
            cp_async16(&Ws[st][row][kk], W + (size_t)(live ? n0 + row : 0) * ldw + (live ? k0 + kk : 0), live);
        }
    };
    auto load_a = [&](int c) {
        const int st = c % RB_STAGES, k0 = c * RB_K;
        for (int piece = threadIdx.x; piece < MR * 8; piece += RB_THREADS) {
            const int row = piece >> 3, kk = (piece & 7) * 4;
            const bool live = row < M && k0 + kk < K;
            cp_async16(&As[st][row][kk], A + (size_t)(live ? row : 0) * lda + (live ? k0 + kk : 0), live);
        }
    };
    // the weights do not depend on the kernel before this one: their first stages are requested before the wait
    for (int c = 0; c < RB_STAGES - 1 && c < chunks; ++c) load_w(c);
    dd_grid_wait();
    for (int c = 0; c < RB_STAGES - 1; ++c) {
        if (c < chunks) load_a(c);
        asm volatile("cp.async.commit_group;" ::: "memory");     // group c: A of chunk c (and, in group 0, all W so far)
    }
    float acc[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = 0.f;
    for (int c = 0; c < chunks; ++c) {
        asm volatile("cp.async.wait_group %0;" ::"n"(RB_STAGES - 2) : "memory");
        __syncthreads();                                    // chunk c has landed for everyone; stage (c-1) is free
        const int next = c + RB_STAGES - 1;
        if (next < chunks) { load_w(next); load_a(next); }
        asm volatile("cp.async.commit_group;" ::: "memory");
        const int st = c % RB_STAGES;
#pragma unroll
        for (int k4 = 0; k4 < RB_K; k4 += 4) {
            const float4 w = *reinterpret_cast<const float4*>(&Ws[st][nl][k4]);
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const float4 a = *reinterpret_cast<const float4*>(&As[st][mg * PER + i][k4]);
                acc[i] = fmaf(a.x, w.x, acc[i]);
                acc[i] = fmaf(a.y, w.y, acc[i]);
                acc[i] = fmaf(a.z, w.z, acc[i]);
                acc[i] = fmaf(a.w, w.w, acc[i]);
            }
        }
    }
    dd_launch_dependents();
    const int n = n0 + nl;
    if (n >= N) return;
    const float b = bias ? bias[n] : 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int m = mg * PER + i;
        if (m >= M) continue;
        float v = dd_activation(acc[i] + b, act);
        if (residual) v += residual[(size_t)m * ldr + n];
        C[(size_t)m * ldc + n] = dd_from_f32<TO>(v);
    }
}

template <int MR, int RB_N, typename TO>
int launch_rows(const void* A, int lda, const void* W, int ldw, const float* bias, const float* residual, int ldr,
                void* C, int ldc, int M, int N, int K, int act, cudaStream_t s) {
    dd_launch(gemm_simt_rows_kernel<MR, RB_N, TO>, dim3(dd_ceil_div(N, RB_N)), dim3(RB_THREADS), 0, s, (const float*)A, lda,
              (const float*)W, ldw, bias, residual, ldr, (TO*)C, ldc, M, N, K, act);
    return dd_check_launch("dd_gemm_simt");
}

// ---- many rows (a prompt portion): float32 operands ----
// Tiles of 128 x 128 outputs, 256 threads with 8 x 8 outputs each (rows ty + 16 i, features tx + 16 j, so that the
// 16-byte reads of a warp meet no bank twice), k in chunks of 16 through three cp.async stages. Every output is again
// one chain of fmaf over ascending k from zero: the same bits as the other two kernels.
constexpr int BG = 128, BG_K = 16, BG_LD = BG_K + 4, BG_STAGES = 3, BG_THREADS = 256;
constexpr int BG_SMEM = BG_STAGES * 2 * BG * BG_LD * 4;

__global__ void __launch_bounds__(BG_THREADS)
gemm_simt_big_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw,
                     const float* __restrict__ bias, const float* residual, int ldr,
                     float* C, int ldc, int M, int N, int K, int act) {
    extern __shared__ __align__(16) float big_smem[];
    float (*As)[BG][BG_LD] = reinterpret_cast<float (*)[BG][BG_LD]>(big_smem);
    float (*Ws)[BG][BG_LD] = reinterpret_cast<float (*)[BG][BG_LD]>(big_smem + BG_STAGES * BG * BG_LD);
    dd_launch_dependents();
    dd_grid_wait();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * BG, n0 = blockIdx.x * BG;
    const int chunks = (K + BG_K - 1) / BG_K;
    // a chunk: 128 rows x 4 pieces of 16 bytes for each operand, two pieces of each per thread
    auto load = [&](int c) {
        const int st = c % BG_STAGES, k0 = c * BG_K;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int piece = threadIdx.x + i * BG_THREADS, row = piece >> 2, kk = (piece & 3) * 4;
            const bool in_k = k0 + kk < K;
            const bool a_live = in_k && m0 + row < M, w_live = in_k && n0 + row < N;
            cp_async16(&As[st][row][kk], A + (size_t)(a_live ? m0 + row : 0) * lda + (a_live ? k0 + kk : 0), a_live);
            cp_async16(&Ws[st][row][kk], W + (size_t)(w_live ? n0 + row : 0) * ldw + (w_live ? k0 + kk : 0), w_live);
        }
    };
    for (int c = 0; c < BG_STAGES - 1; ++c) {
        if (c < chunks) load(c);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    for (int c = 0; c < chunks; ++c) {
        asm volatile("cp.async.wait_group %0;" ::"n"(BG_STAGES - 2) : "memory");
        __syncthreads();
        if (c + BG_STAGES - 1 < chunks) load(c + BG_STAGES - 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const int st = c % BG_STAGES;
#pragma unroll
        for (int k4 = 0; k4 < BG_K; k4 += 4) {
            float4 a[8], w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] = *reinterpret_cast<const float4*>(&As[st][ty + 16 * i][k4]);
#pragma unroll
            for (int j = 0; j < 8; ++j) w[j] = *reinterpret_cast<const float4*>(&Ws[st][tx + 16 * j][k4]);
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    acc[i][j] = fmaf(a[i].x, w[j].x, acc[i][j]);
                    acc[i][j] = fmaf(a[i].y, w[j].y, acc[i][j]);
                    acc[i][j] = fmaf(a[i].z, w[j].z, acc[i][j]);
                    acc[i][j] = fmaf(a[i].w, w[j].w, acc[i][j]);
                }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + ty + 16 * i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int n = n0 + tx + 16 * j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            v = dd_activation(v, act);
            if (residual) v += residual[(size_t)m * ldr + n];
            C[(size_t)m * ldc + n] = v;
        }
    }
}

int launch_big(const void* A, int lda, const void* W, int ldw, const float* bias, const float* residual, int ldr,
               void* C, int ldc, int M, int N, int K, int act, cudaStream_t s) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_simt_big_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BG_SMEM);
        if (e != cudaSuccess) return dd_fail("dd_gemm_simt: shared memory of %d bytes refused: %s", BG_SMEM, cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid(dd_ceil_div(N, BG), dd_ceil_div(M, BG));
    if (grid.y > 65535) return dd_fail("dd_gemm_simt: too many rows (%d)", M);
    dd_launch(gemm_simt_big_kernel, grid, dim3(BG_THREADS), BG_SMEM, s, (const float*)A, lda, (const float*)W, ldw, bias, residual,
              ldr, (float*)C, ldc, M, N, K, act);
    return dd_check_launch("dd_gemm_simt");
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
    if (in_dtype == DD_F32 && out_dtype == DD_F32) {
        // up to 64 rows with 16-byte aligned rows: the kernel that streams the weights once; more rows: tiles of 128 x 128
        const bool aligned = K % 4 == 0 && lda % 4 == 0 && ldw % 4 == 0 && !(((uintptr_t)A | (uintptr_t)W) & 15);
        const bool narrow = N < 3200;                      // fewer than a hundred blocks of 32 features
        if (aligned && M <= 8) return narrow ? launch_rows<8, 16, float>(A, lda, W, ldw, bias, residual, ldr, C, ldc, M, N, K, act, s)
                                             : launch_rows<8, 32, float>(A, lda, W, ldw, bias, residual, ldr, C, ldc, M, N, K, act, s);
        if (aligned && M <= 16) return narrow ? launch_rows<16, 16, float>(A, lda, W, ldw, bias, residual, ldr, C, ldc, M, N, K, act, s)
                                              : launch_rows<16, 32, float>(A, lda, W, ldw, bias, residual, ldr, C, ldc, M, N, K, act, s);
        if (aligned && M <= 32) return narrow ? launch_rows<32, 16, float>(A, lda, W, ldw, bias, residual, ldr, C, ldc, M, N, K, act, s)
                                              : launch_rows<32, 32, float>(A, lda, W, ldw, bias, residual, ldr, C, ldc, M, N, K, act, s);
        if (aligned && M <= 64) return narrow ? launch_rows<64, 16, float>(A, lda, W, ldw, bias, residual, ldr, C, ldc, M, N, K, act, s)
                                              : launch_rows<64, 32, float>(A, lda, W, ldw, bias, residual, ldr, C, ldc, M, N, K, act, s);
        if (aligned) return launch_big(A, lda, W, ldw, bias, residual, ldr, C, ldc, M, N, K, act, s);
        return launch<float, float>(A, lda, W, ldw, bias, residual, ldr, C, ldc, M, N, K, act, s);
    }
    if (in_dtype == DD_BF16 && out_dtype == DD_F32)
        return launch<__nv_bfloat16, float>(A, lda, W, ldw, bias, residual, ldr, C, ldc, M, N, K, act, s);
    if (in_dtype == DD_BF16 && out_dtype == DD_BF16)
        return launch<__nv_bfloat16, __nv_bfloat16>(A, lda, W, ldw, bias, residual, ldr, C, ldc, M, N, K, act, s);
    return dd_fail("dd_gemm_simt: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
}
