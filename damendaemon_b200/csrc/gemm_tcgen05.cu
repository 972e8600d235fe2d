// bfloat16 GEMM on the 5th-generation tensor cores: out[M,N] = act(X[M,K] . W[N,K]^T + bias) (+ residual).
//
// Three kernels share the pipeline (TMA loads of 64-element k slices with the 128-byte swizzle into a ring of
// stages guarded by full/empty mbarriers; one thread issuing tcgen05.mma from shared-memory descriptors and
// releasing stages with tcgen05.commit; epilogue warps reading the accumulator with tcgen05.ld) and differ in
// which operand is the 128-row side of the instruction and in how the work is spread:
//
//   by feature (token tiles of 16, 32 or 64): the product is computed transposed, D^T = W . X^T. The weight rows
//   (output features) are the 128 lanes of the accumulator and the tokens its columns, so a step of a few tokens
//   wastes no tensor-core rows; an epilogue thread owns one feature, its bias is one register, and a warp's 32
//   lanes write 32 consecutive features of a token row. Up to 64 tokens this is the cluster kernel: a cluster of
//   CTAs splits K, every CTA streams its share of the weight tile, and the partial tiles are summed over
//   distributed shared memory in a fixed order (deterministic), so the weights come from HBM once while all
//   SMs pull. Above 64 tokens the persistent kernel may use these tiles too (with a workspace split over K).
//
//   by token (token tiles of 128, persistent kernel): D = X . W^T, 128 tokens are the lanes and 128, 192 or 256
//   features the columns; an epilogue thread owns a token row and writes 16 features at a time as 16-byte
//   stores, with the residual read the same way. At most one CTA per SM walks over the tiles, the producer
//   runs ahead across tiles and the accumulator is double buffered in TMEM, so the epilogue of one tile
//   overlaps the MMAs of the next; eight epilogue warps, two per lane quarter, share a tile's columns.
//
//   two SMs per tile (pair kernel): tcgen05.mma.cta_group::2 over 256 tokens x up to 256 features; each CTA of
//   the pair loads its 128 tokens and half of the weight tile, so a weight byte is read into shared memory once
//   per 256 tokens.
//
// dd_gemm_tcgen05_plan chooses among them from the shape by counting rounds of tiles over the SMs.
// Weights, bias and everything else that does not come from the kernel before are fetched before
// griddepcontrol.wait, so that under programmatic dependent launch they overlap the previous kernel's tail.
//
// Every mbarrier wait is bounded (tcgen05.cuh); on a timeout the kernel sets bit 8 of the
// error word, stops waiting everywhere, frees its TMEM and returns.
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128;          // output features per tile (tcgen05.mma M)
constexpr int BK = 64;           // k elements per stage: one 128-byte swizzle row of bf16
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;     // cluster kernel: warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int EPI_WARPS = 8;     // persistent and two-SM kernels: two warps per TMEM lane quarter, each half of the tokens
constexpr int THREADS_P = 64 + 32 * EPI_WARPS;

struct GemmParams {
    const float* bias;           // [N] or null
    const float* residual;       // [M, ldr] or null
    void* out;                   // [M, ldo] bf16 or f32
    float* workspace;            // [splits, M, N] f32 (split-K only)
    int* counters;               // one per output tile, zero between launches (split-K only)
    int* error_flag;
    int M, N, K;                 // tokens, output features, reduction
    int ldr, ldo;
    int act, out_dtype;
    int splits, kblocks_per_split;
    int vec;                     // out, residual and bias allow 16-byte accesses at every row start (tiles of 128 tokens)
    const uint8_t* prefetch;        // null, or memory a later kernel will stream (the next weight matrix):
    unsigned long long prefetch_bytes;   // every block asks L2 to fetch its share while this kernel runs
};


template <int BN> struct Config {
    static constexpr bool BY_TOKEN = BN >= 128;      // accumulator lanes are tokens (else output features)
    static constexpr int STAGES = BN >= 256 ? 4 : (BN >= 192 ? 4 : (BN >= 128 ? 6 : 8));
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int ACC_COLS = BN == 192 ? 256 : (BN < 16 ? 16 : BN);   // columns of one accumulator (a power of two)
    static constexpr int TMEM_COLS = 2 * ACC_COLS < 32 ? 32 : 2 * ACC_COLS;   // two accumulators, a power of two >= 32
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// gelu_new for a bfloat16 result: the hardware tanh (tanh.approx.f32, relative error about 2^-11) is below what
// bfloat16 keeps; with tanhf the epilogue of a 128x128 tile took longer than its MMAs (93 us against 57 us for
// the 6400-wide projection of 2,048 tokens). float32 outputs and the erf form keep the exact functions.
__device__ __forceinline__ float activation_for(float u, int act, int out_dtype) {
    if (act == DD_ACT_GELU_NEW && out_dtype == DD_BF16) {
        float t;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * (u + 0.044715f * u * u * u)));
        return 0.5f * u * (1.0f + t);
    }
    return dd_activation(u, act);
}

// The cluster variant keeps a reduce buffer of (BM + 8) x BN floats beside the stages.
template <int BN, bool DEEP = false> struct ClusterConfig {
    // 16 tokens: 5 stages, so that two blocks fit on an SM, with enough splits that a block seldom reuses a stage
    // (with the splits of the 8-stage rings, 5 stages measured 15-40% slower; with more splits, 5-20% faster)
    // DEEP (16 tokens only): 10 stages, one block per SM, for a long K: a block's whole share of the weights is
    // asked for before the activations exist
    static constexpr int STAGES = DEEP ? 10 : (BN >= 64 ? 6 : (BN == 16 ? 5 : 8));
    static constexpr int STAGE_BYTES = Config<BN>::STAGE_BYTES;
    static constexpr int A_BYTES = Config<BN>::A_BYTES;
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    static constexpr int REDUCE_BYTES = (BM + 8) * BN * 4;
    static constexpr int BIAS_BYTES = BM * 4;               // the bias of this block's slice of features
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + REDUCE_BYTES + BIAS_BYTES;
};

// Which 16-byte piece of its row (BN floats) feature lf's piece c is stored at: c ^ reduce_swizzle(lf). Rows of 64
// bytes (16 tokens) come two to a 128-byte line, so the feature's bit 0 already separates them.
template <int BN> __device__ __forceinline__ int reduce_swizzle(int lf) { return BN >= 32 ? (lf & 7) : ((lf >> 1) & 3); }

// Ask L2 to fetch this block's share of p.prefetch (16-byte granules, 32 KB per request).
__device__ __forceinline__ void prefetch_share(const GemmParams& p) {
    if (!p.prefetch_bytes) return;
    const unsigned long long share = ((p.prefetch_bytes + gridDim.x - 1) / gridDim.x + 127) & ~127ull;
    const unsigned long long begin = (unsigned long long)blockIdx.x * share;
    if (begin >= p.prefetch_bytes) return;
    const unsigned long long end = min(p.prefetch_bytes, begin + share) & ~15ull;
    for (unsigned long long at = begin; at < end; at += 32768) {
        const unsigned n = (unsigned)min(32768ull, end - at);
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.prefetch + at), "r"(n) : "memory");
    }
}

// Epilogue of 16 consecutive tokens (m_first ..) of one output feature n, specialised at compile time on the
// activation, the output type and the presence of a residual, so that the element loop has no run-time choices
// (with them in the loop the epilogue of a 128x128 tile took 14.6 us against 7.5 us, and it is the epilogue, not
// the MMAs at 5 us, that bounds a K = 1600 tile). The residual may be the output itself, so all 16 residual
// values are read before anything is written: the loads stay independent instead of being ordered behind each
// store.
template <int ACT, bool BF16_OUT, bool RESIDUAL>
__device__ __forceinline__ void store16(const GemmParams& p, int m_first, int n, const float* acc, float b, const float* r) {
    const int live = min(16, p.M - m_first);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        if (j >= live) break;
        float v = acc[j] + b;
        if (ACT == DD_ACT_GELU_NEW) {
            if (BF16_OUT) {
                float t;
                asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * (v + 0.044715f * v * v * v)));
                v = 0.5f * v * (1.0f + t);
            } else v = dd_activation(v, DD_ACT_GELU_NEW);
        } else if (ACT == DD_ACT_GELU_ERF) v = dd_activation(v, DD_ACT_GELU_ERF);
        if (RESIDUAL) v += r[j];
        if (BF16_OUT) reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)(m_first + j) * p.ldo + n] = __float2bfloat16_rn(v);
        else reinterpret_cast<float*>(p.out)[(size_t)(m_first + j) * p.ldo + n] = v;
    }
}

template <int ACT, bool BF16_OUT>
__device__ __forceinline__ void store16_r(const GemmParams& p, int m_first, int n, const float* acc, float b, const float* r) {
    if (p.residual) store16<ACT, BF16_OUT, true>(p, m_first, n, acc, b, r);
    else store16<ACT, BF16_OUT, false>(p, m_first, n, acc, b, r);
}

template <int ACT>
__device__ __forceinline__ void store16_o(const GemmParams& p, int m_first, int n, const float* acc, float b, const float* r) {
    if (p.out_dtype == DD_BF16) store16_r<ACT, true>(p, m_first, n, acc, b, r);
    else store16_r<ACT, false>(p, m_first, n, acc, b, r);
}

// The 16 residual values of tokens m_first.. at feature n (zeros without a residual or past the last token).
__device__ __forceinline__ void load_residual16(const GemmParams& p, int m_first, int n, float* r) {
#pragma unroll
    for (int j = 0; j < 16; ++j)
        r[j] = (p.residual && m_first + j < p.M) ? p.residual[(size_t)(m_first + j) * p.ldr + n] : 0.f;
}

// r: residual values already loaded (load_residual16), issued by the caller before it waits for the accumulator.
__device__ __forceinline__ void store_out16(const GemmParams& p, int m_first, int n, const float* acc, const float* r, float b) {
    if (p.act == DD_ACT_NONE) store16_o<DD_ACT_NONE>(p, m_first, n, acc, b, r);
    else if (p.act == DD_ACT_GELU_NEW) store16_o<DD_ACT_GELU_NEW>(p, m_first, n, acc, b, r);
    else store16_o<DD_ACT_GELU_ERF>(p, m_first, n, acc, b, r);
}

__device__ __forceinline__ void store_out16(const GemmParams& p, int m_first, int n, const float* acc) {
    float r[16];
    load_residual16(p, m_first, n, r);
    store_out16(p, m_first, n, acc, r, p.bias ? p.bias[n] : 0.f);
}

// ---- epilogue of tiles whose accumulator lanes are tokens (tiles of 128 tokens x BN features) ----
// A thread holds 16 consecutive features n_first.. of its own token m: the bias comes in four 16-byte loads
// that are the same for every thread, the residual and the result move as 16-byte pieces of the thread's own row.
// With one output feature per thread instead (the orientation of the few-token tiles) a 128 x 128 tile needs 16
// scalar stores per thread and chunk, and that epilogue, not the MMAs, bounded the tiles of a 2,048-token step.
__device__ __forceinline__ void load_residual_row16(const GemmParams& p, int m, int n_first, float* r) {
    if (!p.residual) {
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] = 0.f;
        return;
    }
    const float* src = p.residual + (size_t)m * p.ldr + n_first;
    if (p.vec && n_first + 16 <= p.N) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 v = *reinterpret_cast<const float4*>(src + 4 * q);
            r[4 * q] = v.x; r[4 * q + 1] = v.y; r[4 * q + 2] = v.z; r[4 * q + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] = n_first + j < p.N ? src[j] : 0.f;
    }
}

// The bias of 16 consecutive features (zeros without one): the same for every thread, asked for while the accumulator
// is still on its way from TMEM, like the residual values.
__device__ __forceinline__ void load_bias16(const GemmParams& p, int n_first, float* v) {
    if (p.bias && p.vec && n_first + 16 <= p.N) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + n_first) + q);
            v[4 * q] = b.x; v[4 * q + 1] = b.y; v[4 * q + 2] = b.z; v[4 * q + 3] = b.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = (p.bias && n_first + j < p.N) ? __ldg(p.bias + n_first + j) : 0.f;
    }
}

template <int ACT, bool BF16_OUT, bool RESIDUAL>
__device__ __forceinline__ void store_row16(const GemmParams& p, int m, int n_first, const uint32_t* acc, const float* r, float* v) {
    const bool whole = p.vec && n_first + 16 <= p.N;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        float u = __uint_as_float(acc[j]) + v[j];
        if (ACT == DD_ACT_GELU_NEW) {
            if (BF16_OUT) {
                float t;
                asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * (u + 0.044715f * u * u * u)));
                u = 0.5f * u * (1.0f + t);
            } else u = dd_activation(u, DD_ACT_GELU_NEW);
        } else if (ACT == DD_ACT_GELU_ERF) u = dd_activation(u, DD_ACT_GELU_ERF);
        if (RESIDUAL) u += r[j];
        v[j] = u;
    }
    if (BF16_OUT) {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.ldo + n_first;
        if (whole) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * q + 2 * i], v[8 * q + 2 * i + 1]);
                    w[i] = *reinterpret_cast<const uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(dst + 8 * q) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (n_first + j < p.N) dst[j] = __float2bfloat16_rn(v[j]);
        }
    } else {
        float* dst = reinterpret_cast<float*>(p.out) + (size_t)m * p.ldo + n_first;
        if (whole) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
                *reinterpret_cast<float4*>(dst + 4 * q) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (n_first + j < p.N) dst[j] = v[j];
        }
    }
}

template <int ACT, bool BF16_OUT>
__device__ __forceinline__ void store_row16_r(const GemmParams& p, int m, int n_first, const uint32_t* acc, const float* r, float* v) {
    if (p.residual) store_row16<ACT, BF16_OUT, true>(p, m, n_first, acc, r, v);
    else store_row16<ACT, BF16_OUT, false>(p, m, n_first, acc, r, v);
}

template <int ACT>
__device__ __forceinline__ void store_row16_o(const GemmParams& p, int m, int n_first, const uint32_t* acc, const float* r, float* v) {
    if (p.out_dtype == DD_BF16) store_row16_r<ACT, true>(p, m, n_first, acc, r, v);
    else store_row16_r<ACT, false>(p, m, n_first, acc, r, v);
}

// v: the bias of the 16 features (load_bias16); it is used up as scratch
__device__ __forceinline__ void store_out_row16(const GemmParams& p, int m, int n_first, const uint32_t* acc, const float* r, float* v) {
    if (p.act == DD_ACT_NONE) store_row16_o<DD_ACT_NONE>(p, m, n_first, acc, r, v);
    else if (p.act == DD_ACT_GELU_NEW) store_row16_o<DD_ACT_GELU_NEW>(p, m, n_first, acc, r, v);
    else store_row16_o<DD_ACT_GELU_ERF>(p, m, n_first, acc, r, v);
}

// One SM per tile, persistent over tiles, two accumulators in TMEM so that the epilogue of one tile runs under the
// MMAs of the next. The 128 accumulator lanes (operand A, map_a) are output features when BN <= 64, the
// orientation for a few tokens: the weights fill the 128-row side of the MMA whatever the token count, and a
// thread of the epilogue owns one feature. For BN >= 128 the lanes are tokens and the BN columns are features,
// so that a thread of the epilogue owns a piece of one output row and moves it in 16-byte accesses.
template <int BN>
__global__ void __launch_bounds__(THREADS_P, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmParams p) {
    using C = Config<BN>;
    constexpr bool BY_TOKEN = C::BY_TOKEN;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(16) float bias_s[2][256];        // tiles of tokens: the bias of a tile's features, tiles alternating
    // the swizzled tiles need 1024-byte alignment
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + C::STAGES;
    uint64_t* tmem_full_bar = empty_bar + C::STAGES;      // [2]: accumulator a is complete
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;         // [2]: accumulator a has been read out
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* last_flag = const_cast<int*>(abort_flag) + 1;
    int* epilogue_abort = last_flag + 1;                  // written by epilogue threads only

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows_a = BY_TOKEN ? p.M : p.N, rows_b = BY_TOKEN ? p.N : p.M;
    const int tiles_a = (rows_a + BM - 1) / BM;
    const int tiles_b = (rows_b + BN - 1) / BN;
    const int n_items = tiles_a * tiles_b * p.splits;
    const int total_kblocks = (p.K + BK - 1) / BK;
    // which operand holds the weights
    const CUtensorMap* map_w = BY_TOKEN ? &map_b : &map_a;
    const CUtensorMap* map_x = BY_TOKEN ? &map_a : &map_b;
    constexpr int W_OFFSET = BY_TOKEN ? C::A_BYTES : 0, X_OFFSET = BY_TOKEN ? 0 : C::A_BYTES;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            tc::mbar_init(&full_bar[s], 1);
            tc::mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            tc::mbar_init(&tmem_full_bar[a], 1);
            tc::mbar_init(&tmem_empty_bar[a], EPI_WARPS);   // one arrival per epilogue warp
        }
        *abort_flag = 0;
        *last_flag = 0;
        *epilogue_abort = 0;
        tc::fence_barrier_init();
        tc::fence_proxy_async();
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, C::TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    dd_launch_dependents();      // the next kernel may begin its own set-up now

    // Work item -> (tile along A, tile along B, split). Tiles along A vary fastest, so blocks that run side by
    // side share the same B tile in L2.
#define DD_ITEM_COORDS(item)                                              \
    const int split = (item) % p.splits;                                  \
    const int tile = (item) / p.splits;                                   \
    const int a0 = (tile % tiles_a) * BM;                                 \
    const int b0 = (tile / tiles_a) * BN;                                 \
    const int w0 = BY_TOKEN ? b0 : a0, x0 = BY_TOKEN ? a0 : b0;           \
    const int kb_begin = split * p.kblocks_per_split;                     \
    const int n_kblocks = min(total_kblocks, kb_begin + p.kblocks_per_split) - kb_begin;

    if (warp == 0) {
        if (tc::elect_one()) {
            tc::prefetch_tensormap(&map_a);
            tc::prefetch_tensormap(&map_b);
            uint32_t it = 0;                               // k-blocks issued so far, across items
            bool ok = true;
            // Weights never change, so the weight tiles of the first stages are requested before the
            // kernel that produces the activations has finished; the activation tiles follow the wait.
            int ahead = 0;
            if (blockIdx.x < n_items) {
                DD_ITEM_COORDS(blockIdx.x)
                (void)x0;
                ahead = min(n_kblocks, C::STAGES);
                for (int i = 0; i < ahead; ++i) {
                    tc::mbar_expect_tx(&full_bar[i], C::STAGE_BYTES);
                    tc::tma_load_2d(tiles + i * C::STAGE_BYTES + W_OFFSET, map_w, (kb_begin + i) * BK, w0, &full_bar[i]);
                }
            }
            prefetch_share(p);
            dd_grid_wait();
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                DD_ITEM_COORDS(item)
                for (int i = 0; i < n_kblocks; ++i, ++it) {
                    const int s = it % C::STAGES;
                    uint8_t* stage = tiles + s * C::STAGE_BYTES;
                    if ((int)it < ahead) {                 // the weight tile of this stage is already on its way
                        tc::tma_load_2d(stage + X_OFFSET, map_x, (kb_begin + i) * BK, x0, &full_bar[s]);
                        continue;
                    }
                    const uint32_t phase = (it / C::STAGES) & 1;
                    if (!tc::mbar_wait(&empty_bar[s], phase ^ 1, abort_flag)) { ok = false; break; }
                    tc::mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
                    tc::tma_load_2d(stage + W_OFFSET, map_w, (kb_begin + i) * BK, w0, &full_bar[s]);
                    tc::tma_load_2d(stage + X_OFFSET, map_x, (kb_begin + i) * BK, x0, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (tc::elect_one()) {
            constexpr uint32_t idesc = tc::idesc_bf16_f32(BM, BN);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++local) {
                DD_ITEM_COORDS(item)
                (void)w0; (void)x0;
                const uint32_t acc = local & 1;
                // the epilogue must have drained this accumulator (passes at once the first two times)
                if (!tc::mbar_wait(&tmem_empty_bar[acc], ((local >> 1) & 1) ^ 1, abort_flag)) break;
                tc::fence_after_sync();
                const uint32_t tmem_d = tmem_base + acc * C::ACC_COLS;
                for (int i = 0; i < n_kblocks; ++i, ++it) {
                    const int s = it % C::STAGES;
                    const uint32_t phase = (it / C::STAGES) & 1;
                    if (!tc::mbar_wait(&full_bar[s], phase, abort_flag)) { ok = false; break; }
                    tc::fence_after_sync();
                    const uint32_t a_addr = tc::smem_u32(tiles + s * C::STAGE_BYTES);
                    const uint32_t b_addr = a_addr + C::A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t da = tc::smem_desc_sw128(a_addr + k * UMMA_K * 2);
                        const uint64_t db = tc::smem_desc_sw128(b_addr + k * UMMA_K * 2);
                        tc::mma_bf16(tmem_d, da, db, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    }
                    tc::mma_commit(&empty_bar[s]);     // the stage is free once these MMAs have read it
                }
                if (ok) tc::mma_commit(&tmem_full_bar[acc]);   // the accumulator is complete
            }
        }
    } else {
        // epilogue: warp w may touch TMEM lanes 32*(w%4) .. 32*(w%4)+31
        dd_grid_wait();              // bias is constant, but residual, workspace and counters are earlier kernels' data
        const int quarter = warp & 3;
        // the two warps of a lane quarter split the tile's columns in halves (in chunks of 16)
        constexpr int FIRST_HALF = ((BN / 16 + 1) / 2) * 16;
        constexpr int CHUNKS = FIRST_HALF / 16 < 1 ? 1 : FIRST_HALF / 16;   // chunks of 16 columns a warp finishes of a tile, at most
        constexpr int AHEAD = CHUNKS < 3 ? CHUNKS : 3;
        const int c_begin = warp >= 6 ? FIRST_HALF : 0;
        const int c_limit = warp >= 6 ? BN : FIRST_HALF;
        uint32_t local = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++local) {
            DD_ITEM_COORDS(item)
            (void)n_kblocks; (void)w0; (void)x0;
            const uint32_t acc = local & 1;
            const int row = a0 + quarter * 32 + lane;      // this thread's token (BY_TOKEN) or output feature
            const bool row_ok = row < rows_a;
            // the bias of this thread's feature is a weight: it is on its way before the accumulator is waited for
            const float feature_bias = (!BY_TOKEN && row_ok && p.bias) ? __ldg(p.bias + row) : 0.f;
            // Tiles of tokens: the bias of the tile's features goes to shared memory, and the first chunks of this thread's
            // piece of the residual row into registers, while the MMAs of the tile still run (see the two-SM kernel).
            float* bias_tile = bias_s[local & 1];
            float res_ahead[AHEAD][16];
            if (BY_TOKEN && p.splits == 1) {
                const int f = (int)threadIdx.x - 64;
                if (f < BN) bias_tile[f] = (p.bias && b0 + f < p.N) ? __ldg(p.bias + b0 + f) : 0.f;
                if (p.residual) {
#pragma unroll
                    for (int ci = 0; ci < AHEAD; ++ci) {
                        const int c0 = c_begin + ci * 16;
                        if (row_ok && c0 < c_limit && b0 + c0 < rows_b) load_residual_row16(p, row, b0 + c0, res_ahead[ci]);
                    }
                }
            }
            if (!tc::mbar_wait(&tmem_full_bar[acc], (local >> 1) & 1, abort_flag)) *epilogue_abort = 1;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (*epilogue_abort) break;                   // the same decision in all eight warps
            tc::fence_after_sync();
            const uint32_t lane_addr = tmem_base + acc * C::ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            if (c_begin >= c_limit || b0 + c_begin >= rows_b) {      // no columns for this warp in this tile
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&tmem_empty_bar[acc]);
            }
            if (BY_TOKEN && p.splits == 1 && p.residual) {
#pragma unroll
                for (int ci = 0; ci < CHUNKS; ++ci) {
                    const int c0 = c_begin + ci * 16;
                    if (c0 >= c_limit || b0 + c0 >= rows_b) break;
                    uint32_t r[16];
                    tc::tmem_ld_x16(lane_addr + c0, r);
                    float bias16[16];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float4 b4 = *reinterpret_cast<const float4*>(bias_tile + c0 + 4 * q);
                        bias16[4 * q] = b4.x; bias16[4 * q + 1] = b4.y; bias16[4 * q + 2] = b4.z; bias16[4 * q + 3] = b4.w;
                    }
                    tc::tmem_ld_wait();
                    if (c0 + 16 >= c_limit || b0 + c0 + 16 >= rows_b) {  // this warp's last read of the accumulator
                        tc::fence_before_sync();
                        __syncwarp();
                        if (lane == 0) tc::mbar_arrive(&tmem_empty_bar[acc]);
                    }
                    if (row_ok) store_out_row16(p, row, b0 + c0, r, res_ahead[ci % AHEAD], bias16);
                    const int c_next = c0 + AHEAD * 16;
                    if (ci + AHEAD < CHUNKS && row_ok && c_next < c_limit && b0 + c_next < rows_b)
                        load_residual_row16(p, row, b0 + c_next, res_ahead[ci % AHEAD]);
                }
            } else if (p.splits == 1) {
                for (int c0 = c_begin; c0 < c_limit && b0 + c0 < rows_b; c0 += 16) {
                    uint32_t r[16];
                    tc::tmem_ld_x16(lane_addr + c0, r);
                    float res[16], bias16[16];
                    if (row_ok) {                                        // in flight while the accumulator is read
                        if (BY_TOKEN) {                                  // no residual on this path
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const float4 b4 = *reinterpret_cast<const float4*>(bias_tile + c0 + 4 * q);
                                bias16[4 * q] = b4.x; bias16[4 * q + 1] = b4.y; bias16[4 * q + 2] = b4.z; bias16[4 * q + 3] = b4.w;
                            }
                        } else load_residual16(p, b0 + c0, row, res);
                    }
                    tc::tmem_ld_wait();
                    if (c0 + 16 >= c_limit || b0 + c0 + 16 >= rows_b) {  // this warp's last read of the accumulator
                        tc::fence_before_sync();
                        __syncwarp();
                        if (lane == 0) tc::mbar_arrive(&tmem_empty_bar[acc]);
                    }
                    if (row_ok) {
                        if (BY_TOKEN) store_out_row16(p, row, b0 + c0, r, res, bias16);
                        else {
                            float accv[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) accv[j] = __uint_as_float(r[j]);
                            store_out16(p, b0 + c0, row, accv, res, feature_bias);
                        }
                    }
                }
            } else if (!BY_TOKEN) {
                // partial sums to the workspace, then the last block of this tile reduces
                const int n = row, m0 = b0;
                float* ws = p.workspace + (size_t)split * p.M * p.N;
                for (int c0 = c_begin; c0 < c_limit && m0 + c0 < p.M; c0 += 16) {
                    uint32_t r[16];
                    tc::tmem_ld_x16(lane_addr + c0, r);
                    tc::tmem_ld_wait();
                    if (c0 + 16 >= c_limit || m0 + c0 + 16 >= p.M) {
                        tc::fence_before_sync();
                        __syncwarp();
                        if (lane == 0) tc::mbar_arrive(&tmem_empty_bar[acc]);
                    }
                    if (row_ok) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int m = m0 + c0 + j;
                            if (m < p.M) ws[(size_t)m * p.N + n] = __uint_as_float(r[j]);
                        }
                    }
                }
                __threadfence();
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    const int prev = atomicAdd(&p.counters[tile], 1);
                    *last_flag = (prev == p.splits - 1) ? 1 : 0;
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");
                const bool last = *last_flag != 0;
                if (last) {
                    __threadfence();
                    if (row_ok) {
                        // 16 tokens at a time, so that 16 independent loads are in flight; splits are added in
                        // ascending order (deterministic)
                        for (int c0 = c_begin; c0 < c_limit && m0 + c0 < p.M; c0 += 16) {
                            float v[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) v[j] = 0.f;
                            for (int s0 = 0; s0 < p.splits; ++s0) {
                                const float* src = p.workspace + ((size_t)s0 * p.M + m0 + c0) * p.N + n;
                                float t[16];
#pragma unroll
                                for (int j = 0; j < 16; ++j) t[j] = m0 + c0 + j < p.M ? __ldcg(src + (size_t)j * p.N) : 0.f;
#pragma unroll
                                for (int j = 0; j < 16; ++j) v[j] += t[j];
                            }
                            store_out16(p, m0 + c0, n, v);
                        }
                    }
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");        // last_flag is reused by the next item
                if (last && warp == 2 && lane == 0) p.counters[tile] = 0;
            }
        }
    }
#undef DD_ITEM_COORDS

    tc::fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicOr(p.error_flag, 8);
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// Two SMs on one tile (tcgen05 cta_group::2), for steps of many tokens: a cluster of two blocks owns 256 tokens
// x BN output features. Each block loads its own 128 token rows and its own half of the BN weight rows with TMA,
// all bytes counted on the leader's barrier; the leader (rank 0) issues tcgen05.mma.cta_group::2, which reads both
// blocks' shared memory and leaves each block the 128 x BN accumulator of its own tokens in its own TMEM;
// tcgen05.commit with a cluster mask frees the stages and publishes the accumulator in both blocks. Per block and
// k-block this moves 16 KB + BN/2 x 128 B for a 128 x BN x 64 product: less L2-to-SM traffic per flop than the
// one-SM tile, which at 2,048 tokens is what bounds it.
template <int BN> struct PairConfig {
    static constexpr int HALF = BN / 2;
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = HALF * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = BN >= 256 ? 6 : (BN >= 192 ? 7 : 8);
    static constexpr int ACC_COLS = BN == 192 ? 256 : BN;
    static constexpr int TMEM_COLS = 2 * ACC_COLS;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

template <int BN>
__global__ void __launch_bounds__(THREADS_P, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                         const GemmParams p) {
    using C = PairConfig<BN>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(16) float bias_s[2][256];        // the bias of a tile's features, tiles alternating
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + C::STAGES * C::STAGE_BYTES);   // used in the leader only
    uint64_t* empty_bar = full_bar + C::STAGES;
    uint64_t* tmem_full_bar = empty_bar + C::STAGES;      // [2]
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;         // [2] used in the leader only: 8 epilogue warps arrive
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* epilogue_abort = const_cast<int*>(abort_flag) + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = tc::cluster_rank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int tiles_a = (p.M + 2 * BM - 1) / (2 * BM);     // along the tokens, 256 per pair
    const int tiles_b = (p.N + BN - 1) / BN;               // along the output features
    const int n_items = tiles_a * tiles_b;
    const int n_kblocks = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            tc::mbar_init(&full_bar[s], 1);
            tc::mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            tc::mbar_init(&tmem_full_bar[a], 1);
            tc::mbar_init(&tmem_empty_bar[a], 2 * EPI_WARPS);
        }
        *abort_flag = 0;
        *epilogue_abort = 0;
        tc::fence_barrier_init();
        tc::fence_proxy_async();
    }
    if (warp == 1) {
        tc::tmem_alloc_pair(tmem_slot, C::TMEM_COLS);
        tc::tmem_relinquish_pair();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::cluster_arrive();
    tc::cluster_wait();                  // the other block's barriers exist before anything signals them
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    dd_launch_dependents();

#define DD_PAIR_COORDS(item)                                     \
    const int a0 = ((item) % tiles_a) * 2 * BM + (int)rank * BM; \
    const int b0 = ((item) / tiles_a) * BN;

    if (warp == 0) {
        if (tc::elect_one()) {
            tc::prefetch_tensormap(&map_w);
            tc::prefetch_tensormap(&map_x);
            // Weights do not depend on the kernel before this one: the weight halves of the first tile's first stages
            // are on their way before the wait; the activations follow after it.
            int ahead = 0;
            if (pair < n_items) {
                const int b_first = (pair / tiles_a) * BN;
                ahead = min(n_kblocks, C::STAGES);
                for (int i = 0; i < ahead; ++i) {
                    if (rank == 0) tc::mbar_expect_tx(&full_bar[i], 2 * C::STAGE_BYTES);     // both blocks' bytes
                    tc::tma_load_2d_pair(tiles + i * C::STAGE_BYTES + C::A_BYTES, &map_w, i * BK, b_first + (int)rank * C::HALF,
                                         tc::map_to_rank(&full_bar[i], 0));
                }
            }
            dd_grid_wait();
            uint32_t it = 0;
            bool ok = true;
            for (int item = pair; item < n_items && ok; item += n_pairs) {
                DD_PAIR_COORDS(item)
                for (int i = 0; i < n_kblocks; ++i, ++it) {
                    const int s = it % C::STAGES;
                    uint8_t* a_dst = tiles + s * C::STAGE_BYTES;
                    uint8_t* b_dst = a_dst + C::A_BYTES;
                    const uint32_t leader_full = tc::map_to_rank(&full_bar[s], 0);
                    if ((int)it < ahead) {                 // the weight half of this stage is already on its way
                        tc::tma_load_2d_pair(a_dst, &map_x, i * BK, a0, leader_full);
                        continue;
                    }
                    if (!tc::mbar_wait(&empty_bar[s], ((it / C::STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    if (rank == 0) tc::mbar_expect_tx(&full_bar[s], 2 * C::STAGE_BYTES);     // both blocks' bytes
                    tc::tma_load_2d_pair(a_dst, &map_x, i * BK, a0, leader_full);
                    tc::tma_load_2d_pair(b_dst, &map_w, i * BK, b0 + (int)rank * C::HALF, leader_full);
                }
            }
        }
    } else if (warp == 1) {
        if (rank == 0 && tc::elect_one()) {
            constexpr uint32_t idesc = tc::idesc_bf16_f32(2 * BM, BN);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int item = pair; item < n_items && ok; item += n_pairs, ++local) {
                const uint32_t acc = local & 1;
                if (!tc::mbar_wait(&tmem_empty_bar[acc], ((local >> 1) & 1) ^ 1, abort_flag)) break;
                tc::fence_after_sync();
                const uint32_t tmem_d = tmem_base + acc * C::ACC_COLS;
                for (int i = 0; i < n_kblocks; ++i, ++it) {
                    const int s = it % C::STAGES;
                    if (!tc::mbar_wait(&full_bar[s], (it / C::STAGES) & 1, abort_flag)) { ok = false; break; }
                    tc::fence_after_sync();
                    const uint32_t a_addr = tc::smem_u32(tiles + s * C::STAGE_BYTES);
                    const uint32_t b_addr = a_addr + C::A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        tc::mma_bf16_pair(tmem_d, tc::smem_desc_sw128(a_addr + k * UMMA_K * 2),
                                          tc::smem_desc_sw128(b_addr + k * UMMA_K * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
                    tc::mma_commit_pair(&empty_bar[s], 3);            // the stage is free in both blocks
                }
                if (ok) tc::mma_commit_pair(&tmem_full_bar[acc], 3);   // both halves of the accumulator are complete
            }
        }
    } else {
        dd_grid_wait();
        const int quarter = warp & 3;
        // the two warps of a lane quarter split the tile's features in halves (in chunks of 16)
        constexpr int FIRST_HALF = ((BN / 16 + 1) / 2) * 16;
        constexpr int CHUNKS = FIRST_HALF / 16;       // chunks of 16 features a warp finishes of a tile, at most
        constexpr int AHEAD = CHUNKS < 3 ? CHUNKS : 3;
        const int c_begin = warp >= 6 ? FIRST_HALF : 0;
        const int c_limit = warp >= 6 ? BN : FIRST_HALF;
        uint32_t local = 0;
        for (int item = pair; item < n_items; item += n_pairs, ++local) {
            DD_PAIR_COORDS(item)
            const uint32_t acc = local & 1;
            const int m = a0 + quarter * 32 + lane;
            const bool m_ok = m < p.M;
            // The bias of the tile's features is a weight: the eight warps put it into shared memory while the MMAs run
            // (a chunk that asked L2 for it just before it was needed waited for the answer, six or eight times a tile).
            float* bias_tile = bias_s[local & 1];
            {
                const int f = (int)threadIdx.x - 64;
                if (f < BN) bias_tile[f] = (p.bias && b0 + f < p.N) ? __ldg(p.bias + b0 + f) : 0.f;
            }
            // The residual is an earlier kernel's data (or an earlier tile's own rows elsewhere): the first AHEAD chunks of
            // this thread's piece of its row are asked for now, while the MMAs of the tile still run, and each later
            // chunk while the chunk AHEAD before it is finished; read chunk by chunk when the accumulator is there, a
            // warp paid a trip to memory six or eight times a tile.
            float res[AHEAD][16];
            if (p.residual) {
#pragma unroll
                for (int ci = 0; ci < AHEAD; ++ci) {
                    const int c0 = c_begin + ci * 16;
                    if (m_ok && c0 < c_limit && b0 + c0 < p.N) load_residual_row16(p, m, b0 + c0, res[ci]);
                }
            }
            if (!tc::mbar_wait(&tmem_full_bar[acc], (local >> 1) & 1, abort_flag)) *epilogue_abort = 1;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (*epilogue_abort) break;
            tc::fence_after_sync();
            const uint32_t lane_addr = tmem_base + acc * C::ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            if (b0 + c_begin >= p.N) {                                 // no features for this warp in this tile
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive_cluster(tc::map_to_rank(&tmem_empty_bar[acc], 0));
            }
            if (p.residual) {
#pragma unroll
                for (int ci = 0; ci < CHUNKS; ++ci) {
                    const int c0 = c_begin + ci * 16;
                    if (c0 >= c_limit || b0 + c0 >= p.N) break;
                    uint32_t r[16];
                    tc::tmem_ld_x16(lane_addr + c0, r);
                    float bias16[16];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float4 b4 = *reinterpret_cast<const float4*>(bias_tile + c0 + 4 * q);
                        bias16[4 * q] = b4.x; bias16[4 * q + 1] = b4.y; bias16[4 * q + 2] = b4.z; bias16[4 * q + 3] = b4.w;
                    }
                    tc::tmem_ld_wait();
                    if (c0 + 16 >= c_limit || b0 + c0 + 16 >= p.N) {      // this warp's last read: hand it back to the leader
                        tc::fence_before_sync();
                        __syncwarp();
                        if (lane == 0) tc::mbar_arrive_cluster(tc::map_to_rank(&tmem_empty_bar[acc], 0));
                    }
                    if (m_ok) store_out_row16(p, m, b0 + c0, r, res[ci % AHEAD], bias16);
                    // the residual of the chunk AHEAD further on, into the registers this chunk has just given up
                    const int c_next = c0 + AHEAD * 16;
                    if (ci + AHEAD < CHUNKS && m_ok && c_next < c_limit && b0 + c_next < p.N)
                        load_residual_row16(p, m, b0 + c_next, res[ci % AHEAD]);
                }
            } else {
                for (int c0 = c_begin; c0 < c_limit && b0 + c0 < p.N; c0 += 16) {
                    uint32_t r[16];
                    tc::tmem_ld_x16(lane_addr + c0, r);
                    float bias16[16];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float4 b4 = *reinterpret_cast<const float4*>(bias_tile + c0 + 4 * q);
                        bias16[4 * q] = b4.x; bias16[4 * q + 1] = b4.y; bias16[4 * q + 2] = b4.z; bias16[4 * q + 3] = b4.w;
                    }
                    tc::tmem_ld_wait();
                    if (c0 + 16 >= c_limit || b0 + c0 + 16 >= p.N) {      // this warp's last read: hand it back to the leader
                        tc::fence_before_sync();
                        __syncwarp();
                        if (lane == 0) tc::mbar_arrive_cluster(tc::map_to_rank(&tmem_empty_bar[acc], 0));
                    }
                    if (m_ok) store_out_row16(p, m, b0 + c0, r, bias16, bias16);    // no residual: the second argument is not read
                }
            }
        }
    }
#undef DD_PAIR_COORDS
    __syncwarp();
    tc::fence_before_sync();
    tc::cluster_arrive();
    tc::cluster_wait();                  // neither block leaves while the other may still read its tiles or signal its barriers
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicOr(p.error_flag, 8);
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
    }
}

// Split-K inside a thread-block cluster, for a handful of tokens: the S blocks of a cluster share one
// output tile and each streams 1/S of K, so that ~150 blocks pull a weight matrix that has only a few
// dozen tiles, and with at most STAGES k-blocks per block the whole weight slice is requested before
// the preceding kernel has even finished. The partial tiles are reduced over distributed shared
// memory: block r owns every S-th slice of the tile's 128 features; each block writes, for every
// feature, its partial row of BN tokens into the owner's shared memory (st.shared::cluster), one
// cluster barrier later the owner adds the S partials in rank order (deterministic) and applies the
// epilogue. No global workspace, no counters, no second pass through L2.
template <int BN, bool DEEP>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_cluster_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                            const GemmParams p) {
    using C = ClusterConfig<BN, DEEP>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + C::STAGES;
    uint64_t* tmem_full_bar = empty_bar + C::STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // partial tiles sent to this block: [source rank][feature of my slice][BN tokens], the 16-byte pieces of a
    // feature's row swizzled by the feature (reduce_swizzle) so that eight neighbouring features' pieces lie in
    // different banks, for the remote writes as for the reads below
    float* reduce_buf = reinterpret_cast<float*>(tiles + C::STAGES * C::STAGE_BYTES + 256);

    dd_launch_dependents();      // the next kernel may begin its own set-up (and ask for its weights) at once
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = (int)tc::cluster_size();
    const int rank = (int)tc::cluster_rank();
    const int slice = (BM + S - 1) / S;                   // features each block reduces
    const int tiles_n = (p.N + BM - 1) / BM;
    const int tile = blockIdx.x / S;
    const int n0 = (tile % tiles_n) * BM;
    const int m0 = (tile / tiles_n) * BN;
    const int total_kblocks = (p.K + BK - 1) / BK;
    const int kb_begin = rank * p.kblocks_per_split;
    const int n_kblocks = max(0, min(total_kblocks, kb_begin + p.kblocks_per_split) - kb_begin);

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            tc::mbar_init(&full_bar[s], 1);
            tc::mbar_init(&empty_bar[s], 1);
        }
        tc::mbar_init(tmem_full_bar, 1);
        *abort_flag = 0;
        tc::fence_barrier_init();
        tc::fence_proxy_async();
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, C::TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    tc::cluster_arrive();        // "my shared memory exists": waited for before the first remote write

    if (warp == 0) {
        if (tc::elect_one()) {
            tc::prefetch_tensormap(&map_w);
            tc::prefetch_tensormap(&map_x);
            // weights first: they do not depend on the kernel before this one
            const int ahead = min(n_kblocks, C::STAGES);
            for (int i = 0; i < ahead; ++i) {
                tc::mbar_expect_tx(&full_bar[i], C::STAGE_BYTES);
                tc::tma_load_2d(tiles + i * C::STAGE_BYTES, &map_w, (kb_begin + i) * BK, n0, &full_bar[i]);
            }
            prefetch_share(p);
            dd_grid_wait();
            for (int i = 0; i < n_kblocks; ++i) {
                const int s = i % C::STAGES;
                uint8_t* a_dst = tiles + s * C::STAGE_BYTES;
                uint8_t* b_dst = a_dst + C::A_BYTES;
                if (i < ahead) {
                    tc::tma_load_2d(b_dst, &map_x, (kb_begin + i) * BK, m0, &full_bar[s]);
                    continue;
                }
                const uint32_t phase = (i / C::STAGES) & 1;
                if (!tc::mbar_wait(&empty_bar[s], phase ^ 1, abort_flag)) break;
                tc::mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
                tc::tma_load_2d(a_dst, &map_w, (kb_begin + i) * BK, n0, &full_bar[s]);
                tc::tma_load_2d(b_dst, &map_x, (kb_begin + i) * BK, m0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        if (tc::elect_one()) {
            constexpr uint32_t idesc = tc::idesc_bf16_f32(BM, BN);
            bool ok = true;
            for (int i = 0; i < n_kblocks; ++i) {
                const int s = i % C::STAGES;
                const uint32_t phase = (i / C::STAGES) & 1;
                if (!tc::mbar_wait(&full_bar[s], phase, abort_flag)) { ok = false; break; }
                tc::fence_after_sync();
                const uint32_t a_addr = tc::smem_u32(tiles + s * C::STAGE_BYTES);
                const uint32_t b_addr = a_addr + C::A_BYTES;
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    const uint64_t da = tc::smem_desc_sw128(a_addr + k * UMMA_K * 2);
                    const uint64_t db = tc::smem_desc_sw128(b_addr + k * UMMA_K * 2);
                    tc::mma_bf16(tmem_base, da, db, idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                tc::mma_commit(&empty_bar[s]);
            }
            if (ok) tc::mma_commit(tmem_full_bar);
        }
    }
    __syncwarp();
    tc::cluster_wait();          // every block of the cluster is up: remote shared memory may be written

    // The bias of the features this block will finish is a weight: it is fetched into shared memory now, while the
    // weights stream, instead of costing a trip to L2 at the very end of the block.
    float* bias_s = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(reduce_buf) + C::REDUCE_BYTES);
    if (warp >= 2) {
        const int quarter = warp & 3;
        const int f = quarter * 32 + lane;                // feature of the tile this thread holds in TMEM
        {
            const int n = n0 + rank * slice + f;
            bias_s[f] = (p.bias && f < slice && n < p.N) ? __ldg(p.bias + n) : 0.f;
        }
        const bool have = n_kblocks > 0 && tc::mbar_wait(tmem_full_bar, 0, abort_flag);
        tc::fence_after_sync();
        const int owner = f / slice, lf = f - owner * slice;
        // my partial row of feature f (BN tokens) goes to the block that owns f, 16 bytes a store
        const uint32_t remote = tc::map_to_rank(reduce_buf + ((size_t)rank * slice + lf) * BN, (uint32_t)owner);
        const int sw = reduce_swizzle<BN>(lf);
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += 16) {
            uint32_t r[16];
            if (have) { tc::tmem_ld_x16(lane_addr + c0, r); tc::tmem_ld_wait(); }
            else {
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = 0;    // a block without k-blocks (or one that gave up) adds zeros
            }
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (m0 + c0 + 4 * q < p.M)                // pieces beyond the last token are never read
                    tc::st_cluster_f32x4(remote + (uint32_t)(((c0 / 4 + q) ^ sw) * 16), r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
        }
    }
    __syncwarp();
    tc::cluster_arrive();
    tc::cluster_wait();          // all partial rows have landed

    if (warp >= 2) {
        dd_grid_wait();          // residual is an earlier kernel's data
        const int tid = threadIdx.x - 64;                 // 0..127
        const int first_feature = rank * slice;
        const int my_features = max(0, min(slice, BM - first_feature));
        // A thread finishes four consecutive tokens of one feature at a time (neighbouring threads, neighbouring
        // features): their residual values (the output itself, as a rule, so no load may be moved across a store by
        // the compiler) are requested before the partial rows are summed; one after the other, each cost a trip to L2.
        constexpr int CHUNKS = BN / 4;
        const int items = my_features * min(CHUNKS, (p.M - m0 + 3) / 4);      // only pieces that hold a token
        for (int item = tid; item < items; item += 128) {
            const int lf = item % my_features, c = item / my_features;
            const int n = n0 + first_feature + lf, m = m0 + 4 * c;
            float res[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                res[j] = (p.residual && n < p.N && m + j < p.M) ? p.residual[(size_t)(m + j) * p.ldr + n] : 0.f;
            const float* mine = reduce_buf + (size_t)lf * BN + 4 * (c ^ reduce_swizzle<BN>(lf));
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < S; ++r) {
                const float4 a = *reinterpret_cast<const float4*>(mine + (size_t)r * slice * BN);
                v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
            }
            if (n >= p.N) continue;
            const float u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (m + j >= p.M) break;
                const float y = activation_for(u[j] + bias_s[lf], p.act, p.out_dtype) + res[j];
                if (p.out_dtype == DD_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)(m + j) * p.ldo + n] = __float2bfloat16_rn(y);
                else reinterpret_cast<float*>(p.out)[(size_t)(m + j) * p.ldo + n] = y;
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicOr(p.error_flag, 8);
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(sym);
    }
    return fn;
}

// rows x K bf16 matrix with row stride ld elements; boxes of box_rows x 64, 128-byte swizzle
int make_map(CUtensorMap* map, const void* base, int rows, int K, int ld, int box_rows, const char* what) {
    EncodeTiled enc = encode_fn();
    if (!enc) return dd_fail("dd_gemm_tcgen05: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return dd_fail("dd_gemm_tcgen05: cannot describe %s to TMA (driver error %d)", what, (int)r);
    return 0;
}

// ma: the operand on the 128 accumulator lanes (the weights, or the tokens for BN >= 128); mb: the other one
template <int BN>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, cudaStream_t s) {
    using C = Config<BN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return dd_fail("dd_gemm_tcgen05: shared memory of %d bytes refused: %s", C::SMEM_BYTES, cudaGetErrorString(e));
        configured = true;
    }
    const int items = (C::BY_TOKEN ? dd_ceil_div(p.M, BM) * dd_ceil_div(p.N, BN) : dd_ceil_div(p.N, BM) * dd_ceil_div(p.M, BN)) * p.splits;
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 148;
    }
    dd_launch(gemm_tcgen05_kernel<BN>, dim3(items < sm_count ? items : sm_count), dim3(THREADS_P), C::SMEM_BYTES, s, ma, mb, p);
    return dd_check_launch("dd_gemm_tcgen05");
}

template <int BN, bool DEEP = false>
int launch_cluster(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, cudaStream_t s) {
    using C = ClusterConfig<BN, DEEP>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_cluster_kernel<BN, DEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return dd_fail("dd_gemm_tcgen05: shared memory of %d bytes refused: %s", C::SMEM_BYTES, cudaGetErrorString(e));
        e = cudaFuncSetAttribute(gemm_tcgen05_cluster_kernel<BN, DEEP>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return dd_fail("dd_gemm_tcgen05: clusters of more than 8 blocks refused: %s", cudaGetErrorString(e));
        configured = true;
    }
    const int tiles = dd_ceil_div(p.N, BM) * dd_ceil_div(p.M, BN);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(tiles * p.splits);
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = C::SMEM_BYTES;
    config.stream = s;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = p.splits;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attrs;
    config.numAttrs = dd_pdl_enabled ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&config, gemm_tcgen05_cluster_kernel<BN, DEEP>, mw, mx, p);
    if (e != cudaSuccess) return dd_fail("dd_gemm_tcgen05 (cluster of %d): %s", p.splits, cudaGetErrorString(e));
    return dd_check_launch("dd_gemm_tcgen05");
}

template <int BN>
int launch_pair(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, cudaStream_t s) {
    using C = PairConfig<BN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return dd_fail("dd_gemm_tcgen05: shared memory of %d bytes refused: %s", C::SMEM_BYTES, cudaGetErrorString(e));
        configured = true;
    }
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 148;
    }
    const int items = dd_ceil_div(p.M, 2 * BM) * dd_ceil_div(p.N, BN);
    const int pairs = items < sm_count / 2 ? items : sm_count / 2;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * pairs);
    config.blockDim = dim3(THREADS_P);
    config.dynamicSmemBytes = C::SMEM_BYTES;
    config.stream = s;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = 2;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attrs;
    config.numAttrs = dd_pdl_enabled ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&config, gemm_tcgen05_pair_kernel<BN>, mw, mx, p);
    if (e != cudaSuccess) return dd_fail("dd_gemm_tcgen05 (two SMs per tile): %s", cudaGetErrorString(e));
    return dd_check_launch("dd_gemm_tcgen05");
}

}  // namespace


// Chooses the token tile, the K split and how the split is reduced (*cluster = 1: inside a thread-block
// cluster over distributed shared memory; 0: through a global workspace). Returns splits (>= 1).
DD_API int dd_gemm_tcgen05_plan(int M, int N, int K, int sm_count, int* token_tile, int* cluster) {
    // Up to 64 tokens the tile is 128 features x 16, 32 or 64 tokens. Above, it is 128 tokens x 128, 192 or 256
    // features (the value returned in *token_tile is then the feature width).
    const int kblocks = dd_ceil_div(K, BK);
    const bool long_k = kblocks > 32;                 // more than 2,048: worth splitting even for 17 to 64 tokens
    int bn = 128;
    // 33 to 64 tokens: two tiles of 32 tokens double the blocks, which pays while the feature tiles alone do not fill the
    // GPU; a matrix with more feature tiles than SMs (the LM head) would only be streamed twice (55 against 33 us)
    const bool many_tiles = dd_ceil_div(N, BM) >= sm_count;
    if (M <= 16) bn = 16; else if (M <= 32) bn = 32; else if (M <= 64) bn = (long_k || many_tiles) ? 64 : 32;
    else {
        // Tiles of 128 tokens x c features on one SM, or of 256 tokens x c features on a pair of SMs (less L2
        // traffic per flop). A round of one tile per SM was measured to take about as long as c + 64 columns
        // (2,048 and 4,096 tokens, 1600 to 6400 features), so the choice minimises rounds x (c + 64); ties go to
        // the pair and to the wider tile.
        long long best = -1;
        bool pair = false;
        // Up to a few hundred tokens the tiles of 128 features x 32 or 64 tokens can still cover the output in one
        // round, and a round of them is shorter (1600 features, 256 tokens: 7.5 us in 32-token tiles, 12.7 us in
        // tiles of 128 tokens x 128 features); the same cost, rounds x (columns + 64), orders them.
        for (int c = 32; c <= 64; c += 32) {
            const long long t = (long long)dd_ceil_div(N, BM) * dd_ceil_div(M, c);
            const long long cost = (long long)dd_ceil_div(t, sm_count) * (c + 64);
            if (best < 0 || cost < best) { best = cost; bn = c; }
        }
        const int candidates[3] = {128, 192, 256};
        for (int two = 0; two <= ((cluster != nullptr && sm_count >= 2) ? 1 : 0); ++two) {
            const int rows = two ? 2 * BM : BM, units = two ? sm_count / 2 : sm_count;
            for (int i = 0; i < 3; ++i) {
                const int c = candidates[i];
                const long long t = (long long)dd_ceil_div(M, rows) * dd_ceil_div(N, c);
                const long long cost = (long long)dd_ceil_div(t, units) * (c + 64);
                if (best < 0 || cost <= best) { best = cost; bn = c; pair = two != 0; }
            }
        }
        if (token_tile) *token_tile = bn;
        if (cluster) *cluster = pair ? 2 : 0;
        return 1;
    }
    // 17 to 64 tokens and a short K: tiles of 16 tokens in clusters, if about 1.35 blocks per SM (and no more than 1.45)
    // leave every tile at least two splits. Measured at 32 tokens: 1600 x 1600 takes 4.7 us in 26 tiles x 5 splits
    // against 7.1 us unsplit in tiles of 32 tokens, 6400 x 1600 7.8 against 8.4 us; with more blocks than that the
    // clusters come in two waves (4800 x 1600 at 48 tokens: 8.0 us in 114 tiles x 2 against 7.6 us unsplit).
    int mid_splits = 0;
    if (M > 16 && !long_k && cluster) {
        const int t16 = dd_ceil_div(N, BM) * dd_ceil_div(M, 16);
        int s = (sm_count * 27 / 20 + t16 / 2) / t16;
        while (s >= 2 && t16 * s > sm_count * 29 / 20) --s;
        if (s > kblocks / 2) s = kblocks / 2;
        if (s >= 2) {
            mid_splits = s;
            bn = 16;
        }
    }
    if (token_tile) *token_tile = bn;
    if (cluster) *cluster = 0;
    if (mid_splits) {
        *cluster = 1;
        return mid_splits;
    }
    const int tiles = dd_ceil_div(N, BM) * dd_ceil_div(M, bn);
    // A step of a few tokens has a few dozen tiles at most: split K inside clusters so that about as many
    // blocks as there are SMs stream the weights, all in one wave (a cluster must be resident as a whole).
    // From 17 tokens on the reduction of the wider tiles costs more than the split saves unless K is long: measured
    // at 64 tokens and K = 1600, 1600 features take 13.4 us split eightfold and 7.3 us unsplit in tiles of 32 tokens
    // (6400 features: 9.9 against 8.8 us); with K = 6400 the eightfold split stays ahead (12.5 against 18.8 us).
    int splits = 1;
    if (M <= 64 && tiles * 2 <= sm_count && (M <= 16 || (long_k && (M <= 32 || tiles <= 16)))) {
        // Up to 16 tokens the rings are 5 stages deep, so two blocks fit on an SM and the next GEMM's blocks can ask for
        // their weights beside this one's: about 1.35 blocks per SM measured best (4800 features: 5 or 6 splits 6.3 us,
        // 3 splits 7.0; 6400 features: 4 splits 6.8, 2 splits 8.5; more than two blocks per SM: 10.7 and more).
        splits = bn == 16 ? (sm_count * 27 / 20 + tiles / 2) / tiles : sm_count / tiles;
        // clusters of up to 16 blocks exist, but beyond 8 the wider tiles lose (6400 -> 1600 at 32 tokens: 7.2 us in 8
        // splits, 12.7 in 10), and the tiles of 16 tokens gain little beyond 12 (1600 x 1600 at 8 tokens: 4.25 us in 7
        // splits, 4.1 in 9; 6400 -> 1600: 7.0 in 8, 6.8 in 10 to 12, 7.1 in 16)
        const int most = bn == 16 ? 12 : 8;
        if (splits > most) splits = most;
        if (bn == 16 && cluster && tiles * 8 <= sm_count) {
            // A narrow product (1600 features: 13 tiles): one block per SM with a ring of 10 stages, clusters of at most 8
            // (two of them fit a GPC), at least 5 k-blocks a block. Measured at 8 tokens: 1600 x 1600 3.7 us in 5 splits
            // against 4.1 us in 9 splits of 5-stage rings; 6400 -> 1600 6.6 us in 8 splits against 6.9 us in 12.
            const int deep = kblocks / 5 < 8 ? kblocks / 5 : 8;
            if (deep >= 2) {
                *cluster = 3;
                return deep;
            }
        }
        if (splits > kblocks / 2) splits = kblocks / 2;
        if (splits < 1) splits = 1;
        if (splits > 1 && cluster) *cluster = 1;
    }
    return splits;
}

// X [M,K] bf16 (row stride ldx), W [N,K] bf16 (row stride ldw); bias [N] f32 or null; residual [M,N] f32
// (row stride ldr, may alias out) or null; out [M,N] bf16 or f32 (row stride ldo). token_tile 16/32/64: tiles
// of 128 features x token_tile tokens; 128/192/256: tiles of 128 tokens x token_tile features, no K split.
// cluster = 1: splits (at most 16) are the blocks of a cluster and reduce over distributed shared memory
// (token_tile <= 64); cluster = 3: the same with rings of 10 stages and one block per SM (token_tile 16); cluster = 2: two SMs per tile of 256 tokens x token_tile features (tcgen05
// cta_group::2), token_tile 128/192/256; cluster = 0 with splits > 1 (token_tile <= 64): workspace f32
// [splits*M*N] and counters int32 [tiles], zero before the first launch. prefetch/prefetch_bytes: null/0, or memory that a later kernel streams once (the next
// weight matrix of a decode step): this kernel's blocks ask L2 to fetch it while they run.
DD_API int dd_gemm_tcgen05(const void* X, int ldx, const void* W, int ldw, const float* bias, const float* residual,
                           int ldr, void* out, int ldo, int M, int N, int K, int act, int out_dtype, int splits,
                           int token_tile, int cluster, float* workspace, int* counters, int n_counters,
                           const void* prefetch, long long prefetch_bytes, int* error_flag, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ldx % 8 || ldw % 8)
        return dd_fail("dd_gemm_tcgen05: K=%d and the row strides (%d, %d) must be multiples of 8 (TMA needs 16-byte rows)", K, ldx, ldw);
    if (((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return dd_fail("dd_gemm_tcgen05: operands must be 16-byte aligned");
    if (out_dtype != DD_BF16 && out_dtype != DD_F32) return dd_fail("dd_gemm_tcgen05: unknown output dtype %d", out_dtype);
    const int kblocks = dd_ceil_div(K, BK);
    if (splits < 1 || splits > kblocks) return dd_fail("dd_gemm_tcgen05: bad split count %d for %d k-blocks", splits, kblocks);
    if (cluster == 3 && token_tile != 16) return dd_fail("dd_gemm_tcgen05: the deep rings are for token tiles of 16 (got %d)", token_tile);
    if ((cluster == 1 || cluster == 3) && (splits > 16 || token_tile > 64))
        return dd_fail("dd_gemm_tcgen05: a cluster has at most 16 blocks and a token tile of at most 64 (got %d, %d)", splits, token_tile);
    if (cluster == 2 && (splits != 1 || (token_tile != 128 && token_tile != 192 && token_tile != 256)))
        return dd_fail("dd_gemm_tcgen05: two SMs per tile take no K split and a token tile of 128, 192 or 256 (got %d, %d)", splits, token_tile);
    GemmParams p;
    p.bias = bias; p.residual = residual; p.out = out; p.workspace = workspace; p.counters = counters;
    p.error_flag = error_flag; p.M = M; p.N = N; p.K = K; p.ldr = ldr; p.ldo = ldo; p.act = act; p.out_dtype = out_dtype;
    p.prefetch = (const uint8_t*)prefetch;
    p.prefetch_bytes = (prefetch && prefetch_bytes > 0 && !((uintptr_t)prefetch & 15)) ? (unsigned long long)prefetch_bytes : 0;
    p.splits = splits; p.kblocks_per_split = dd_ceil_div(kblocks, splits);
    p.splits = dd_ceil_div(kblocks, p.kblocks_per_split);     // no empty split
    if (p.splits == 1 && (cluster == 1 || cluster == 3)) cluster = 0;
    if (p.splits > 1 && !cluster) {
        const int tiles = dd_ceil_div(N, BM) * dd_ceil_div(M, token_tile);
        if (!workspace || !counters || n_counters < tiles)
            return dd_fail("dd_gemm_tcgen05: split-K needs a workspace and %d counters", tiles);
    }
    // 16-byte accesses in the epilogue of the 128-token tiles: every row of out, residual and bias must allow them
    const int out_elem = out_dtype == DD_BF16 ? 2 : 4;
    p.vec = !((uintptr_t)out & 15) && ((size_t)ldo * out_elem) % 16 == 0 &&
            (!residual || (!((uintptr_t)residual & 15) && ldr % 4 == 0)) && (!bias || !((uintptr_t)bias & 15));
    const bool by_token = token_tile >= 128;       // 128 tokens x token_tile features per tile
    if (by_token && p.splits > 1)
        return dd_fail("dd_gemm_tcgen05: tiles of 128 tokens take no K split (got %d splits with tile %d)", p.splits, token_tile);
    CUtensorMap mw, mx;
    const int w_box = by_token ? (cluster == 2 ? token_tile / 2 : token_tile) : BM;
    const int x_box = by_token ? BM : token_tile;
    if (int e = make_map(&mw, W, N, K, ldw, w_box, "the weight matrix")) return e;
    if (int e = make_map(&mx, X, M, K, ldx, x_box, "the activations")) return e;
    cudaStream_t s = (cudaStream_t)stream;
    if (cluster == 2) {
        switch (token_tile) {
            case 128: return launch_pair<128>(mw, mx, p, s);
            case 192: return launch_pair<192>(mw, mx, p, s);
            case 256: return launch_pair<256>(mw, mx, p, s);
        }
    }
    if (cluster == 3) return launch_cluster<16, true>(mw, mx, p, s);
    if (cluster) {
        switch (token_tile) {
            case 16: return launch_cluster<16>(mw, mx, p, s);
            case 32: return launch_cluster<32>(mw, mx, p, s);
            case 64: return launch_cluster<64>(mw, mx, p, s);
        }
        return dd_fail("dd_gemm_tcgen05: token tile %d is not one of 16, 32, 64 for a cluster", token_tile);
    }
    switch (token_tile) {
        case 16: return launch<16>(mw, mx, p, s);
        case 32: return launch<32>(mw, mx, p, s);
        case 64: return launch<64>(mw, mx, p, s);
        case 128: return launch<128>(mx, mw, p, s);
        case 192: return launch<192>(mx, mw, p, s);
        case 256: return launch<256>(mx, mw, p, s);
    }
    return dd_fail("dd_gemm_tcgen05: token tile %d is not one of 16, 32, 64, 128, 192, 256", token_tile);
}
