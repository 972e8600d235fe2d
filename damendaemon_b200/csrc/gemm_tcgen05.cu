// bfloat16 GEMM on the 5th-generation tensor cores: out[M,N] = act(X[M,K] . W[N,K]^T + bias) (+ residual).
//
// The product is computed transposed, D^T = W . X^T: the weight rows (output features)
// are the 128-row M side of tcgen05.mma and the tokens its N side (16..256), so the same
// kernel serves a decode step of a few tokens (narrow N tile, split over K to fill the
// SMs while the weights stream from HBM once) and a prompt portion of thousands (N tile
// 256). In TMEM the accumulator has one output feature per lane and one token per
// column; an epilogue thread therefore owns one feature, its bias is one register, and a
// warp's 32 lanes write 32 consecutive features of a token row: coalesced stores with no
// staging through shared memory.
//
// The kernel is persistent: at most one CTA per SM walks over (tile, split) work items, the TMA
// producer runs ahead across items, and the accumulator is double buffered in TMEM so that the
// epilogue of one tile overlaps the MMAs of the next.
//
// Pipeline per CTA: warp 0 issues TMA loads (W tile 128x64 and X tile BNx64 bf16, 128-byte
// swizzle) into a ring of stages guarded by full/empty mbarriers; warp 1 allocates TMEM
// and issues tcgen05.mma from shared-memory descriptors, releasing stages with
// tcgen05.commit; warps 2-5 read the accumulator with tcgen05.ld and apply the epilogue.
// With split-K each CTA writes its float32 partial tile to a workspace; the CTA that
// arrives last at the tile's counter sums the partials in split order (deterministic) and
// applies the epilogue, then resets the counter for the next launch.
//
// Every mbarrier wait is bounded (tcgen05.cuh); on a timeout the kernel sets bit 8 of the
// error word, stops waiting everywhere, frees its TMEM and returns.
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128;          // output features per tile (tcgen05.mma M)
constexpr int BK = 64;           // k elements per stage: one 128-byte swizzle row of bf16
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;     // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue

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
    const uint8_t* prefetch;        // null, or memory a later kernel will stream (the next weight matrix):
    unsigned long long prefetch_bytes;   // every block asks L2 to fetch its share while this kernel runs
    unsigned long long* timeline;   // null, or 8 time stamps (ns) per block for looking at where a block's time goes
};

unsigned long long* g_timeline = nullptr;

template <int BN> struct Config {
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
template <int BN> struct ClusterConfig {
    // deep rings: with 5 stages (two blocks per SM, so that the next kernel's blocks could prefetch beside this
    // kernel's) every size measured 15-40% slower than with one block per SM and 8 stages
    static constexpr int STAGES = BN >= 64 ? 6 : 8;
    static constexpr int STAGE_BYTES = Config<BN>::STAGE_BYTES;
    static constexpr int A_BYTES = Config<BN>::A_BYTES;
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    static constexpr int REDUCE_BYTES = (BM + 8) * BN * 4;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + REDUCE_BYTES;
};

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
__device__ __forceinline__ void store_out16(const GemmParams& p, int m_first, int n, const float* acc, const float* r) {
    const float b = p.bias ? p.bias[n] : 0.f;
    if (p.act == DD_ACT_NONE) store16_o<DD_ACT_NONE>(p, m_first, n, acc, b, r);
    else if (p.act == DD_ACT_GELU_NEW) store16_o<DD_ACT_GELU_NEW>(p, m_first, n, acc, b, r);
    else store16_o<DD_ACT_GELU_ERF>(p, m_first, n, acc, b, r);
}

__device__ __forceinline__ void store_out16(const GemmParams& p, int m_first, int n, const float* acc) {
    float r[16];
    load_residual16(p, m_first, n, r);
    store_out16(p, m_first, n, acc, r);
}

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const GemmParams p) {
    using C = Config<BN>;
    extern __shared__ uint8_t smem_raw[];
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
    const int tiles_n = (p.N + BM - 1) / BM;              // tiles along the output features
    const int tiles_m = (p.M + BN - 1) / BN;              // tiles along the tokens
    const int n_items = tiles_n * tiles_m * p.splits;
    const int total_kblocks = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            tc::mbar_init(&full_bar[s], 1);
            tc::mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            tc::mbar_init(&tmem_full_bar[a], 1);
            tc::mbar_init(&tmem_empty_bar[a], 4);         // one arrival per epilogue warp
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

    // Work item -> (feature tile, token tile, split). Feature tiles vary fastest, so CTAs that run
    // side by side share the same token tile in L2.
#define DD_ITEM_COORDS(item)                                              \
    const int split = (item) % p.splits;                                  \
    const int tile = (item) / p.splits;                                   \
    const int n0 = (tile % tiles_n) * BM;                                 \
    const int m0 = (tile / tiles_n) * BN;                                 \
    const int kb_begin = split * p.kblocks_per_split;                     \
    const int n_kblocks = min(total_kblocks, kb_begin + p.kblocks_per_split) - kb_begin;

    if (warp == 0) {
        if (tc::elect_one()) {
            tc::prefetch_tensormap(&map_w);
            tc::prefetch_tensormap(&map_x);
            uint32_t it = 0;                               // k-blocks issued so far, across items
            bool ok = true;
            // Weights never change, so the weight tiles of the first stages are requested before the
            // kernel that produces the activations has finished; the activation tiles follow the wait.
            int ahead = 0;
            if (blockIdx.x < n_items) {
                DD_ITEM_COORDS(blockIdx.x)
                (void)m0;
                ahead = min(n_kblocks, C::STAGES);
                for (int i = 0; i < ahead; ++i) {
                    tc::mbar_expect_tx(&full_bar[i], C::STAGE_BYTES);
                    tc::tma_load_2d(tiles + i * C::STAGE_BYTES, &map_w, (kb_begin + i) * BK, n0, &full_bar[i]);
                }
            }
            prefetch_share(p);
            dd_grid_wait();
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                DD_ITEM_COORDS(item)
                for (int i = 0; i < n_kblocks; ++i, ++it) {
                    const int s = it % C::STAGES;
                    uint8_t* a_dst = tiles + s * C::STAGE_BYTES;
                    uint8_t* b_dst = a_dst + C::A_BYTES;
                    if ((int)it < ahead) {                 // the weight tile of this stage is already on its way
                        tc::tma_load_2d(b_dst, &map_x, (kb_begin + i) * BK, m0, &full_bar[s]);
                        continue;
                    }
                    const uint32_t phase = (it / C::STAGES) & 1;
                    if (!tc::mbar_wait(&empty_bar[s], phase ^ 1, abort_flag)) { ok = false; break; }
                    tc::mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
                    tc::tma_load_2d(a_dst, &map_w, (kb_begin + i) * BK, n0, &full_bar[s]);
                    tc::tma_load_2d(b_dst, &map_x, (kb_begin + i) * BK, m0, &full_bar[s]);
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
                (void)n0; (void)m0;
                const uint32_t acc = local & 1;
                // the epilogue must have drained this accumulator (passes at once the first two times)
                if (!tc::mbar_wait(&tmem_empty_bar[acc], ((local >> 1) & 1) ^ 1, abort_flag)) break;
                tc::fence_after_sync();
                if (p.timeline && local < 3) p.timeline[blockIdx.x * 16 + 1 + 4 * local] = tc::global_ns();
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
                if (p.timeline && local < 3) p.timeline[blockIdx.x * 16 + 2 + 4 * local] = tc::global_ns();
                if (ok) tc::mma_commit(&tmem_full_bar[acc]);   // the accumulator is complete
            }
        }
    } else {
        // epilogue: warp w may touch TMEM lanes 32*(w%4) .. 32*(w%4)+31
        if (p.timeline && threadIdx.x == 64) p.timeline[blockIdx.x * 16] = tc::global_ns();
        dd_grid_wait();              // bias is constant, but residual, workspace and counters are earlier kernels' data
        const int quarter = warp & 3;
        uint32_t local = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++local) {
            DD_ITEM_COORDS(item)
            (void)n_kblocks;
            const uint32_t acc = local & 1;
            const int n = n0 + quarter * 32 + lane;
            const bool n_ok = n < p.N;
            if (!tc::mbar_wait(&tmem_full_bar[acc], (local >> 1) & 1, abort_flag)) *epilogue_abort = 1;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*epilogue_abort) break;                   // the same decision in all four warps
            tc::fence_after_sync();
            if (p.timeline && threadIdx.x == 64 && local < 3) p.timeline[blockIdx.x * 16 + 3 + 4 * local] = tc::global_ns();
            const uint32_t lane_addr = tmem_base + acc * C::ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            if (p.splits == 1) {
                for (int c0 = 0; c0 < BN && m0 + c0 < p.M; c0 += 16) {
                    uint32_t r[16];
                    tc::tmem_ld_x16(lane_addr + c0, r);
                    float res[16];
                    if (n_ok) load_residual16(p, m0 + c0, n, res);       // in flight while the accumulator is read
                    tc::tmem_ld_wait();
                    if (c0 + 16 >= BN || m0 + c0 + 16 >= p.M) {      // last read of this accumulator: hand it back
                        tc::fence_before_sync();
                        __syncwarp();
                        if (lane == 0) tc::mbar_arrive(&tmem_empty_bar[acc]);
                    }
                    if (n_ok) {
                        float accv[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) accv[j] = __uint_as_float(r[j]);
                        store_out16(p, m0 + c0, n, accv, res);
                    }
                }
                if (p.timeline && threadIdx.x == 64 && local < 3) p.timeline[blockIdx.x * 16 + 4 + 4 * local] = tc::global_ns();
            } else {
                // partial sums to the workspace, then the last CTA of this tile reduces
                float* ws = p.workspace + (size_t)split * p.M * p.N;
                for (int c0 = 0; c0 < BN && m0 + c0 < p.M; c0 += 16) {
                    uint32_t r[16];
                    tc::tmem_ld_x16(lane_addr + c0, r);
                    tc::tmem_ld_wait();
                    if (c0 + 16 >= BN || m0 + c0 + 16 >= p.M) {
                        tc::fence_before_sync();
                        __syncwarp();
                        if (lane == 0) tc::mbar_arrive(&tmem_empty_bar[acc]);
                    }
                    if (n_ok) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int m = m0 + c0 + j;
                            if (m < p.M) ws[(size_t)m * p.N + n] = __uint_as_float(r[j]);
                        }
                    }
                }
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    const int prev = atomicAdd(&p.counters[tile], 1);
                    *last_flag = (prev == p.splits - 1) ? 1 : 0;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const bool last = *last_flag != 0;
                if (last) {
                    __threadfence();
                    if (n_ok) {
                        // 16 tokens at a time, so that 16 independent loads are in flight for every split
                        for (int c0 = 0; c0 < BN && m0 + c0 < p.M; c0 += 16) {
                            float v[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) v[j] = 0.f;
                            // splits are added in ascending order (deterministic), two splits' loads in flight at once
                            for (int s0 = 0; s0 < p.splits; s0 += 2) {
                                float t[2][16];
#pragma unroll
                                for (int u = 0; u < 2; ++u) {
                                    const float* src = p.workspace + ((size_t)(s0 + u) * p.M + m0 + c0) * p.N + n;
#pragma unroll
                                    for (int j = 0; j < 16; ++j)
                                        t[u][j] = (s0 + u < p.splits && m0 + c0 + j < p.M) ? __ldcg(src + (size_t)j * p.N) : 0.f;
                                }
#pragma unroll
                                for (int u = 0; u < 2; ++u)
#pragma unroll
                                    for (int j = 0; j < 16; ++j) v[j] += t[u][j];
                            }
                            store_out16(p, m0 + c0, n, v);
                        }
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");        // last_flag is reused by the next item
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

// Two SMs on one tile (tcgen05 cta_group::2), for steps of many tokens: a cluster of two blocks owns 256 output
// features x BN tokens. Each block loads its own 128 weight rows and its own half of the token rows with TMA, all
// bytes counted on the leader's barrier; the leader (rank 0) issues tcgen05.mma.cta_group::2, which reads both
// blocks' shared memory and leaves each block its 128 x BN half of the accumulator in its own TMEM; tcgen05.commit
// with a cluster mask frees the stages and publishes the accumulator in both blocks. Per block and k-block this
// moves 16 KB + BN/2 x 128 B for a 128 x BN x 64 product: half the L2-to-SM traffic per flop of the one-SM tile.
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
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                         const GemmParams p) {
    using C = PairConfig<BN>;
    extern __shared__ uint8_t smem_raw[];
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
    const int tiles_n = (p.N + 2 * BM - 1) / (2 * BM);
    const int tiles_m = (p.M + BN - 1) / BN;
    const int n_items = tiles_n * tiles_m;
    const int n_kblocks = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            tc::mbar_init(&full_bar[s], 1);
            tc::mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            tc::mbar_init(&tmem_full_bar[a], 1);
            tc::mbar_init(&tmem_empty_bar[a], 8);
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
    const int n0 = ((item) % tiles_n) * 2 * BM + (int)rank * BM; \
    const int m0 = ((item) / tiles_n) * BN;

    if (warp == 0) {
        if (tc::elect_one()) {
            tc::prefetch_tensormap(&map_w);
            tc::prefetch_tensormap(&map_x);
            dd_grid_wait();
            uint32_t it = 0;
            bool ok = true;
            for (int item = pair; item < n_items && ok; item += n_pairs) {
                DD_PAIR_COORDS(item)
                for (int i = 0; i < n_kblocks; ++i, ++it) {
                    const int s = it % C::STAGES;
                    if (!tc::mbar_wait(&empty_bar[s], ((it / C::STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* a_dst = tiles + s * C::STAGE_BYTES;
                    uint8_t* b_dst = a_dst + C::A_BYTES;
                    if (rank == 0) tc::mbar_expect_tx(&full_bar[s], 2 * C::STAGE_BYTES);     // both blocks' bytes
                    const uint32_t leader_full = tc::map_to_rank(&full_bar[s], 0);
                    tc::tma_load_2d_pair(a_dst, &map_w, i * BK, n0, leader_full);
                    tc::tma_load_2d_pair(b_dst, &map_x, i * BK, m0 + (int)rank * C::HALF, leader_full);
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
        uint32_t local = 0;
        for (int item = pair; item < n_items; item += n_pairs, ++local) {
            DD_PAIR_COORDS(item)
            const uint32_t acc = local & 1;
            const int n = n0 + quarter * 32 + lane;
            const bool n_ok = n < p.N;
            if (!tc::mbar_wait(&tmem_full_bar[acc], (local >> 1) & 1, abort_flag)) *epilogue_abort = 1;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*epilogue_abort) break;
            tc::fence_after_sync();
            const uint32_t lane_addr = tmem_base + acc * C::ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            for (int c0 = 0; c0 < BN && m0 + c0 < p.M; c0 += 16) {
                uint32_t r[16];
                tc::tmem_ld_x16(lane_addr + c0, r);
                tc::tmem_ld_wait();
                if (c0 + 16 >= BN || m0 + c0 + 16 >= p.M) {           // last read: hand the accumulator back to the leader
                    tc::fence_before_sync();
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive_cluster(tc::map_to_rank(&tmem_empty_bar[acc], 0));
                }
                if (n_ok) {
                    float accv[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) accv[j] = __uint_as_float(r[j]);
                    store_out16(p, m0 + c0, n, accv);
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
template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_cluster_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                            const GemmParams p) {
    using C = ClusterConfig<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + C::STAGES;
    uint64_t* tmem_full_bar = empty_bar + C::STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // partial tiles sent to this block: [source rank][BN tokens][features of my slice]; neighbouring threads hold
    // neighbouring features, so both the remote writes and the reads below walk consecutive banks
    float* reduce_buf = reinterpret_cast<float*>(tiles + C::STAGES * C::STAGE_BYTES + 256);

    if (p.timeline && threadIdx.x == 0) p.timeline[blockIdx.x * 8 + 0] = tc::global_ns();
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
    if (p.timeline && threadIdx.x == 0) p.timeline[blockIdx.x * 8 + 1] = tc::global_ns();
    dd_launch_dependents();
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
            if (p.timeline) p.timeline[blockIdx.x * 8 + 2] = tc::global_ns();
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
                if (p.timeline && i == 0) p.timeline[blockIdx.x * 8 + 3] = tc::global_ns();
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
            if (p.timeline) p.timeline[blockIdx.x * 8 + 4] = tc::global_ns();
            if (ok) tc::mma_commit(tmem_full_bar);
        }
    }
    __syncwarp();
    tc::cluster_wait();          // every block of the cluster is up: remote shared memory may be written

    if (warp >= 2) {
        const int quarter = warp & 3;
        const int f = quarter * 32 + lane;                // feature of the tile this thread holds in TMEM
        const bool have = n_kblocks > 0 && tc::mbar_wait(tmem_full_bar, 0, abort_flag);
        tc::fence_after_sync();
        if (p.timeline && threadIdx.x == 64) p.timeline[blockIdx.x * 8 + 5] = tc::global_ns();
        const int owner = f / slice, lf = f - owner * slice;
        // my partial row of feature f goes to the block that owns f
        const uint32_t remote = tc::map_to_rank(reduce_buf + (size_t)rank * BN * slice + lf, (uint32_t)owner);
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
            for (int j = 0; j < 16; ++j) tc::st_cluster_f32(remote + (uint32_t)((c0 + j) * slice) * 4, __uint_as_float(r[j]));
        }
    }
    __syncwarp();
    tc::cluster_arrive();
    tc::cluster_wait();          // all partial rows have landed
    if (p.timeline && threadIdx.x == 64) p.timeline[blockIdx.x * 8 + 6] = tc::global_ns();

    if (warp >= 2) {
        dd_grid_wait();          // residual is an earlier kernel's data
        const int tid = threadIdx.x - 64;                 // 0..127
        const int first_feature = rank * slice;
        const int my_features = max(0, min(slice, BM - first_feature));
        for (int idx = tid; idx < my_features * BN; idx += 128) {
            const int lf = idx % my_features, tok = idx / my_features;     // neighbouring threads, neighbouring features
            const int n = n0 + first_feature + lf, m = m0 + tok;
            if (n >= p.N || m >= p.M) continue;
            float v = 0.f;
            for (int r = 0; r < S; ++r) v += reduce_buf[((size_t)r * BN + tok) * slice + lf];
            if (p.bias) v += p.bias[n];
            v = activation_for(v, p.act, p.out_dtype);
            if (p.residual) v += p.residual[(size_t)m * p.ldr + n];
            if (p.out_dtype == DD_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.ldo + n] = __float2bfloat16_rn(v);
            else reinterpret_cast<float*>(p.out)[(size_t)m * p.ldo + n] = v;
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (p.timeline && threadIdx.x == 0) p.timeline[blockIdx.x * 8 + 7] = tc::global_ns();
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

template <int BN>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, cudaStream_t s) {
    using C = Config<BN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return dd_fail("dd_gemm_tcgen05: shared memory of %d bytes refused: %s", C::SMEM_BYTES, cudaGetErrorString(e));
        configured = true;
    }
    const int items = dd_ceil_div(p.N, BM) * dd_ceil_div(p.M, BN) * p.splits;
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 148;
    }
    dd_launch(gemm_tcgen05_kernel<BN>, dim3(items < sm_count ? items : sm_count), dim3(THREADS), C::SMEM_BYTES, s, mw, mx, p);
    return dd_check_launch("dd_gemm_tcgen05");
}

template <int BN>
int launch_cluster(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, cudaStream_t s) {
    using C = ClusterConfig<BN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_cluster_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return dd_fail("dd_gemm_tcgen05: shared memory of %d bytes refused: %s", C::SMEM_BYTES, cudaGetErrorString(e));
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
    cudaError_t e = cudaLaunchKernelEx(&config, gemm_tcgen05_cluster_kernel<BN>, mw, mx, p);
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
    const int items = dd_ceil_div(p.N, 2 * BM) * dd_ceil_div(p.M, BN);
    const int pairs = items < sm_count / 2 ? items : sm_count / 2;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * pairs);
    config.blockDim = dim3(THREADS);
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

// Debugging aid: a device buffer of time stamps (ns) that the kernels fill, null switches it off: 8 per block from
// the cluster kernel; 16 per block from the persistent kernel (0 start, then for the first three tiles: MMAs begin,
// MMAs issued, epilogue begins, epilogue done).
DD_API void dd_gemm_tcgen05_timeline(unsigned long long* buffer) { g_timeline = buffer; }

// Chooses the token tile, the K split and how the split is reduced (*cluster = 1: inside a thread-block
// cluster over distributed shared memory; 0: through a global workspace). Returns splits (>= 1).
DD_API int dd_gemm_tcgen05_plan(int M, int N, int K, int sm_count, int* token_tile, int* cluster) {
    // Above 64 tokens: the tile among 128, 192 and 256 tokens that needs the least time in whole rounds of one tile
    // per SM (rounds x tokens per tile); ties go to the smaller tile, which balances better.
    int bn = 128;
    if (M <= 16) bn = 16; else if (M <= 32) bn = 32; else if (M <= 64) bn = 64;
    else {
        // Wide outputs (measured at 4800 and 6400 features: 5-10% faster) go to two SMs per 256-feature tile;
        // with 1600 features the 256-feature tiles waste an eighth of their rows and the one-SM kernel wins.
        const bool pair = N >= 2048 && cluster != nullptr;
        const int rows = pair ? 2 * BM : BM, units = pair ? sm_count / 2 : sm_count;
        long long best = -1;
        const int candidates[3] = {128, 192, 256};
        for (int i = 0; i < 3; ++i) {
            const int c = candidates[i];
            const long long t = (long long)dd_ceil_div(N, rows) * dd_ceil_div(M, c);
            const long long cost = (long long)dd_ceil_div(t, units) * c;
            if (best < 0 || cost < best) { best = cost; bn = c; }
        }
        if (token_tile) *token_tile = bn;
        if (cluster) *cluster = pair ? 2 : 0;
        return 1;
    }
    if (token_tile) *token_tile = bn;
    if (cluster) *cluster = 0;
    const int tiles = dd_ceil_div(N, BM) * dd_ceil_div(M, bn);
    const int kblocks = dd_ceil_div(K, BK);
    // A step of a few tokens has a few dozen tiles at most: split K inside clusters so that about as many
    // blocks as there are SMs stream the weights, all in one wave (a cluster must be resident as a whole).
    // Above 32 tokens the reduction of a wide tile costs more than the split saves unless the tiles are very few
    // (measured at 64 tokens: 4800 and 6400 features faster unsplit, 1600 features faster split).
    int splits = 1;
    if (M <= 64 && tiles * 2 <= sm_count && (M <= 32 || tiles <= 16)) {
        splits = sm_count / tiles;       // fewer, so that two kernels' blocks could sit side by side, measured slower
        if (splits > 8) splits = 8;
        if (splits > kblocks / 2) splits = kblocks / 2;
        if (splits < 1) splits = 1;
        if (splits > 1 && cluster) *cluster = 1;
    }
    return splits;
}

// X [M,K] bf16 (row stride ldx), W [N,K] bf16 (row stride ldw); bias [N] f32 or null; residual [M,N] f32
// (row stride ldr, may alias out) or null; out [M,N] bf16 or f32 (row stride ldo). cluster = 1: splits
// (at most 8) are the blocks of a cluster and reduce over distributed shared memory (token_tile <= 64);
// cluster = 2: two SMs per 256-feature tile (tcgen05 cta_group::2), token_tile 128/192/256, no split;
// cluster = 0 with splits > 1: workspace f32 [splits*M*N] and counters int32 [tiles], zero before the
// first launch. prefetch/prefetch_bytes: null/0, or memory that a later kernel streams once (the next
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
    if (cluster == 1 && (splits > 8 || token_tile > 64))
        return dd_fail("dd_gemm_tcgen05: a cluster has at most 8 blocks and a token tile of at most 64 (got %d, %d)", splits, token_tile);
    if (cluster == 2 && (splits != 1 || (token_tile != 128 && token_tile != 192 && token_tile != 256)))
        return dd_fail("dd_gemm_tcgen05: two SMs per tile take no K split and a token tile of 128, 192 or 256 (got %d, %d)", splits, token_tile);
    GemmParams p;
    p.bias = bias; p.residual = residual; p.out = out; p.workspace = workspace; p.counters = counters;
    p.error_flag = error_flag; p.M = M; p.N = N; p.K = K; p.ldr = ldr; p.ldo = ldo; p.act = act; p.out_dtype = out_dtype;
    p.timeline = g_timeline;
    p.prefetch = (const uint8_t*)prefetch;
    p.prefetch_bytes = (prefetch && prefetch_bytes > 0 && !((uintptr_t)prefetch & 15)) ? (unsigned long long)prefetch_bytes : 0;
    p.splits = splits; p.kblocks_per_split = dd_ceil_div(kblocks, splits);
    p.splits = dd_ceil_div(kblocks, p.kblocks_per_split);     // no empty split
    if (p.splits == 1 && cluster == 1) cluster = 0;
    if (p.splits > 1 && !cluster) {
        const int tiles = dd_ceil_div(N, BM) * dd_ceil_div(M, token_tile);
        if (!workspace || !counters || n_counters < tiles)
            return dd_fail("dd_gemm_tcgen05: split-K needs a workspace and %d counters", tiles);
    }
    CUtensorMap mw, mx;
    if (int e = make_map(&mw, W, N, K, ldw, BM, "the weight matrix")) return e;
    if (int e = make_map(&mx, X, M, K, ldx, cluster == 2 ? token_tile / 2 : token_tile, "the activations")) return e;
    cudaStream_t s = (cudaStream_t)stream;
    if (cluster == 2) {
        switch (token_tile) {
            case 128: return launch_pair<128>(mw, mx, p, s);
            case 192: return launch_pair<192>(mw, mx, p, s);
            case 256: return launch_pair<256>(mw, mx, p, s);
        }
    }
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
        case 128: return launch<128>(mw, mx, p, s);
        case 192: return launch<192>(mw, mx, p, s);
        case 256: return launch<256>(mw, mx, p, s);
    }
    return dd_fail("dd_gemm_tcgen05: token tile %d is not one of 16, 32, 64, 128, 192, 256", token_tile);
}
