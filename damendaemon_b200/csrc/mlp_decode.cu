// The whole feed-forward of a decode step in ONE kernel, for up to 16 tokens:
//     x += W_down . act(W_up . LayerNorm(x) + b_up) + b_down
// Three launches (norm, up projection, down projection) become one, and the down projection's
// weights stream into shared memory while the up projection is still being reduced: on a step of a
// few tokens every launch is a chain of latencies (set-up, first bytes from HBM, drain) that the
// amount of work cannot hide, so fewer, longer kernels are what makes such a step faster.
//
// Measured on a B200 at GPT-2 XL sizes it is SLOWER than the three kernels it replaces (28 us against 17 us
// for 8 tokens), so the engine does not take it unless asked (Runtime.fuse): every block reads the same 51 KB
// of residual rows for the statistics and the same partial tiles for the second operand, and a hundred
// blocks hitting the same few L2 slices at once wait on each other (statistics 4 us, second operand 14 us in
// the per-block timeline). It stays as a tested starting point for a kernel that shares those reads.
//
// One block per SM, all resident at once, because the two halves are separated by a grid-wide
// barrier (an atomic counter, spun on with a time limit). Work item = (tile of 128 output features,
// K split); the splits of the up projection store float32 partial tiles that the down projection's
// operand preparation adds up (in split order, so this half is deterministic), applies bias and
// activation to and writes as the bf16 K-major operand; the splits of the down projection add
// straight into the float32 residual stream with atomics (their order, and so the last bit of the
// sum, may differ from run to run).
//
// Roles per block: warp 0 streams weight tiles with TMA through one ring of stages that runs across
// both halves (it never touches activations, so it does not wait for the preceding kernel); warp 1
// issues tcgen05.mma (A = weight tile, B = the activation operand in shared memory, written by the
// block itself in the 128-byte-swizzled K-major layout, N = 16 tokens); warps 2-5 compute the
// LayerNorm statistics of all rows, prepare both operands, read the accumulators from TMEM and run
// the barrier.
#include "common.cuh"
#include "tcgen05.cuh"

namespace {
constexpr int BM = 128, BK = 64, BN = 16, UMMA_K = 16;
constexpr int THREADS = 192, WORKERS = 128;
constexpr int STAGES = 8;
constexpr int A_BYTES = BM * BK * 2;          // one weight tile
constexpr int X_TILE_BYTES = BN * BK * 2;     // one k-block of the activation operand
constexpr int MAX_KB = 16;                    // k-blocks per work item at most
constexpr int SMEM_BYTES = STAGES * A_BYTES + MAX_KB * X_TILE_BYTES + 1024 + 1024;

struct MlpParams {
    float* x;                 // [M, width] float32 residual stream, updated in place
    int ldx;
    const float* gamma;       // LayerNorm weight [width]
    const float* beta;        // LayerNorm bias [width] or null
    float eps;
    const float* b_up;        // [inner] or null
    const float* b_down;      // [width] or null
    float* partial;           // [up_splits, 16, inner] float32 scratch
    int* sync;                // [2] zero before the first launch; left zero
    int* error_flag;
    int M, width, inner, act;
    int up_tiles, up_splits, up_kb;        // tiles of 128 features, K splits, k-blocks per split
    int down_tiles, down_splits, down_kb;
    unsigned long long* timeline;          // null, or 12 time stamps (ns) per block (debugging aid)
};

unsigned long long* g_mlp_timeline = nullptr;
#define DD_STAMP(i) do { if (p.timeline && (threadIdx.x == 64)) p.timeline[blockIdx.x * 12 + (i)] = tc::global_ns(); } while (0)

__device__ __forceinline__ void worker_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// 8 consecutive k (one 16-byte chunk) of token row r at chunk index ch of k-block kb
__device__ __forceinline__ uint8_t* operand_chunk(uint8_t* xbuf, int kb, int r, int ch) {
    return xbuf + kb * X_TILE_BYTES + r * 128 + ((ch ^ (r & 7)) << 4);
}

__global__ void __launch_bounds__(THREADS, 1)
mlp_decode_kernel(const __grid_constant__ CUtensorMap map_up, const __grid_constant__ CUtensorMap map_down,
                  const MlpParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* xbuf = tiles + STAGES * A_BYTES;                         // 1024-aligned
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(xbuf + MAX_KB * X_TILE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* x_ready = empty_bar + STAGES;          // [2] the operand of half h is in shared memory
    uint64_t* acc_ready = x_ready + 2;               // [2] the accumulator of half h is complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* stats = reinterpret_cast<float*>(tmem_slot + 4);           // [16 rows][mean, rstd]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x, G = gridDim.x;
    const int up_items = p.up_tiles * p.up_splits, down_items = p.down_tiles * p.down_splits;
    const bool has_up = cta < up_items, has_down = cta < down_items;
    const int up_tile = cta / p.up_splits, up_split = cta % p.up_splits;
    const int down_tile = cta / p.down_splits, down_split = cta % p.down_splits;
    const int up_total = (p.width + BK - 1) / BK, down_total = (p.inner + BK - 1) / BK;
    const int up_begin = up_split * p.up_kb, down_begin = down_split * p.down_kb;
    const int n_up = has_up ? max(0, min(up_total, up_begin + p.up_kb) - up_begin) : 0;
    const int n_down = has_down ? max(0, min(down_total, down_begin + p.down_kb) - down_begin) : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full_bar[s], 1);
            tc::mbar_init(&empty_bar[s], 1);
        }
        for (int h = 0; h < 2; ++h) {
            tc::mbar_init(&x_ready[h], 1);
            tc::mbar_init(&acc_ready[h], 1);
        }
        *abort_flag = 0;
        tc::fence_barrier_init();
        tc::fence_proxy_async();
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, 32);
        tc::tmem_relinquish();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    dd_launch_dependents();

    if (warp == 0) {
        if (tc::elect_one()) {
            tc::prefetch_tensormap(&map_up);
            tc::prefetch_tensormap(&map_down);
            // one ring across both halves; weights only, so no wait for the preceding kernel
            for (int it = 0; it < n_up + n_down; ++it) {
                const int s = it % STAGES;
                if (it >= STAGES && !tc::mbar_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1, abort_flag)) break;
                tc::mbar_expect_tx(&full_bar[s], A_BYTES);
                if (it < n_up) tc::tma_load_2d(tiles + s * A_BYTES, &map_up, (up_begin + it) * BK, up_tile * BM, &full_bar[s]);
                else tc::tma_load_2d(tiles + s * A_BYTES, &map_down, (down_begin + it - n_up) * BK, down_tile * BM, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        if (tc::elect_one()) {
            constexpr uint32_t idesc = tc::idesc_bf16_f32(BM, BN);
            int it = 0;
            bool ok = true;
            for (int half = 0; half < 2 && ok; ++half) {
                const int n = half == 0 ? n_up : n_down;
                if (n == 0) continue;
                if (!tc::mbar_wait(&x_ready[half], 0, abort_flag)) break;
                tc::fence_after_sync();
                const uint32_t tmem_d = tmem_base + half * BN;
                for (int i = 0; i < n; ++i, ++it) {
                    const int s = it % STAGES;
                    if (!tc::mbar_wait(&full_bar[s], (it / STAGES) & 1, abort_flag)) { ok = false; break; }
                    tc::fence_after_sync();
                    const uint32_t a_addr = tc::smem_u32(tiles + s * A_BYTES);
                    const uint32_t b_addr = tc::smem_u32(xbuf + i * X_TILE_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        tc::mma_bf16(tmem_d, tc::smem_desc_sw128(a_addr + k * UMMA_K * 2),
                                     tc::smem_desc_sw128(b_addr + k * UMMA_K * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
                    tc::mma_commit(&empty_bar[s]);
                }
                if (ok) tc::mma_commit(&acc_ready[half]);
            }
        }
    } else {
        const int tid = threadIdx.x - 64, wq = warp & 3;         // worker index 0..127; TMEM lane quarter
        DD_STAMP(0);
        dd_grid_wait();
        DD_STAMP(1);                                           // x is the preceding kernel's output
        // LayerNorm statistics of all rows (every block with an up item computes them itself: M x width floats from
        // L2). One sweep with many loads in flight: sums of (x - pivot) and (x - pivot)^2, pivot = the row's first
        // element, so that a large mean does not cancel against the mean of squares.
        if (n_up > 0) {
            float* red = reinterpret_cast<float*>(xbuf);            // [4 warps][16 rows][2], free until the operand is written
            const bool vec = p.width % 4 == 0 && p.ldx % 4 == 0 && !((uintptr_t)p.x & 15) && p.width <= 4 * 4 * WORKERS;
            for (int r0 = 0; r0 < p.M; r0 += 4) {
                // four rows at a time, 16 loads of 16 bytes in flight per thread
                float s1[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f}, pivot[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) pivot[u] = r0 + u < p.M ? p.x[(size_t)(r0 + u) * p.ldx] : 0.f;
                if (vec) {
                    const int n4 = p.width >> 2;
                    float4 v[4][4];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int c = tid + k * WORKERS;
                            v[u][k] = (r0 + u < p.M && c < n4) ? reinterpret_cast<const float4*>(p.x + (size_t)(r0 + u) * p.ldx)[c]
                                                                : make_float4(pivot[u], pivot[u], pivot[u], pivot[u]);
                        }
#pragma unroll
                    for (int u = 0; u < 4; ++u)
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const float a = v[u][k].x - pivot[u], b = v[u][k].y - pivot[u], c = v[u][k].z - pivot[u], d = v[u][k].w - pivot[u];
                            s1[u] += (a + b) + (c + d);
                            s2[u] += (a * a + b * b) + (c * c + d * d);
                        }
                } else {
                    for (int u = 0; u < 4 && r0 + u < p.M; ++u)
                        for (int c = tid; c < p.width; c += WORKERS) {
                            const float v = p.x[(size_t)(r0 + u) * p.ldx + c] - pivot[u];
                            s1[u] += v;
                            s2[u] = fmaf(v, v, s2[u]);
                        }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    s1[u] = dd_warp_sum(s1[u]);
                    s2[u] = dd_warp_sum(s2[u]);
                    if (lane == 0) { red[((warp - 2) * 16 + r0 + u) * 2] = s1[u]; red[((warp - 2) * 16 + r0 + u) * 2 + 1] = s2[u]; }
                }
            }
            worker_sync();
            if (tid < p.M) {
                float s1 = 0.f, s2 = 0.f;
#pragma unroll
                for (int w = 0; w < 4; ++w) { s1 += red[(w * 16 + tid) * 2]; s2 += red[(w * 16 + tid) * 2 + 1]; }
                const float pivot = p.x[(size_t)tid * p.ldx];
                const float inv = 1.0f / (float)p.width;
                const float d = s1 * inv;                           // mean - pivot
                stats[2 * tid] = pivot + d;
                stats[2 * tid + 1] = 1.0f / sqrtf(fmaxf(s2 * inv - d * d, 0.f) + p.eps);
            }
            worker_sync();
        }
        DD_STAMP(2);
        // operand of the up projection: LayerNorm(x)[:, my k range] as bf16, K-major, 128-byte swizzle
        if (n_up > 0) {
            const bool vec1 = p.width % 8 == 0 && !(((uintptr_t)p.x | (uintptr_t)p.gamma | (uintptr_t)p.beta) & 15) && p.ldx % 4 == 0;
            for (int idx0 = tid; idx0 < n_up * BN * 8; idx0 += WORKERS * 4) {
                // four chunks at a time: every load is issued before the first result is needed
                float4 xv[4][2], gv[4][2], bv[4][2];
                bool live[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int idx = idx0 + u * WORKERS;
                    const int ch = idx & 7, r = (idx >> 3) & 15, kb = idx >> 7;
                    const int c0 = (up_begin + kb) * BK + ch * 8;
                    live[u] = idx < n_up * BN * 8 && r < p.M && c0 < p.width;
                    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
                    xv[u][0] = xv[u][1] = gv[u][0] = gv[u][1] = bv[u][0] = bv[u][1] = z;
                    if (live[u]) {
                        const float* row = p.x + (size_t)r * p.ldx + c0;
                        if (vec1) {
                            xv[u][0] = *reinterpret_cast<const float4*>(row); xv[u][1] = *reinterpret_cast<const float4*>(row + 4);
                            gv[u][0] = *reinterpret_cast<const float4*>(p.gamma + c0); gv[u][1] = *reinterpret_cast<const float4*>(p.gamma + c0 + 4);
                            if (p.beta) { bv[u][0] = *reinterpret_cast<const float4*>(p.beta + c0); bv[u][1] = *reinterpret_cast<const float4*>(p.beta + c0 + 4); }
                        } else {
                            float* xs = reinterpret_cast<float*>(xv[u]); float* gs = reinterpret_cast<float*>(gv[u]); float* bs = reinterpret_cast<float*>(bv[u]);
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                if (c0 + j < p.width) { xs[j] = row[j]; gs[j] = p.gamma[c0 + j]; bs[j] = p.beta ? p.beta[c0 + j] : 0.f; }
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int idx = idx0 + u * WORKERS;
                    if (idx >= n_up * BN * 8) continue;
                    const int ch = idx & 7, r = (idx >> 3) & 15, kb = idx >> 7;
                    uint4 packed = make_uint4(0, 0, 0, 0);
                    if (live[u]) {
                        const float mean = stats[2 * r], rstd = stats[2 * r + 1];
                        const float* xs = reinterpret_cast<const float*>(xv[u]);
                        const float* gs = reinterpret_cast<const float*>(gv[u]);
                        const float* bs = reinterpret_cast<const float*>(bv[u]);
                        const int c0 = (up_begin + kb) * BK + ch * 8;
                        float y[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) y[j] = c0 + j < p.width ? (xs[j] - mean) * rstd * gs[j] + bs[j] : 0.f;
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(y[0], y[1]), h1 = __floats2bfloat162_rn(y[2], y[3]);
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(y[4], y[5]), h3 = __floats2bfloat162_rn(y[6], y[7]);
                        packed.x = *reinterpret_cast<uint32_t*>(&h0); packed.y = *reinterpret_cast<uint32_t*>(&h1);
                        packed.z = *reinterpret_cast<uint32_t*>(&h2); packed.w = *reinterpret_cast<uint32_t*>(&h3);
                    }
                    *reinterpret_cast<uint4*>(operand_chunk(xbuf, kb, r, ch)) = packed;
                }
            }
            tc::fence_proxy_async();                              // generic-proxy writes -> visible to the tensor core
            worker_sync();
            if (tid == 0) tc::mbar_arrive(&x_ready[0]);
            DD_STAMP(3);
            // partial tile of the up projection -> scratch [split][row][feature]
            const bool have = tc::mbar_wait(&acc_ready[0], 0, abort_flag);
            tc::fence_after_sync();
            DD_STAMP(4);
            if (have) {
                uint32_t r[16];
                tc::tmem_ld_x16(tmem_base + ((uint32_t)(wq * 32) << 16), r);
                tc::tmem_ld_wait();
                const int n = up_tile * BM + wq * 32 + lane;
                if (n < p.inner) {
                    float* dst = p.partial + (size_t)up_split * 16 * p.inner + n;
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (j < p.M) dst[(size_t)j * p.inner] = __uint_as_float(r[j]);
                }
            }
        }
        DD_STAMP(5);
        // grid-wide barrier: every block's partial tiles are in memory
        __threadfence();
        worker_sync();
        if (tid == 0) {
            atomicAdd(&p.sync[0], 1);
            const unsigned long long start = tc::global_ns();
            while (*reinterpret_cast<volatile int*>(&p.sync[0]) < G) {
                if (*abort_flag || tc::global_ns() - start > tc::WAIT_LIMIT_NS) { *abort_flag = 1; break; }
            }
            __threadfence();
        }
        worker_sync();
        DD_STAMP(6);
        if (n_down > 0 && !*abort_flag) {
            // operand of the down projection: act(sum of the up partials + bias)[:, my k range]
            const bool vec2 = p.up_splits <= 4;          // inner is a multiple of 8 and the scratch is 16-byte aligned
            for (int idx0 = tid; idx0 < n_down * BN * 8; idx0 += WORKERS * 4) {
                float4 pv[4][4][2];                       // [chunk][split][half]
                float4 biasv[4][2];
                bool live[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int idx = idx0 + u * WORKERS;
                    const int ch = idx & 7, r = (idx >> 3) & 15, kb = idx >> 7;
                    const int c0 = (down_begin + kb) * BK + ch * 8;
                    live[u] = idx < n_down * BN * 8 && r < p.M && c0 < p.inner;
                    biasv[u][0] = biasv[u][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (live[u] && p.b_up) {
                        if (!((uintptr_t)p.b_up & 15)) {
                            biasv[u][0] = *reinterpret_cast<const float4*>(p.b_up + c0);
                            biasv[u][1] = *reinterpret_cast<const float4*>(p.b_up + c0 + 4);
                        } else {
                            float* bs = reinterpret_cast<float*>(biasv[u]);
#pragma unroll
                            for (int j = 0; j < 8; ++j) bs[j] = p.b_up[c0 + j];
                        }
                    }
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
                        pv[u][s][0] = pv[u][s][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (vec2 && live[u] && s < p.up_splits) {
                            const float4* src = reinterpret_cast<const float4*>(p.partial + ((size_t)s * 16 + r) * p.inner + c0);
                            pv[u][s][0] = __ldcg(src);
                            pv[u][s][1] = __ldcg(src + 1);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int idx = idx0 + u * WORKERS;
                    if (idx >= n_down * BN * 8) continue;
                    const int ch = idx & 7, r = (idx >> 3) & 15, kb = idx >> 7;
                    const int c0 = (down_begin + kb) * BK + ch * 8;
                    uint4 packed = make_uint4(0, 0, 0, 0);
                    if (live[u]) {
                        float y[8];
                        const float* bs = reinterpret_cast<const float*>(biasv[u]);
#pragma unroll
                        for (int j = 0; j < 8; ++j) y[j] = bs[j];
                        if (vec2) {
#pragma unroll
                            for (int s = 0; s < 4; ++s) {          // splits in ascending order: deterministic
                                y[0] += pv[u][s][0].x; y[1] += pv[u][s][0].y; y[2] += pv[u][s][0].z; y[3] += pv[u][s][0].w;
                                y[4] += pv[u][s][1].x; y[5] += pv[u][s][1].y; y[6] += pv[u][s][1].z; y[7] += pv[u][s][1].w;
                            }
                        } else {
                            for (int s = 0; s < p.up_splits; ++s) {
                                const float* src = p.partial + ((size_t)s * 16 + r) * p.inner + c0;
#pragma unroll
                                for (int j = 0; j < 8; ++j) y[j] += __ldcg(src + j);
                            }
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            if (p.act == DD_ACT_GELU_NEW) {     // the result is rounded to bfloat16: the hardware tanh is exact enough
                                float t;
                                asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * (y[j] + 0.044715f * y[j] * y[j] * y[j])));
                                y[j] = 0.5f * y[j] * (1.0f + t);
                            } else y[j] = dd_activation(y[j], p.act);
                        }
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(y[0], y[1]), h1 = __floats2bfloat162_rn(y[2], y[3]);
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(y[4], y[5]), h3 = __floats2bfloat162_rn(y[6], y[7]);
                        packed.x = *reinterpret_cast<uint32_t*>(&h0); packed.y = *reinterpret_cast<uint32_t*>(&h1);
                        packed.z = *reinterpret_cast<uint32_t*>(&h2); packed.w = *reinterpret_cast<uint32_t*>(&h3);
                    }
                    *reinterpret_cast<uint4*>(operand_chunk(xbuf, kb, r, ch)) = packed;
                }
            }
            DD_STAMP(10);
            tc::fence_proxy_async();
            worker_sync();
            if (tid == 0) tc::mbar_arrive(&x_ready[1]);
            DD_STAMP(7);
            const bool have = tc::mbar_wait(&acc_ready[1], 0, abort_flag);
            tc::fence_after_sync();
            DD_STAMP(8);
            if (have) {
                uint32_t r[16];
                tc::tmem_ld_x16(tmem_base + BN + ((uint32_t)(wq * 32) << 16), r);
                tc::tmem_ld_wait();
                const int n = down_tile * BM + wq * 32 + lane;
                if (n < p.width) {
                    const float b = (down_split == 0 && p.b_down) ? p.b_down[n] : 0.f;
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (j < p.M) atomicAdd(p.x + (size_t)j * p.ldx + n, __uint_as_float(r[j]) + b);
                }
            }
        }
        DD_STAMP(9);
        // the last block out puts the barrier back to zero for the next launch
        __threadfence();
        worker_sync();
        if (tid == 0) {
            const int prev = atomicAdd(&p.sync[1], 1);
            if (prev == G - 1) { p.sync[0] = 0; p.sync[1] = 0; __threadfence(); }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicOr(p.error_flag, 8);
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, 32);
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int weight_map(CUtensorMap* map, const void* base, int rows, int K, int ld) {
    static EncodeTiled enc = nullptr;
    if (!enc) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            enc = reinterpret_cast<EncodeTiled>(sym);
    }
    if (!enc) return dd_fail("dd_mlp_decode: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)BM};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return dd_fail("dd_mlp_decode: cannot describe a weight matrix to TMA (driver error %d)", (int)r);
    return 0;
}

// tiles x splits <= blocks, k-blocks per split <= MAX_KB; returns 0 if impossible
int plan_half(int features, int K, int blocks, int* tiles, int* splits, int* kb) {
    *tiles = dd_ceil_div(features, BM);
    const int total = dd_ceil_div(K, BK);
    if (*tiles > blocks) return 0;
    int s = blocks / *tiles;
    if (s > total) s = total;
    *kb = dd_ceil_div(total, s);
    if (*kb > MAX_KB) return 0;
    *splits = dd_ceil_div(total, *kb);
    return 1;
}
}  // namespace

DD_API void dd_mlp_decode_timeline(unsigned long long* buffer) { g_mlp_timeline = buffer; }

// Floats of scratch (the `partial` argument) that dd_mlp_decode needs, or 0 if it does not take the problem
// (more than 16 tokens, widths that are no multiple of 8, or more work than one wave of blocks holds).
DD_API long long dd_mlp_decode_scratch(int M, int width, int inner, int sm_count) {
    int t, s, kb, t2, s2, kb2;
    if (M < 1 || M > BN || width % 8 || inner % 8) return 0;
    if (!plan_half(inner, width, sm_count, &t, &s, &kb) || !plan_half(width, inner, sm_count, &t2, &s2, &kb2)) return 0;
    return (long long)s * 16 * inner;
}

// x [M, width] float32 (row stride ldx), updated in place. w_up [inner, width], w_down [width, inner] bf16 row-major
// (row strides ld_up, ld_down). partial: float32 scratch of dd_mlp_decode_scratch() floats; sync: int32 [2], zero
// before the first launch (the kernel leaves it zero).
DD_API int dd_mlp_decode(float* x, int ldx, const float* gamma, const float* beta, float eps, const void* w_up, int ld_up,
                         const float* b_up, const void* w_down, int ld_down, const float* b_down, float* partial,
                         int* sync, int M, int width, int inner, int act, int sm_count, int* error_flag, void* stream) {
    if (M <= 0) return 0;
    MlpParams p;
    if (M > BN || width % 8 || inner % 8 || ld_up % 8 || ld_down % 8 ||
        !plan_half(inner, width, sm_count, &p.up_tiles, &p.up_splits, &p.up_kb) ||
        !plan_half(width, inner, sm_count, &p.down_tiles, &p.down_splits, &p.down_kb))
        return dd_fail("dd_mlp_decode: %d tokens, width %d, inner %d do not fit one wave of %d blocks", M, width, inner, sm_count);
    if (((uintptr_t)w_up & 15) || ((uintptr_t)w_down & 15) || !partial || !sync)
        return dd_fail("dd_mlp_decode: unaligned weights or missing scratch");
    p.x = x; p.ldx = ldx; p.gamma = gamma; p.beta = beta; p.eps = eps; p.b_up = b_up; p.b_down = b_down;
    p.timeline = g_mlp_timeline;
    p.partial = partial; p.sync = sync; p.error_flag = error_flag; p.M = M; p.width = width; p.inner = inner; p.act = act;
    CUtensorMap map_up, map_down;
    if (int e = weight_map(&map_up, w_up, inner, width, ld_up)) return e;
    if (int e = weight_map(&map_down, w_down, width, inner, ld_down)) return e;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(mlp_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return dd_fail("dd_mlp_decode: shared memory of %d bytes refused: %s", SMEM_BYTES, cudaGetErrorString(e));
        configured = true;
    }
    const int up_items = p.up_tiles * p.up_splits, down_items = p.down_tiles * p.down_splits;
    const int blocks = up_items > down_items ? up_items : down_items;
    cudaError_t e = dd_launch(mlp_decode_kernel, dim3(blocks), dim3(THREADS), SMEM_BYTES, (cudaStream_t)stream, map_up, map_down, p);
    if (e != cudaSuccess) return dd_fail("dd_mlp_decode: %s", cudaGetErrorString(e));
    return dd_check_launch("dd_mlp_decode");
}
