// A chain of dependent matrix products for a step of at most eight tokens, in ONE persistent kernel:
//     phase p:   in_p = (LayerNorm of a float32 [M, K] matrix)  or  (a bfloat16 [M, K] matrix)
//                out_p = act(in_p . W_p^T + bias_p) (+ residual_p), bfloat16 or float32
// Each phase may read what the phases before it wrote (the next phase's LayerNorm reads the residual stream the
// phase before it added into; the second matrix of a feed-forward reads the activated output of the first), so a
// grid-wide barrier stands between two phases. A decode step of a transformer layer is such a chain: output
// projection + residual -> norm -> up projection + activation -> down projection + residual -> next layer's norm ->
// next layer's query/key/value projection; as separate kernels each of them is a latency chain of its own
// (launch, first bytes, drain) over a few megabytes of weights. Nothing here knows what a layer is: a phase is a
// matrix, an optional norm in front and an epilogue.
//
// How it runs. One block of 16 warps per SM, all resident at once. A phase's weight matrix [N, K] is cut into tiles
// of 8 output features; a tile belongs to a group of 2..16 warps of one block, which split its K range in chunks of
// 32 among them (tiles go round the blocks first, so every SM streams about the same bytes). The eight tokens'
// activations of the phase lie in the block's shared memory ([8][K] bfloat16, computed by the block itself: the
// LayerNorm of eight rows is cheaper to repeat in every block than to hand around). A warp multiplies on the tensor
// cores with the tokens as the rows of mma.sync m16n8k16 and the tile's 8 features as its columns: a thread's 16
// bytes of a weight row, loaded straight from global memory into registers (no shared-memory stage for the weights:
// each byte is used once), feed two MMAs, against 16 bytes of the matching activations from shared memory; the k
// index inside a chunk is permuted the same way on both sides so that both are single 16-byte accesses. Eight such
// loads per thread are in flight. The warps of a group add their partial sums through shared memory in warp order
// (the result does not depend on timing), then bias, activation and residual, and store.
// Weights do not depend on activations: when a phase begins, the block asks L2 for the weight rows of its tiles of
// the NEXT phase (cp.async.bulk.prefetch.L2), so HBM keeps streaming through the barrier and the next phase's
// prologue, and the first two phases' rows are asked for before the kernel waits for its predecessor on the stream.
//
// The barrier is a counter and a generation word in global memory (the last block to arrive resets the counter and
// bumps the generation); its wait is bounded (error bit 8, then every block leaves). The kernel lets its successor
// on the stream launch only after its own first barrier, when all its blocks are known to be resident: a successor
// that took an SM before would wait for this kernel, which would wait for that SM.
#include "common.cuh"

namespace {

constexpr int MAX_PHASES = 4, WARPS = 16, THREADS = WARPS * 32, TOKENS = 8, TILE = 8, CHUNK = 32, RING = 8;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;
constexpr int MAX_K = 12288;          // eight rows of activations of the widest phase must fit into shared memory

struct Phase {
    const __nv_bfloat16* w;        // [N, K], row stride ldw
    const float* bias;             // [N] or null
    const __nv_bfloat16* in;       // [M, K] bfloat16 (row stride ld_in), or null when norm_src is given
    const float* norm_src;         // float32 [M, K] (row stride ld_norm): the input is its LayerNorm
    const float* gamma;            // [K]
    const float* beta;             // [K] or null
    __nv_bfloat16* norm_out;       // null, or [M, K] (dense) that also receives the normed rows
    void* out;                     // [M, N] bfloat16 or float32, row stride ld_out
    const float* residual;         // float32 [M, N] (row stride ld_res) or null; may be out itself
    float eps;
    int N, K, ldw, ld_in, ld_norm, ld_out, ld_res, act, out_f32, warps_per_tile;
};

struct Params {
    Phase phase[MAX_PHASES];
    int n_phases, M;
    unsigned* barrier;             // [2]: arrivals, generation
    int* error_flag;
};

__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_weights(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void prefetch_l2(const void* p, unsigned bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
__device__ __forceinline__ void group_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// D[16 tokens x 8 features] += A[16 tokens x 16 k] . B[16 k x 8 features]; tokens 8..15 do not exist (a1 = a3 = 0).
__device__ __forceinline__ void mma_tokens(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    const uint32_t zero = 0;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(zero), "r"(a2), "r"(zero), "r"(b0), "r"(b1));
}

// Tiles of a phase go round the blocks first, then round a block's groups, then into another round.
struct Split {
    int tiles, groups, rounds, chunks, per_warp;      // per_warp: chunks of a tile one warp takes (the last may be empty)
    __device__ Split(const Phase& ph, int n_blocks) {
        tiles = ph.N / TILE;
        groups = WARPS / ph.warps_per_tile;
        rounds = (tiles + n_blocks * groups - 1) / (n_blocks * groups);
        chunks = ph.K / CHUNK;
        per_warp = (chunks + ph.warps_per_tile - 1) / ph.warps_per_tile;
    }
    __device__ int tile(int round, int group, int block, int n_blocks) const {
        return (round * groups + group) * n_blocks + block;
    }
};

// Ask L2 for the weight rows of this block's tiles of a phase: lane r of each group's first warp takes row r of a tile.
__device__ void prefetch_phase(const Phase& ph, int n_blocks) {
    const Split s(ph, n_blocks);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = warp / ph.warps_per_tile;
    if (warp % ph.warps_per_tile != 0 || lane >= TILE) return;
    const unsigned row_bytes = (unsigned)ph.K * 2u;
    for (int r = 0; r < s.rounds; ++r) {
        const int tile = s.tile(r, group, blockIdx.x, n_blocks);
        if (tile < s.tiles) prefetch_l2(ph.w + (size_t)(tile * TILE + lane) * ph.ldw, row_bytes);
    }
}

// Returns false if the wait ran out (or another thread of the block saw that before).
__device__ bool grid_barrier(unsigned* bar, unsigned n_blocks, int* abort) {
    __syncthreads();
    if (threadIdx.x == 0 && !*abort) {
        const unsigned generation = ld_acquire(bar + 1);      // cannot move before this block has arrived
        __threadfence();
        if (atomicAdd(bar, 1u) == n_blocks - 1) {
            bar[0] = 0;
            __threadfence();
            atomicAdd(bar + 1, 1u);
        } else {
            const unsigned long long start = now_ns();
            unsigned spins = 0;
            while (ld_acquire(bar + 1) == generation) {
                if ((++spins & 0xff) == 0 && now_ns() - start > WAIT_LIMIT_NS) { *abort = 1; break; }
            }
        }
    }
    __syncthreads();
    return *abort == 0;
}

// The phase's input rows into shared memory: acts[token][K] bfloat16 with row stride `stride` (bytes).
__device__ void stage_input(const Phase& ph, int M, unsigned char* acts, int stride, float* stats) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K = ph.K;
    if (ph.norm_src == nullptr) {
        const int vecs = K / 8;                          // 16-byte pieces per row
        for (int i = threadIdx.x; i < TOKENS * vecs; i += THREADS) {
            const int token = i / vecs, v = i - token * vecs;
            uint4 val = make_uint4(0, 0, 0, 0);
            if (token < M) val = __ldcg(reinterpret_cast<const uint4*>(ph.in + (size_t)token * ph.ld_in) + v);
            *reinterpret_cast<uint4*>(acts + (size_t)token * stride + v * 16) = val;
        }
        return;
    }
    // LayerNorm: two warps per token, float32 two-pass statistics (mean, then squared deviations from it)
    const int token = warp >> 1, half = warp & 1;
    const int n4 = K / 4;
    const float4* row = reinterpret_cast<const float4*>(ph.norm_src + (size_t)token * ph.ld_norm);
    constexpr int VPT = 8;
    const bool in_regs = n4 <= 64 * VPT;
    float4 v[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    float sum = 0.f;
    if (token < M) {
        if (in_regs) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int c = half * 32 + lane + i * 64;
                v[i] = c < n4 ? __ldcg(row + c) : make_float4(0.f, 0.f, 0.f, 0.f);
                sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
            }
        } else {
            for (int c = half * 32 + lane; c < n4; c += 64) {
                const float4 t = __ldcg(row + c);
                sum += (t.x + t.y) + (t.z + t.w);
            }
        }
    }
    sum = dd_warp_sum(sum);
    if (lane == 0) stats[warp] = sum;
    __syncthreads();
    const float mean = (stats[warp & ~1] + stats[warp | 1]) / (float)K;
    float sq = 0.f;
    if (token < M) {
        if (in_regs) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                if (half * 32 + lane + i * 64 < n4) {
                    const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
                    sq += (a * a + b * b) + (c * c + d * d);
                }
            }
        } else {
            for (int c = half * 32 + lane; c < n4; c += 64) {
                const float4 t = __ldcg(row + c);
                const float a = t.x - mean, b = t.y - mean, cc = t.z - mean, d = t.w - mean;
                sq += (a * a + b * b) + (cc * cc + d * d);
            }
        }
    }
    sq = dd_warp_sum(sq);
    __syncthreads();
    if (lane == 0) stats[warp] = sq;
    __syncthreads();
    const float rstd = 1.0f / sqrtf((stats[warp & ~1] + stats[warp | 1]) / (float)K + ph.eps);
    const float4* gamma = reinterpret_cast<const float4*>(ph.gamma);
    const float4* beta = reinterpret_cast<const float4*>(ph.beta);
    __nv_bfloat16* copy = (ph.norm_out && blockIdx.x == 0 && token < M) ? ph.norm_out + (size_t)token * K : nullptr;
    auto emit = [&](int c, float4 t) {
        uint2 packed = make_uint2(0, 0);
        if (token < M) {
            const float4 g = __ldg(gamma + c);
            const float4 b = beta ? __ldg(beta + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            const __nv_bfloat162 lo = __floats2bfloat162_rn((t.x - mean) * rstd * g.x + b.x, (t.y - mean) * rstd * g.y + b.y);
            const __nv_bfloat162 hi = __floats2bfloat162_rn((t.z - mean) * rstd * g.z + b.z, (t.w - mean) * rstd * g.w + b.w);
            packed.x = *reinterpret_cast<const uint32_t*>(&lo);
            packed.y = *reinterpret_cast<const uint32_t*>(&hi);
            if (copy) *reinterpret_cast<uint2*>(copy + 4 * c) = packed;
        }
        *reinterpret_cast<uint2*>(acts + (size_t)token * stride + c * 8) = packed;
    };
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int c = half * 32 + lane + i * 64;
            if (c < n4) emit(c, v[i]);
        }
    } else {
        for (int c = half * 32 + lane; c < n4; c += 64)
            emit(c, token < M ? __ldcg(row + c) : make_float4(0.f, 0.f, 0.f, 0.f));
    }
}

__global__ void __launch_bounds__(THREADS, 1)
decode_chain_kernel(const __grid_constant__ Params p) {
    extern __shared__ __align__(16) unsigned char smem[];
    // [acts: TOKENS rows of the widest K] [partial sums: 2 x WARPS x 64 floats] [LayerNorm statistics] [abort]
    __shared__ float stats[WARPS];
    __shared__ int abort_flag;
    __shared__ __align__(16) float partial[2][WARPS][TOKENS * TILE];
    const int n_blocks = gridDim.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    if (threadIdx.x == 0) abort_flag = 0;

    // weights of the first two phases: asked of L2 before this kernel waits for the one before it on the stream
    prefetch_phase(p.phase[0], n_blocks);
    if (p.n_phases > 1) prefetch_phase(p.phase[1], n_blocks);
    if (p.n_phases == 1) dd_launch_dependents();
    dd_grid_wait();

    int parity = 0;
    for (int ip = 0; ip < p.n_phases; ++ip) {
        const Phase& ph = p.phase[ip];
        if (ip > 0) {
            if (!grid_barrier(p.barrier, n_blocks, &abort_flag)) break;
            if (ip == 1) dd_launch_dependents();         // every block of this kernel is resident now
            if (ip + 1 < p.n_phases) prefetch_phase(p.phase[ip + 1], n_blocks);
        }
        const int stride = ph.K * 2 + ((ph.K & 63) ? 0 : 64);      // rows 64 bytes apart modulo 128: 16-byte reads of eight
                                                                   // rows by a quarter warp touch every bank once
        stage_input(ph, p.M, smem, stride, stats);
        __syncthreads();

        const Split s(ph, n_blocks);
        const int wpt = ph.warps_per_tile;
        const int group = warp / wpt, slot = warp - group * wpt;
        const int total = s.rounds * s.per_warp;
        const unsigned char* my_acts = smem + (size_t)g * stride + t * 16;

        // a warp's items: (round, j) with chunk = slot + j * wpt of tile(round); loads run RING items ahead
        int lr = 0, lj = 0;
        auto load = [&]() -> uint4 {
            uint4 w = make_uint4(0, 0, 0, 0);
            if (lr < s.rounds) {
                const int tile = s.tile(lr, group, blockIdx.x, n_blocks), chunk = slot + lj * wpt;
                if (tile < s.tiles && chunk < s.chunks)
                    w = ld_weights(ph.w + (size_t)(tile * TILE + g) * ph.ldw + chunk * CHUNK + t * 8);
                if (++lj == s.per_warp) { lj = 0; ++lr; }
            }
            return w;
        };
        uint4 ring[RING];
#pragma unroll
        for (int u = 0; u < RING; ++u) ring[u] = load();
        int cr = 0, cj = 0;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int base = 0; base < total; base += RING) {
#pragma unroll
            for (int u = 0; u < RING; ++u) {
                if (base + u >= total) break;
                const uint4 w = ring[u];
                ring[u] = load();
                const int chunk = slot + cj * wpt;
                if (chunk < s.chunks) {
                    const uint4 a = *reinterpret_cast<const uint4*>(my_acts + chunk * (CHUNK * 2));
                    mma_tokens(acc, a.x, a.y, w.x, w.y);
                    mma_tokens(acc, a.z, a.w, w.z, w.w);
                }
                if (++cj == s.per_warp) {
                    // the tile is done: partial sums of the group's warps, added in warp order
                    const int tile = s.tile(cr, group, blockIdx.x, n_blocks);
                    *reinterpret_cast<float2*>(&partial[parity][warp][g * TILE + 2 * t]) = make_float2(acc[0], acc[1]);
                    group_sync(1 + group, wpt * 32);
                    const int idx = slot * 32 + lane;                 // the group's first 64 threads: one output each
                    if (idx < TOKENS * TILE && tile < s.tiles) {
                        const int token = idx >> 3, n = tile * TILE + (idx & 7);
                        if (token < p.M) {
                            float v = 0.f;
                            for (int q = 0; q < wpt; ++q) v += partial[parity][group * wpt + q][idx];
                            if (ph.bias) v += __ldg(ph.bias + n);
                            v = dd_activation(v, ph.act);
                            if (ph.residual) v += __ldcg(ph.residual + (size_t)token * ph.ld_res + n);
                            if (ph.out_f32) reinterpret_cast<float*>(ph.out)[(size_t)token * ph.ld_out + n] = v;
                            else reinterpret_cast<__nv_bfloat16*>(ph.out)[(size_t)token * ph.ld_out + n] = __float2bfloat16_rn(v);
                        }
                    }
                    parity ^= 1;
                    acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                    cj = 0;
                    ++cr;
                }
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag) atomicOr(p.error_flag, 8);
}

int best_warps_per_tile(int N, int n_blocks) {
    // fewest bytes on the busiest SM (rounds x groups tiles of equal size); among equals the widest group,
    // whose tiles end soonest
    int best = WARPS, best_cost = 1 << 30;
    for (int wpt = WARPS; wpt >= 2; wpt /= 2) {
        const int groups = WARPS / wpt, tiles = N / TILE;
        const int cost = ((tiles + n_blocks * groups - 1) / (n_blocks * groups)) * groups;
        if (cost < best_cost) { best_cost = cost; best = wpt; }
    }
    return best;
}

}  // namespace

// The C face of a phase (pointers, then numbers); see Phase above. out_f32: 1 float32 output, 0 bfloat16.
struct DdChainPhase {
    const void* w; const float* bias; const void* in; const float* norm_src; const float* gamma; const float* beta;
    void* norm_out; void* out; const float* residual;
    float eps;
    int N, K, ldw, ld_in, ld_norm, ld_out, ld_res, act, out_f32;
};

// 1 if a product of these sizes can be a phase: at most 8 tokens, K a multiple of 32, N a multiple of 8.
DD_API int dd_decode_chain_supported(int M, int N, int K) {
    return M >= 1 && M <= TOKENS && N > 0 && K > 0 && N % TILE == 0 && K % CHUNK == 0 && K <= MAX_K;
}

DD_API int dd_decode_chain_max_phases() { return MAX_PHASES; }

// barrier: two zeroed unsigned words on the device that belong to this library's chains alone (they return to zero
// and even after every launch that ends without an error). n_blocks: blocks to launch, at most the SM count.
DD_API int dd_decode_chain(const DdChainPhase* phases, int n_phases, int M, unsigned* barrier, int n_blocks,
                           int* error_flag, void* stream) {
    if (n_phases < 1 || n_phases > MAX_PHASES) return dd_fail("dd_decode_chain: %d phases (1..%d are taken)", n_phases, MAX_PHASES);
    if (M < 1 || M > TOKENS) return dd_fail("dd_decode_chain: %d tokens (1..%d are taken)", M, TOKENS);
    if (!barrier || !error_flag || n_blocks < 1) return dd_fail("dd_decode_chain: barrier, error flag and a block count are needed");
    Params p;
    p.n_phases = n_phases; p.M = M; p.barrier = barrier; p.error_flag = error_flag;
    int widest = 0;
    for (int i = 0; i < n_phases; ++i) {
        const DdChainPhase& s = phases[i];
        Phase& d = p.phase[i];
        if (!dd_decode_chain_supported(M, s.N, s.K))
            return dd_fail("dd_decode_chain: phase %d: N=%d must be a multiple of %d and K=%d of %d", i, s.N, TILE, s.K, CHUNK);
        if (!s.w || !s.out || (!s.in == !s.norm_src) || (s.norm_src && !s.gamma))
            return dd_fail("dd_decode_chain: phase %d: weights, an output and exactly one input (rows or rows to be normed) are needed", i);
        if (s.ldw % 8 || ((uintptr_t)s.w & 15) || (s.in && (s.ld_in % 8 || ((uintptr_t)s.in & 15))) ||
            (s.norm_src && (s.ld_norm % 4 || (((uintptr_t)s.norm_src | (uintptr_t)s.gamma | (uintptr_t)s.beta) & 15))) ||
            (s.norm_out && ((uintptr_t)s.norm_out & 7)))
            return dd_fail("dd_decode_chain: phase %d: rows must start on 16-byte boundaries", i);
        d.w = (const __nv_bfloat16*)s.w; d.bias = s.bias; d.in = (const __nv_bfloat16*)s.in; d.norm_src = s.norm_src;
        d.gamma = s.gamma; d.beta = s.beta; d.norm_out = (__nv_bfloat16*)s.norm_out; d.out = s.out; d.residual = s.residual;
        d.eps = s.eps; d.N = s.N; d.K = s.K; d.ldw = s.ldw; d.ld_in = s.ld_in; d.ld_norm = s.ld_norm; d.ld_out = s.ld_out;
        d.ld_res = s.ld_res; d.act = s.act; d.out_f32 = s.out_f32;
        d.warps_per_tile = best_warps_per_tile(s.N, n_blocks);
        widest = s.K > widest ? s.K : widest;
    }
    const size_t smem = (size_t)TOKENS * (widest * 2 + 64);
    static bool granted = false;
    if (!granted) {
        cudaError_t e = cudaFuncSetAttribute(decode_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             TOKENS * (MAX_K * 2 + 64));
        if (e != cudaSuccess) return dd_fail("dd_decode_chain: shared memory for rows of %d: %s", MAX_K, cudaGetErrorString(e));
        granted = true;
    }
    if (n_phases > 1) {
        int per_sm = 0, device = 0, sms = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_chain_kernel, THREADS, smem);
        if (per_sm < 1 || n_blocks > per_sm * sms)
            return dd_fail("dd_decode_chain: %d blocks cannot be resident at once (%d SMs x %d)", n_blocks, sms, per_sm);
    }
    dd_launch(decode_chain_kernel, dim3(n_blocks), dim3(THREADS), smem, (cudaStream_t)stream, p);
    return dd_check_launch("dd_decode_chain");
}
