// Prompt-portion attention on the tcgen05 tensor cores, for bfloat16 caches and head size 64.
//
// A block owns a pair of tiles of 128 consecutive query tokens each (256 tokens of one request, one head) and walks
// the request's keys in blocks of 128, which the two tiles share: the upper tile goes one block further than the
// lower (with a window they may also start at different blocks). Three roles:
//   warp 0      TMA: both query tiles once, then per key block either one box per cache page for the keys and one
//               for the values (each lane issues one box), or, for a block that lies wholly in this step, one box
//               of 128 rows each straight from the projection's output; several blocks ahead;
//   warp 1      one thread issues the MMAs: for each tile S_t = Q_t K^T (128 x 128, its own 128 TMEM columns) as
//               soon as the tile's softmax warps hold the scores of its block before in registers, and
//               O_t += P_t V (128 x 64, accumulated in TMEM over all blocks) for whichever tile has its P ready
//               first, with P read from tensor memory (64 columns of its own per tile) and V read as it lies in
//               memory, as an MN-major operand;
//   warps 2..5 and 6..9  softmax of the lower and of the upper tile: a thread owns one query row (its TMEM lane),
//               takes the row's 128 scores of a block into registers with four TMEM loads in flight, and writes
//               P as bfloat16 pairs into tensor memory. Scaling and row sums use float32 pair instructions and
//               the maximum a three-input instruction: the warps are bound by what they can issue as much as by
//               the special-function unit. The exponentials, the row sum and the output are relative to a
//               maximum that follows the true running maximum only when that has moved ahead by more than 8 (a
//               factor of 256): only then does a thread rescale its output row in TMEM, which is rare after the
//               first blocks; the result is the same, since the sum is kept relative to the same maximum.
// Scores, softmax and the weighted sum of values are float32 (damendaemon/kernels.py:147-178 for the mask and
// the stable softmax; damendaemon/qwen2.py:754-770 for the offset-aware causal rule). Keys outside the live
// range (beyond the last query of the pair, before the window, pages that were given back) are never multiplied
// in: their scores are replaced, not scaled, and their value rows are zeroed in shared memory, so that stale
// cache contents of any bit pattern cannot reach the result.
// On request (store_new) the block also writes its tiles' keys and values into the cache pages, by TMA from the
// shared memory they were loaded into, which saves the cache-write kernel and its pass over the projection's output.
// Every wait is bounded; a wait that runs out sets the error flag and the block leaves through the common exit.
#include "common.cuh"
#include "tcgen05.cuh"
#include <math_constants.h>

namespace {
constexpr int BQ = 128, TILES = 2, BKV = 128, D = 64, THREADS = 64 + TILES * 128, STAGES = 4;
constexpr int TILE_BYTES = BKV * D * 2;             // one 128 x 64 bf16 tile: 16 KB
constexpr int Q_BYTES = TILES * TILE_BYTES;         // the two query tiles, one after the other
constexpr int STAGE_BYTES = 2 * TILE_BYTES;         // keys, then values
constexpr int SMEM_BYTES = Q_BYTES + STAGES * STAGE_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 512;                      // per tile: scores 128 columns, P 64, output 64
__host__ __device__ constexpr int s_col(int t) { return t * BKV; }
__host__ __device__ constexpr int p_col(int t) { return TILES * BKV + t * (BKV / 2); }
__host__ __device__ constexpr int o_col(int t) { return TILES * BKV + TILES * (BKV / 2) + t * D; }

struct AttnParams {
    const int* entry_start;
    const int* entry_pos0;
    const int* block_table;
    __nv_bfloat16* out;
    int* error_flag;
    int n_entries, max_blocks, out_stride, H, KH, P, n_pages, window;
    float scale_log2e;
    int new_rows;                   // 1: this step's keys and values are also at hand as rows beside the queries
    int store_new;                  // 1: the kernel itself puts those rows into the cache (every entry starts on a key-block boundary)
};


__device__ __forceinline__ float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two float32 operations in one instruction (sm_100): the softmax warps are bound by the number of instructions they
// issue, not by any one pipe, so the scaling and the row sums work on pairs, and the maximum takes three inputs.
__device__ __forceinline__ unsigned long long pair_of(uint32_t lo, uint32_t hi) {
    unsigned long long v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(lo), "r"(hi));
    return v;
}
__device__ __forceinline__ void halves_of(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma_pair(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long add_pair(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max_of_three(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                                 const __grid_constant__ CUtensorMap map_k_new, const __grid_constant__ CUtensorMap map_v_new,
                                 const AttnParams p) {
    dd_launch_dependents();
    // Which pair of 128-row tiles of which entry is this block's? Blocks beyond the real count leave at once. The
    // heads of a pair are neighbours in launch order and an entry's pairs come last pair first: the last one has the
    // most key blocks to walk, and the blocks that are launched last, which decide when the kernel ends, should be
    // short ones.
    int e = 0, pair = blockIdx.y, len = 0;
    for (; e < p.n_entries; ++e) {
        len = p.entry_start[e + 1] - p.entry_start[e];
        const int np = (len + TILES * BQ - 1) / (TILES * BQ);
        if (pair < np) {
            pair = np - 1 - pair;
            break;
        }
        pair -= np;
    }
    if (e == p.n_entries) return;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* sQ = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sKV = sQ + Q_BYTES;
    uint64_t* kv_full = reinterpret_cast<uint64_t*>(sKV + STAGES * STAGE_BYTES);
    uint64_t* kv_empty = kv_full + STAGES;
    uint64_t* q_full = kv_empty + STAGES;
    uint64_t* s_full = q_full + 1;        // [tile]: the scores of the tile's next key block are in tensor memory
    uint64_t* s_free = s_full + TILES;    // [tile]: the softmax warps hold them in registers, the columns may be overwritten
    uint64_t* p_ready = s_free + TILES;   // [tile]: P of the block is in tensor memory (and dead value rows are zeros)
    uint64_t* o_full = p_ready + TILES;   // [tile]: the P.V product of the block has been added to the tile's output
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + TILES);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.x, kh = h / (p.H / p.KH);
    const int q0 = pair * TILES * BQ;
    const int rows_all = min(TILES * BQ, len - q0);
    const int n_tiles = rows_all > BQ ? 2 : 1;
    const int row0 = p.entry_start[e] + q0;
    const int pos0 = p.entry_pos0[e];
    const int pos_first = pos0 + q0, pos_last = pos_first + rows_all - 1;       // of the pair
    // first and last position of tile t, the first key its window lets it see, and the key blocks it takes part in
    // (counted from the pair's first): the upper tile walks on where the lower one has met its diagonal
    auto tile_first = [&](int t) { return pos_first + t * BQ; };
    auto tile_last = [&](int t) { return min(pos_first + t * BQ + BQ - 1, pos_last); };
    auto tile_lo = [&](int t) { return p.window > 0 ? max(0, tile_first(t) - p.window + 1) : 0; };
    const int kb_first = tile_lo(0) / BKV * BKV;
    const int n_blocks = (pos_last - kb_first) / BKV + 1;
    auto block_first = [&](int t) { return (tile_lo(t) / BKV * BKV - kb_first) / BKV; };
    auto block_last = [&](int t) { return (tile_last(t) - kb_first) / BKV; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&kv_full[s], 1);
            tc::mbar_init(&kv_empty[s], 1);
        }
        tc::mbar_init(q_full, 1);
        for (int t = 0; t < TILES; ++t) {
            tc::mbar_init(&s_full[t], 1);
            tc::mbar_init(&s_free[t], 4);         // one arrival per softmax warp of the tile
            tc::mbar_init(&p_ready[t], 4);
            tc::mbar_init(&o_full[t], 1);
        }
        *abort_flag = 0;
        tc::fence_barrier_init();
        tc::fence_proxy_async();
        tc::prefetch_tensormap(&map_q);
        tc::prefetch_tensormap(&map_kv);
        tc::prefetch_tensormap(&map_k_new);
        tc::prefetch_tensormap(&map_v_new);
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    dd_grid_wait();              // queries and the cache are earlier kernels' results

    if (warp == 0) {
        // ---- TMA ----
        if (lane == 0) {
            tc::mbar_expect_tx(q_full, Q_BYTES);
            tc::tma_load_2d(sQ, &map_q, h * D, row0, q_full);       // rows past the last token read as zeros
        }
        const int pages_per_block = BKV / p.P;
        const int* bt = p.block_table + (size_t)e * p.max_blocks;
        const uint32_t page_bytes = (uint32_t)p.P * D * 2;
        const int kv_lo = tile_lo(0);
        // The warp holds 32 consecutive entries of the request's block table, one per lane, and the next 32 already
        // requested: a key block's pages never straddle such a window (its first entry is a multiple of the pages
        // per block, which divide 32), and no block waits for a table read of its own.
        auto table_window = [&](int w) { const int i = w * 32 + lane; return i < p.max_blocks ? bt[i] : -1; };
        int window_at = (kb_first / p.P) / 32;
        int held = table_window(window_at), ahead = table_window(window_at + 1);
        for (int j = 0; j < n_blocks; ++j) {
            const int s = j % STAGES;
            if (j >= STAGES) {
                bool ok = true;
                if (lane == 0) ok = tc::mbar_wait(&kv_empty[s], ((j / STAGES) - 1) & 1, abort_flag);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
            }
            const int kb = kb_first + j * BKV;
            uint8_t* k_dst = sKV + s * STAGE_BYTES;
            uint8_t* v_dst = k_dst + TILE_BYTES;
            if (p.new_rows && kb >= pos0) {
                // Every key of this block is one of this step's own: they lie row after row beside the queries, so one
                // box of 128 rows brings the keys and one the values (a box per cache page costs the TMA unit about
                // 60 ns each, 1 us per block with pages of 16 tokens, which is what bounded whole prompts). Rows past
                // the entry are other requests' tokens or zeros: masked by position like any key after the query.
                if (lane == 0) {
                    const int row = (row0 - q0) + kb - pos0;       // the entry's first row + (key - its first position)
                    tc::mbar_expect_tx(&kv_full[s], STAGE_BYTES);
                    tc::tma_load_2d(k_dst, &map_k_new, kh * D, row, &kv_full[s]);
                    tc::tma_load_2d(v_dst, &map_v_new, kh * D, row, &kv_full[s]);
                }
                continue;
            }
            const int first_entry = kb / p.P;
            if (first_entry / 32 != window_at) {
                window_at = first_entry / 32;
                held = ahead;
                ahead = table_window(window_at + 1);
            }
            // lanes 0 .. pages-1 fetch the key boxes of the block's pages, the next `pages` lanes the value boxes
            const int slot = lane < pages_per_block ? lane : lane - pages_per_block;
            const bool values = lane >= pages_per_block;
            const int page = __shfl_sync(0xffffffffu, held, (first_entry + slot) & 31);
            bool valid = false;
            if (lane < 2 * pages_per_block) {
                const int key0 = kb + slot * p.P;
                valid = key0 <= pos_last && key0 + p.P > kv_lo;
                if (valid && (page < 0 || page >= p.n_pages)) {
                    atomicOr(p.error_flag, 4);
                    valid = false;
                }
            }
            const int n_valid = __popc(__ballot_sync(0xffffffffu, valid));          // boxes, keys and values counted apart
            if (lane < 2 * pages_per_block) {
                if (valid) {
                    const int row = ((page * 2 + (values ? 1 : 0)) * p.KH + kh) * p.P;
                    tc::tma_load_2d((values ? v_dst : k_dst) + slot * page_bytes, &map_kv, 0, row, &kv_full[s]);
                } else if (values) {
                    // no live key in this page: its scores are all masked; its value rows must be zeros
                    uint4* z = reinterpret_cast<uint4*>(v_dst + slot * page_bytes);
                    for (uint32_t i = 0; i < page_bytes / 16; ++i) z[i] = make_uint4(0, 0, 0, 0);
                    tc::fence_proxy_async();
                }
            }
            __syncwarp();
            if (lane == 0) tc::mbar_expect_tx(&kv_full[s], (uint32_t)n_valid * page_bytes);
        }
        if (p.store_new && h % (p.H / p.KH) == 0) {
            // The pair's own keys and values are its last key blocks (one per tile), and they lie in shared memory in
            // the layout of the cache's tensor map: TMA writes them into their pages, one box per page, while the block
            // works on them. No block of this launch reads these cache rows: with every entry starting on a key-block
            // boundary, the key blocks that hold this step's tokens are read from k_new/v_new. A page that the entry
            // fills only in part receives whatever follows the entry's last token in its other slots; slots past a
            // request's length are never read by anyone.
            if (pos0 % BKV != 0) {
                if (lane == 0) atomicOr(p.error_flag, 2);        // the caller broke the rule: nothing is written
            } else {
                for (int j = n_blocks - n_tiles; j < n_blocks; ++j) {
                    const int s = j % STAGES, kb = kb_first + j * BKV;
                    if (!tc::mbar_wait(&kv_full[s], (j / STAGES) & 1, abort_flag)) break;
                    if (lane < 2 * pages_per_block) {
                        const int slot = lane < pages_per_block ? lane : lane - pages_per_block;
                        const bool values = lane >= pages_per_block;
                        const int key0 = kb + slot * p.P;
                        if (key0 <= pos_last) {
                            const int page = bt[key0 / p.P];
                            if (page < 0 || page >= p.n_pages) atomicOr(p.error_flag, 2);
                            else
                                tc::tma_store_2d(&map_kv, 0, ((page * 2 + (values ? 1 : 0)) * p.KH + kh) * p.P,
                                                 sKV + s * STAGE_BYTES + (values ? TILE_BYTES : 0) + slot * page_bytes);
                        }
                    }
                }
                tc::bulk_commit();
                tc::bulk_wait_all();         // shared memory has been read and the cache written before the block leaves
            }
        }
    } else if (warp == 1) {
        // ---- MMA ----
        if (tc::elect_one()) {
            constexpr uint32_t idesc_s = tc::idesc_bf16_f32(BQ, BKV);
            constexpr uint32_t idesc_o = tc::idesc_bf16_f32_b_mn(BQ, D);
            const uint32_t q_addr = tc::smem_u32(sQ);
            int first[TILES], last[TILES], scored[TILES], added[TILES];
#pragma unroll
            for (int t = 0; t < TILES; ++t) {
                first[t] = block_first(t);
                last[t] = t < n_tiles ? block_last(t) : -1;
                scored[t] = added[t] = 0;
            }
            bool ok = tc::mbar_wait(q_full, 0, abort_flag);
            tc::fence_after_sync();
            // S_t = Q_t K_j^T for the tiles that take part in key block j, as soon as a tile's softmax warps have taken
            // its previous scores into registers
            auto issue_scores = [&](int j) {
                const int s = j % STAGES;
                if (!tc::mbar_wait(&kv_full[s], (j / STAGES) & 1, abort_flag)) { ok = false; return; }
                const uint32_t k_addr = tc::smem_u32(sKV + s * STAGE_BYTES);
#pragma unroll
                for (int t = 0; t < TILES; ++t) {
                    if (j < first[t] || j > last[t]) continue;
                    if (scored[t] > 0 && !tc::mbar_wait(&s_free[t], (scored[t] - 1) & 1, abort_flag)) { ok = false; return; }
                    tc::fence_after_sync();
#pragma unroll
                    for (int k = 0; k < D / 16; ++k)
                        tc::mma_bf16(tmem_base + s_col(t), tc::smem_desc_sw128(q_addr + t * TILE_BYTES + k * 32),
                                     tc::smem_desc_sw128(k_addr + k * 32), idesc_s, k > 0 ? 1u : 0u);
                    tc::mma_commit(&s_full[t]);
                    ++scored[t];
                }
            };
            if (ok) issue_scores(0);
            for (int j = 0; j < n_blocks && ok; ++j) {
                if (j + 1 < n_blocks) issue_scores(j + 1);
                if (!ok) break;
                // O_t += P_t V_j, for each tile as soon as its P is there, whichever comes first
                const int s = j % STAGES;
                const uint32_t v_addr = tc::smem_u32(sKV + s * STAGE_BYTES + TILE_BYTES);
                uint32_t pending = 0;
#pragma unroll
                for (int t = 0; t < TILES; ++t)
                    if (j >= first[t] && j <= last[t]) pending |= 1u << t;
                const unsigned long long start = tc::global_ns();
                uint32_t spins = 0;
                while (pending && ok) {
#pragma unroll
                    for (int t = 0; t < TILES; ++t) {
                        if (!(pending & (1u << t)) || !tc::mbar_try_wait(&p_ready[t], added[t] & 1)) continue;
                        tc::fence_after_sync();
#pragma unroll
                        for (int k = 0; k < BKV / 16; ++k)
                            tc::mma_bf16_a_tmem(tmem_base + o_col(t), tmem_base + p_col(t) + k * 8,
                                                tc::smem_desc_sw128_mn(v_addr + k * 16 * D * 2, 1024), idesc_o,
                                                (added[t] > 0 || k > 0) ? 1u : 0u);
                        tc::mma_commit(&o_full[t]);
                        ++added[t];
                        pending &= ~(1u << t);
                    }
                    if (pending && (++spins & 0x3ff) == 0 && (*abort_flag || tc::global_ns() - start > tc::WAIT_LIMIT_NS)) {
                        *abort_flag = 1;
                        ok = false;
                    }
                }
                if (ok) tc::mma_commit(&kv_empty[s]);            // keys and values of this block have been read
            }
        }
    } else if (((warp - 2) >> 2) < n_tiles) {
        // ---- softmax and output: four warps per tile, a thread owns one query row (its TMEM lane) ----
        const int t = (warp - 2) >> 2, quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const int t_first = tile_first(t), rows = tile_last(t) - t_first + 1;
        const int qpos = t_first + r;
        const int qlo = p.window > 0 ? max(0, qpos - p.window + 1) : 0;
        const int j_first = block_first(t), j_last = block_last(t);
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        // m: the maximum the row's exponentials, sum and output are relative to. It follows the true running maximum only
        // when that has moved ahead by more than 8 (a factor of 256, harmless in float32 and bfloat16): only then is the
        // output row in TMEM rescaled, which is rare after the first blocks. l: the row's sum.
        float m = -CUDART_INF_F, l = 0.f;
        bool alive = true;
        for (int j = j_first, c = 0; j <= j_last && alive; ++j, ++c) {
            const int kb = kb_first + j * BKV;
            alive = __all_sync(0xffffffffu, tc::mbar_wait(&s_full[t], c & 1, abort_flag));
            if (!alive) break;
            tc::fence_after_sync();
            // the row's 128 scores of the block into registers: four loads in flight, one wait; then the columns are free
            uint32_t sv[BKV];
#pragma unroll
            for (int c0 = 0; c0 < BKV; c0 += 32) tc::tmem_ld_x32(lane_addr + s_col(t) + c0, sv + c0);
            tc::tmem_ld_wait();
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&s_free[t]);
            if (kb + BKV - 1 > qpos || kb < qlo) {
#pragma unroll
                for (int i = 0; i < BKV; ++i)
                    if (kb + i > qpos || kb + i < qlo) sv[i] = 0xff800000u;      // -inf: replaced, whatever was there
            }
            float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
            for (int i = 0; i < BKV; i += 2)
                mx4[(i >> 1) & 3] = max_of_three(mx4[(i >> 1) & 3], __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            const float m_true = fmaxf(m, mx * p.scale_log2e);     // the scale is positive
            const bool move = m_true > m + 8.f || (m == -CUDART_INF_F && m_true != -CUDART_INF_F);
            const float alpha = move ? exp2_approx(m - m_true) : 1.f;      // 0 from -inf
            if (move) m = m_true;
            const float msub = m == -CUDART_INF_F ? 0.f : m;
            if (c > 0) {
                // P of the block before has been read and its product added to the output: P may be overwritten, the
                // output rescaled
                alive = __all_sync(0xffffffffu, tc::mbar_wait(&o_full[t], (c - 1) & 1, abort_flag));
                if (!alive) break;
                tc::fence_after_sync();
                if (__any_sync(0xffffffffu, move)) {
#pragma unroll
                    for (int d0 = 0; d0 < D; d0 += 16) {          // in small pieces: the scores fill the registers
                        uint32_t v[16];
                        tc::tmem_ld_x16(lane_addr + o_col(t) + d0, v);
                        tc::tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        tc::tmem_st_x16(lane_addr + o_col(t) + d0, v);
                    }
                }
            }
            // exponentials (a masked score gives exactly 0), their sum, and P as bfloat16 into tensor memory: two
            // consecutive keys per column
            const unsigned long long scale2 = pair_of(__float_as_uint(p.scale_log2e), __float_as_uint(p.scale_log2e));
            const unsigned long long shift2 = pair_of(__float_as_uint(-msub), __float_as_uint(-msub));
            unsigned long long sums[4] = {0ull, 0ull, 0ull, 0ull};           // pairs of float32 zeros
#pragma unroll
            for (int c0 = 0; c0 < BKV; c0 += 32) {
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float x0, x1;
                    halves_of(fma_pair(pair_of(sv[c0 + 2 * i], sv[c0 + 2 * i + 1]), scale2, shift2), x0, x1);
                    const float p0 = exp2_approx(x0), p1 = exp2_approx(x1);
                    sums[i & 3] = add_pair(sums[i & 3], pair_of(__float_as_uint(p0), __float_as_uint(p1)));
                    packed[i] = pack_bf16(p0, p1);
                }
                tc::tmem_st_x16(lane_addr + p_col(t) + c0 / 2, packed);
            }
            float sum4[4];
            {
                float lo, hi;
                halves_of(add_pair(add_pair(sums[0], sums[1]), add_pair(sums[2], sums[3])), lo, hi);
                sum4[0] = lo; sum4[1] = hi; sum4[2] = 0.f; sum4[3] = 0.f;
            }
            l = l * alpha + (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            if (kb + BKV - 1 > pos_last) {
                // value rows of keys past the pair's last query: unwritten cache slots, to be zeros under P = 0 (where
                // both tiles take part in such a block both write these zeros)
                const int s = j % STAGES;
                alive = __all_sync(0xffffffffu, tc::mbar_wait(&kv_full[s], (j / STAGES) & 1, abort_flag));
                if (!alive) break;
                if (kb + r > pos_last) {
                    uint4* z = reinterpret_cast<uint4*>(sKV + s * STAGE_BYTES + TILE_BYTES + r * 128);
#pragma unroll
                    for (int i = 0; i < 8; ++i) z[i] = make_uint4(0, 0, 0, 0);
                }
            }
            tc::tmem_st_wait();               // P is in tensor memory
            tc::fence_proxy_async();          // the zeroed value rows to the proxy the MMA reads through
            tc::fence_before_sync();          // this thread's TMEM reads and writes are done
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&p_ready[t]);
        }
        // the output row after the last block's P.V
        if (alive) alive = __all_sync(0xffffffffu, tc::mbar_wait(&o_full[t], (j_last - j_first) & 1, abort_flag));
        if (alive) {
            tc::fence_after_sync();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* dst = p.out + (size_t)(row0 + t * BQ + r) * p.out_stride + (size_t)h * D;
#pragma unroll
            for (int d0 = 0; d0 < D; d0 += 32) {
                uint32_t v[32];
                tc::tmem_ld_x32(lane_addr + o_col(t) + d0, v);
                tc::tmem_ld_wait();
                if (r < rows) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        float f[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[c + i]) * inv;
                        *reinterpret_cast<uint4*>(dst + d0 + c) = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]),
                                                                               pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
                    }
                }
            }
        }
    }

    tc::fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicOr(p.error_flag, 8);
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, TMEM_COLS);
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

// rows x cols bf16 with row stride ld elements; boxes of box_rows x 64 columns, 128-byte swizzle
int make_map(CUtensorMap* map, const void* base, unsigned long long rows, int cols, long long ld, int box_rows, const char* what) {
    EncodeTiled enc = encode_fn();
    if (!enc) return dd_fail("dd_attention_prefill_tcgen05: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)D, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return dd_fail("dd_attention_prefill_tcgen05: cannot describe %s to TMA (driver error %d)", what, (int)r);
    return 0;
}
}  // namespace


// Head size 64, pages of 8, 16, 32, 64 or 128 tokens (a page is one TMA box inside a 128-key block).
DD_API int dd_attention_prefill_tcgen05_supported(int n_heads, int n_kv_heads, int head_dim, int page_size, int dtype) {
    return dtype == DD_BF16 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 && head_dim == D &&
           (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128);
}

// The arguments of dd_attention_prefill: entries are runs of consecutive tokens of one request; entry e holds
// flattened tokens entry_start[e] .. entry_start[e+1]-1 at positions entry_pos0[e] ...; block_table row e is its
// pages. cache [n_pages, 2, n_kv_heads, page_size, 64] bf16, which must hold this step's keys and values already
// unless store_new is set.
// k_new/v_new: null, or this step's keys and values as rows of q_stride bf16 (kv head g at g*64), the same values
// the cache holds: key blocks that lie wholly in this step are then read from there, one TMA box per block.
// store_new: the cache does not hold this step's keys and values yet; the kernel writes them from k_new/v_new
// (dd_kv_store's work, done by TMA from the tiles in shared memory). Only for steps in which every entry starts at a
// position that is a multiple of 128, so that no key block mixes cached and new keys (the caller's duty; an entry
// that breaks it sets error bit 2 and writes nothing).
DD_API int dd_attention_prefill_tcgen05(const void* q, int q_stride, const void* k_new, const void* v_new, int store_new, void* cache, const int* entry_start,
                                        const int* entry_pos0, int n_entries, int n_tokens, const int* block_table,
                                        int max_blocks, void* out, int out_stride, int n_heads, int n_kv_heads,
                                        int head_dim, int page_size, int n_pages, int window, float scale,
                                        int* error_flag, void* stream) {
    if (n_tokens <= 0 || n_entries <= 0) return 0;
    if (!dd_attention_prefill_tcgen05_supported(n_heads, n_kv_heads, head_dim, page_size, DD_BF16))
        return dd_fail("dd_attention_prefill_tcgen05: needs head size 64, pages of 8 to 128 tokens (a power of two) and heads a "
                       "multiple of key/value heads (got head size %d, pages of %d, %d and %d heads)",
                       head_dim, page_size, n_heads, n_kv_heads);
    if (q_stride % 8 || out_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)cache & 15) || ((uintptr_t)out & 15))
        return dd_fail("dd_attention_prefill_tcgen05: rows must be 16-byte aligned");
    if (dd_ceil_div(n_tokens, TILES * BQ) + n_entries > 65535) return dd_fail("dd_attention_prefill_tcgen05: too many tokens for one launch");
    if (!(scale > 0.f)) return dd_fail("dd_attention_prefill_tcgen05: the score scale must be positive");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return dd_fail("dd_attention_prefill_tcgen05: shared memory of %d bytes refused: %s", SMEM_BYTES, cudaGetErrorString(e));
        configured = true;
    }
    if ((k_new == nullptr) != (v_new == nullptr) || ((uintptr_t)k_new & 15) || ((uintptr_t)v_new & 15))
        return dd_fail("dd_attention_prefill_tcgen05: k_new and v_new come together, 16-byte aligned");
    if (store_new && !k_new) return dd_fail("dd_attention_prefill_tcgen05: store_new needs k_new and v_new");
    CUtensorMap map_q, map_kv, map_k_new, map_v_new;
    if (int e = make_map(&map_q, q, (unsigned long long)n_tokens, n_heads * D, q_stride, TILES * BQ, "the queries")) return e;
    // this step's keys and values as rows of the same stride as the queries (the fused projection's output), or the
    // queries again as a stand-in that is never read
    if (int e = make_map(&map_k_new, k_new ? k_new : q, (unsigned long long)n_tokens, (k_new ? n_kv_heads : n_heads) * D, q_stride, BKV, "this step's keys")) return e;
    if (int e = make_map(&map_v_new, v_new ? v_new : q, (unsigned long long)n_tokens, (v_new ? n_kv_heads : n_heads) * D, q_stride, BKV, "this step's values")) return e;
    const unsigned long long kv_rows = (unsigned long long)n_pages * 2 * n_kv_heads * page_size;
    if (int e = make_map(&map_kv, cache, kv_rows, D, D, page_size, "the cache")) return e;
    AttnParams p;
    p.entry_start = entry_start; p.entry_pos0 = entry_pos0; p.block_table = block_table;
    p.out = (__nv_bfloat16*)out; p.error_flag = error_flag;
    p.n_entries = n_entries; p.max_blocks = max_blocks; p.out_stride = out_stride; p.H = n_heads; p.KH = n_kv_heads;
    p.P = page_size; p.n_pages = n_pages; p.window = window; p.scale_log2e = scale * 1.4426950408889634f;
    p.new_rows = k_new != nullptr;
    p.store_new = store_new != 0;
    // an upper bound of the number of pairs of 128-row tiles; blocks beyond the real count return at once
    dim3 grid(n_heads, dd_ceil_div(n_tokens, TILES * BQ) + n_entries);
    dd_launch(attention_prefill_tcgen05_kernel, grid, dim3(THREADS), SMEM_BYTES, (cudaStream_t)stream, map_q, map_kv, map_k_new, map_v_new, p);
    return dd_check_launch("dd_attention_prefill_tcgen05");
}
