// Write this step's keys and values into the request's cache pages.
// Cache layout of one layer: [n_pages, 2 (K, V), kv_heads, page_size, head_dim].
// The page of a token is block_table[entry][position / page_size]
// (the reference stores with index assignment, damendaemon/gpt2.py:50-51, and
// through a page table in damendaemon/kernels.py:270-340).
#include "common.cuh"

template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ k_src, const T* __restrict__ v_src, int src_stride,
                                const int* __restrict__ tok_entry, const int* __restrict__ tok_pos,
                                const int* __restrict__ block_table, int max_blocks,
                                T* __restrict__ cache, int n_pages, int kv_heads, int page_size, int head_dim,
                                int* __restrict__ error_flag) {
    dd_launch_dependents();
    // positions, entries and the block table are the step's inputs: the page is known before the projection has finished
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const int block = pos / page_size;
    int page = (pos >= 0 && block < max_blocks) ? block_table[(size_t)tok_entry[t] * max_blocks + block] : -1;
    dd_grid_wait();
    if (page < 0 || page >= n_pages) {
        if (threadIdx.x == 0) atomicOr(error_flag, 2);
        return;
    }
    const int row = kv_heads * head_dim;
    const size_t plane = (size_t)kv_heads * page_size * head_dim;
    T* k_dst = cache + (size_t)page * 2 * plane + (size_t)(pos % page_size) * head_dim;
    T* v_dst = k_dst + plane;
    const T* ks = k_src + (size_t)t * src_stride;
    const T* vs = v_src + (size_t)t * src_stride;
    constexpr int V = 16 / sizeof(T);       // elements per 16-byte copy
    if (head_dim % V == 0 && src_stride % V == 0 && (((uintptr_t)k_src | (uintptr_t)v_src | (uintptr_t)cache) & 15) == 0) {
        for (int c = threadIdx.x * V; c < row; c += blockDim.x * V) {
            const int h = c / head_dim, i = c - h * head_dim;
            const size_t off = (size_t)h * page_size * head_dim + i;
            *reinterpret_cast<uint4*>(k_dst + off) = *reinterpret_cast<const uint4*>(ks + c);
            *reinterpret_cast<uint4*>(v_dst + off) = *reinterpret_cast<const uint4*>(vs + c);
        }
        return;
    }
    for (int c = threadIdx.x; c < row; c += blockDim.x) {
        const int h = c / head_dim, i = c - h * head_dim;
        const size_t off = (size_t)h * page_size * head_dim + i;
        k_dst[off] = ks[c];
        v_dst[off] = vs[c];
    }
}

// k_src/v_src: first key / value element of token 0; rows are src_stride elements apart.
DD_API int dd_kv_store(const void* k_src, const void* v_src, int src_stride, const int* tok_entry,
                       const int* tok_pos, const int* block_table, int max_blocks, void* cache, int n_pages,
                       int kv_heads, int page_size, int head_dim, int n_tokens, int dtype, int* error_flag,
                       void* stream) {
    if (n_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = kv_heads * head_dim >= 1024 ? 256 : 128;
    if (dtype == DD_F32)
        dd_launch(kv_store_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (const float*)k_src, (const float*)v_src, src_stride,
            tok_entry, tok_pos, block_table, max_blocks, (float*)cache, n_pages, kv_heads, page_size, head_dim, error_flag);
    else if (dtype == DD_BF16)
        dd_launch(kv_store_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, s, (const __nv_bfloat16*)k_src, (const __nv_bfloat16*)v_src,
            src_stride, tok_entry, tok_pos, block_table, max_blocks, (__nv_bfloat16*)cache, n_pages, kv_heads, page_size,
            head_dim, error_flag);
    else
        return dd_fail("dd_kv_store: unknown dtype %d", dtype);
    return dd_check_launch("dd_kv_store");
}
