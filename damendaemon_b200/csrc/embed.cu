// Token embedding with the position table fused: x[t] = wte[ids[t]] + wpe[pos[t]].
// Each gather is widened to float32 before the add (damendaemon/gpt2.py:46); the
// residual stream it starts is float32 in both engine dtypes.
#include "common.cuh"

template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const int* __restrict__ pos,
                             const T* __restrict__ wte, const T* __restrict__ wpe,
                             float* __restrict__ out, int width, int vocab, int n_positions,
                             int* __restrict__ error_flag) {
    dd_launch_dependents();
    dd_grid_wait();
    const int row = blockIdx.x;
    int id = ids[row];
    int p = wpe ? pos[row] : 0;
    if (id < 0 || id >= vocab || p < 0 || (wpe && p >= n_positions)) {
        if (threadIdx.x == 0) atomicOr(error_flag, 1);
        id = min(max(id, 0), vocab - 1);
        p = min(max(p, 0), n_positions - 1);
    }
    const T* a = wte + (size_t)id * width;
    const T* b = wpe ? wpe + (size_t)p * width : nullptr;
    float* o = out + (size_t)row * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = dd_to_f32(a[c]);
        if (b) v += dd_to_f32(b[c]);
        o[c] = v;
    }
}

// error_flag: one int on the device; bit 0 is set when an id or a position is out of range.
DD_API int dd_embed(const int* ids, const int* pos, const void* wte, const void* wpe, float* out,
                    int n_tokens, int width, int vocab, int n_positions, int table_dtype,
                    int* error_flag, void* stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0 || vocab <= 0) return dd_fail("dd_embed: bad sizes width=%d vocab=%d", width, vocab);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = width >= 1024 ? 256 : 128;
    if (table_dtype == DD_F32)
        dd_launch(embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, ids, pos, (const float*)wte, (const float*)wpe, out,
                                                         width, vocab, n_positions, error_flag);
    else if (table_dtype == DD_BF16)
        dd_launch(embed_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, s, ids, pos, (const __nv_bfloat16*)wte,
                                                                 (const __nv_bfloat16*)wpe, out, width, vocab,
                                                                 n_positions, error_flag);
    else
        return dd_fail("dd_embed: unknown table dtype %d", table_dtype);
    return dd_check_launch("dd_embed");
}
