// dd_attention_rows_static: paged attention with split keys for callers that cannot allocate.
//
// This entry point has no counterpart in the reference project. It exists for hosts that
// drive these kernels but may not call cudaMalloc, or any routine that allocates for them,
// at the moment they need attention: code that runs inside someone else's memory plan (an
// embedding application that hands this library a fixed arena and nothing more), a
// real-time loop that must not take the allocator's lock, or a process whose device memory
// is already spoken for down to the last page. dd_attention_rows wants two float32
// scratch buffers from its caller when the keys are cut into splits; this variant brings
// its own, a fixed array inside the library image.
//
// What the caller should know:
//  * The scratch is DD_STATIC_SCRATCH_BYTES (8 MiB) of device memory per GPU that loads the
//    library, held until the process exits whether or not this function is ever called.
//  * A call needs n_tokens * n_heads * n_splits * (head_dim + 2) floats of it. A call that
//    needs more is refused with an error message (dd_last_error) and launches nothing. With
//    n_splits == 1 no scratch is used at all.
//  * The first call on each device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current). Make that first call outside any
//    stream capture; later calls only launch kernels.
//  * All calls on a device share the one array and it keeps whatever the last call left.
//    Nothing in it has to start at zero: every slot a call reads, the same call has written
//    first. Two calls that overlap on the GPU (different streams, or graphs replayed side by
//    side) race on it; keep calls of this function on one stream, or order them yourself.
//  * It calls no cudaMalloc, cudaFree or other allocating routine, and takes inputs and
//    outputs exactly as dd_attention_rows does, minus the two scratch pointers.
#pragma once

#define DD_STATIC_SCRATCH_BYTES (8u << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Arguments as dd_attention_rows (attention_rows.cu) without part_o and part_ml.
// Returns 0, or non-zero with a message in dd_last_error().
int dd_attention_rows_static(const void* q, int q_stride, const void* cache, const int* tok_entry,
                             const int* tok_pos, const int* block_table, int max_blocks, void* out,
                             int out_stride, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                             int page_size, int n_pages, int window, float scale, int n_splits, int dtype,
                             int* error_flag, void* stream);

#ifdef __cplusplus
}
#endif
