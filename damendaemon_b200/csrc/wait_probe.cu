// A wait that nobody answers, to show what the pipelined kernels do when one of their waits runs out: one block
// sets up an mbarrier that expects one arrival, lets nobody arrive, and waits on it through tc::mbar_wait, the
// function every TMA and tensor-core pipeline of this library waits with, under a limit of the caller's choosing
// (the kernels' own limit is tc::WAIT_LIMIT_NS). The wait gives up, the block reports it as the kernels do (bit 8
// of the error word) and returns; nothing is in flight, so there is nothing to drain. A second warp waits on the
// same barrier and must leave through the block's abort flag, as the other roles of a pipeline do.
#include "common.cuh"
#include "tcgen05.cuh"

namespace {
__global__ void wait_probe_kernel(unsigned long long limit_ns, int* error_flag, unsigned long long* waited_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        tc::mbar_init(&bar, 1);
        tc::fence_barrier_init();
    }
    __syncthreads();
    const unsigned long long start = tc::global_ns();
    bool done = true;
    if ((threadIdx.x & 31) == 0)        // warp 0 gives up at the limit; warp 1 has ten times as long and leaves with it
        done = tc::mbar_wait(&bar, 0, &abort_flag, threadIdx.x == 0 ? limit_ns : 10 * limit_ns);
    const unsigned long long waited = tc::global_ns() - start;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) waited_ns[threadIdx.x >> 5] = done ? 0 : waited;
    if (threadIdx.x == 0 && abort_flag) atomicOr(error_flag, 8);
}
}  // namespace

// limit_ns: at most one second. waited_ns: two values, how long each of the two waiting warps waited before it gave
// up (0 if its wait, against all expectation, succeeded).
DD_API int dd_wait_probe(unsigned long long limit_ns, int* error_flag, unsigned long long* waited_ns, void* stream) {
    if (limit_ns == 0 || limit_ns > 1000000000ull) return dd_fail("dd_wait_probe: the limit must be between 1 ns and 1 s");
    if (!error_flag || !waited_ns) return dd_fail("dd_wait_probe: null argument");
    wait_probe_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(limit_ns, error_flag, waited_ns);
    return dd_check_launch("dd_wait_probe");
}
