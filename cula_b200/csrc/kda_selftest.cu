// Self-test of the bounded wait all pipelines of the library are built on: one warp waits on an mbarrier that
// nothing ever completes; the wait must run out after `limit` polls, record STATUS_WAIT_TIMEOUT and let the kernel
// return, leaving the context usable. No counterpart in the reference (its device code has no bounded waits).
#include "kda_common.cuh"

namespace kda {

__global__ void kda_selftest_wait_kernel(int* status, int limit) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0 && !mbar_wait(&bar, 0, limit)) atomicExch(status, STATUS_WAIT_TIMEOUT);
}

}  // namespace kda

extern "C" int kda_launch_selftest_wait(int* status, int limit, cudaStream_t stream) {
    kda::kda_selftest_wait_kernel<<<1, 32, 0, stream>>>(status, limit);
    return (int)cudaGetLastError();
}
