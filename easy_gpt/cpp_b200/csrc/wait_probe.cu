// A kernel whose only work is a wait that nothing ends: every thread of one CTA waits on an mbarrier on
// which nobody arrives, through the same bounded wait that the TMA/tcgen05 kernels use (mbarrier.cuh), with
// the poll limit given by the caller.  It shows, on a healthy GPU and in a few microseconds, what a wait
// that runs out does: the first thread to reach the limit raises the abort flag and EG_STATUS_WAIT_TIMEOUT,
// the others see the flag and leave, the kernel returns, and the context goes on working.  For tests and
// for checking an installation; no product path launches it.
#include "mbarrier.cuh"

namespace {
__global__ void wait_probe_kernel(unsigned limit, int* status, int* gave_up) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    const bool ok = mbar_wait_bounded(&bar, 0, &abort_flag, status, limit);      // phase 0 never completes
    if (!ok) atomicAdd(gave_up, 1);
}
}  // namespace

// gave_up[0] is increased by the number of threads whose wait returned false (all `threads` of them).
EG_API int eg_wait_probe(cudaStream_t stream, unsigned limit, int threads, int* status, int* gave_up) {
    if (!status || !gave_up || threads < 1 || threads > 1024 || limit < 1 || limit > (1u << 20)) return (int)cudaErrorInvalidValue;
    wait_probe_kernel<<<1, threads, 0, stream>>>(limit, status, gave_up);
    return eg_launch_status();
}
