// mbarrier helpers shared by the kernels that hand work over inside a CTA (TMA producers, tcgen05 issuers,
// epilogue warps).  Every wait is bounded: after `limit` polls the waiting thread raises the CTA's abort flag
// and EG_STATUS_WAIT_TIMEOUT in the status word and returns false; a thread that sees the abort flag raised by
// another returns false at once.  The caller's roles then leave their loops, wait (bounded again) for their own
// copies in flight, free the TMEM they hold and return, so the context stays usable and the host reads the
// status word.
#pragma once
#include "common.cuh"

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false if it gave up (or another role already did).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                                  unsigned limit) {
    for (unsigned i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    atomicOr(status, EG_STATUS_WAIT_TIMEOUT);
    return false;
}
