// Shared helpers of the sm_100a kernels.  Every launcher is an extern "C"
// function that takes raw device pointers and a stream, returns the
// cudaError_t of the launch as an int, and never allocates.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define EG_API extern "C" __attribute__((visibility("default")))

typedef __nv_bfloat16 bf16;

// dtype codes of the C interface
enum { EG_F32 = 0, EG_BF16 = 1 };

// bits a kernel may set in the device status word instead of faulting
enum {
    EG_STATUS_BAD_TOKEN = 1,      // token id outside [0, vocab)
    EG_STATUS_BAD_PAGE = 2,       // block table entry outside [0, num_pages) where a key was needed
    EG_STATUS_BAD_SLOT = 4,       // cache write position outside the pool
    EG_STATUS_WAIT_TIMEOUT = 8,   // a bounded wait on a barrier gave up
};

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order of the additions depends only on blockDim, never on the data or on what
// else is in the batch.  `scratch` holds 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    float r = (lane < nwarps) ? scratch[lane] : 0.0f;
    r = warp_sum(r);
    return r;
}

// Optional timeline of a launch: the earliest CTA start and the latest CTA end on the GPU's
// nanosecond clock, kept in trace[0] / trace[1] (the host presets them to ~0 / 0), and phase
// stamps of the first CTA in trace[2..15].  A null pointer costs one predicated branch.
struct TraceScope {
    unsigned long long* slot;
    __device__ __forceinline__ static unsigned long long now() {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        return t;
    }
    __device__ __forceinline__ explicit TraceScope(unsigned long long* s) : slot(s) {
        if (slot && threadIdx.x == 0) atomicMin(slot, now());
    }
    __device__ __forceinline__ ~TraceScope() {
        if (slot && threadIdx.x == 0) atomicMax(slot + 1, now());
    }
    // Phase stamps, i < 7: slot[2 + i] the latest over the launch's CTAs, slot[9 + i] the complement of the earliest
    // (so that zero means "none" for both).  every_warp: each warp's first lane stamps, not only the CTA's first thread.
    __device__ __forceinline__ void mark(int i, bool every_warp = false) const {
        if (slot && (every_warp ? (threadIdx.x & 31) == 0 : threadIdx.x == 0)) {
            const unsigned long long t = now();
            atomicMax(slot + 2 + i, t);
            atomicMax(slot + 9 + i, ~t);
        }
    }
};

static inline int eg_launch_status() { return (int)cudaGetLastError(); }

#ifdef EG_NEEDS_TENSOR_MAPS
#include <cuda.h>
// The driver's tensor-map encoder, looked up through the runtime at the first call: the library then has no
// link-time dependency on the driver and loads (for the build check) on a machine without one.
typedef CUresult (*eg_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                       const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                       CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static inline eg_encode_tiled_fn eg_encode_tiled() {
    static eg_encode_tiled_fn fn = nullptr;
    if (!fn) {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult found;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &found) == cudaSuccess &&
            found == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<eg_encode_tiled_fn>(entry);
    }
    return fn;
}
#endif
