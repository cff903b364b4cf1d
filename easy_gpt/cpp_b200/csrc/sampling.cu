// Sampling on float32 logits, one block per row.
//
// Greedy: the lowest index among the maxima (std::max_element over the
// probabilities in the reference, src/sampler.cpp:13-20; the softmax is
// monotonic, so the logits give the same token).
#include "common.cuh"

namespace {
constexpr int SAMPLE_THREADS = 1024;
}

struct ArgMax {
    float v;
    int i;
};

__device__ __forceinline__ ArgMax argmax_better(ArgMax a, ArgMax b) {
    // larger value wins; on a tie the lower index
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ __forceinline__ ArgMax block_argmax(ArgMax a, ArgMax* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b;
        b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
        a = argmax_better(a, b);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = a;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    ArgMax r;
    r.v = -INFINITY;
    r.i = 0x7fffffff;
    if (lane < nwarps) r = scratch[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b;
        b.v = __shfl_xor_sync(0xffffffffu, r.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, r.i, o);
        r = argmax_better(r, b);
    }
    return r;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, long long ld, int vocab, int* __restrict__ out) {
    __shared__ ArgMax scratch[32];
    const float* row = logits + (size_t)blockIdx.x * ld;
    ArgMax best;
    best.v = -INFINITY;
    best.i = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        ArgMax c;
        c.v = row[i];
        c.i = i;
        // NaN never wins; a row of NaNs yields index 0 below
        if (c.v == c.v) best = argmax_better(best, c);
    }
    best = block_argmax(best, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = best.i == 0x7fffffff ? 0 : best.i;
}

EG_API int eg_argmax(cudaStream_t stream, const float* logits, long long ld, int rows, int vocab, int* out) {
    if (rows <= 0) return 0;
    argmax_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, ld, vocab, out);
    return eg_launch_status();
}
