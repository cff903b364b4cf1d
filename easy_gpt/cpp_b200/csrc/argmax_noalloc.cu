// eg_argmax_noalloc: the multi-block argmax of sampling.cu with its scratch memory in a
// file-scope device array instead of caller-provided buffers.  See argmax_noalloc.h for who
// needs this and for the rules; it has no counterpart in the reference.
#include "argmax_noalloc.h"

#include <mutex>

#include "common.cuh"

namespace {

constexpr int BLOCKS_PER_ROW = 32;
constexpr int THREADS = 1024;
constexpr int MAX_DEVICES = 64;

// Scratch of every call on this device: per row, BLOCKS_PER_ROW partial maxima and their indices, and one
// ticket counter.  In HOST code the name `noalloc_scratch` is only a handle for the runtime, not an address a
// kernel could use; the device address comes from cudaGetSymbolAddress below.
struct Scratch {
    float part_val[EG_ARGMAX_NOALLOC_MAX_ROWS * BLOCKS_PER_ROW];
    int part_idx[EG_ARGMAX_NOALLOC_MAX_ROWS * BLOCKS_PER_ROW];
    int counters[EG_ARGMAX_NOALLOC_MAX_ROWS];
};
static __device__ __align__(256) Scratch noalloc_scratch;

struct Best {
    float v;
    int i;
};

__device__ __forceinline__ Best better(Best a, Best b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;          // ties: the lower index
}

__device__ __forceinline__ Best block_best(Best a, Best* shared) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best b;
        b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
        a = better(a, b);
    }
    __syncthreads();
    if (lane == 0) shared[warp] = a;
    __syncthreads();
    Best r;
    r.v = -INFINITY;
    r.i = 0x7fffffff;
    if (lane < (int)(blockDim.x >> 5)) r = shared[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best b;
        b.v = __shfl_xor_sync(0xffffffffu, r.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, r.i, o);
        r = better(r, b);
    }
    return r;
}

__global__ void __launch_bounds__(THREADS)
argmax_noalloc_kernel(const float* __restrict__ logits, long long ld, int vocab, int* __restrict__ out, Scratch* scratch) {
    __shared__ Best shared[32];
    __shared__ int is_last;
    const int r = blockIdx.x, nb = gridDim.y;
    const float* row = logits + (size_t)r * ld;
    const int per = (vocab + nb - 1) / nb;
    const int lo = blockIdx.y * per, hi = min(vocab, lo + per);
    Best best;
    best.v = -INFINITY;
    best.i = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        Best c;
        c.v = row[i];
        c.i = i;
        if (c.v == c.v) best = better(best, c);                        // NaN never wins
    }
    best = block_best(best, shared);
    if (threadIdx.x == 0) {
        scratch->part_val[r * BLOCKS_PER_ROW + blockIdx.y] = best.v;
        scratch->part_idx[r * BLOCKS_PER_ROW + blockIdx.y] = best.i;
        __threadfence();
        is_last = atomicAdd(&scratch->counters[r], 1) == nb - 1;       // the block that arrives last finishes the row
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    Best a;
    a.v = -INFINITY;
    a.i = 0x7fffffff;
    if ((int)threadIdx.x < nb) {
        a.v = __ldcg(&scratch->part_val[r * BLOCKS_PER_ROW + threadIdx.x]);
        a.i = __ldcg(&scratch->part_idx[r * BLOCKS_PER_ROW + threadIdx.x]);
        if (a.i == 0x7fffffff) a.v = -INFINITY;
    }
    a = block_best(a, shared);
    if (threadIdx.x == 0) out[r] = a.i == 0x7fffffff ? 0 : a.i;
}

std::mutex setup_mutex;
Scratch* device_scratch[MAX_DEVICES] = {};     // device address of noalloc_scratch, per device, once looked up

}  // namespace

EG_API int eg_argmax_noalloc(cudaStream_t stream, const float* logits, long long ld, int rows, int vocab, int* out) {
    if (rows == 0) return 0;
    if (rows < 0 || vocab < 1 || !logits || !out || ld < vocab) return EG_NOALLOC_BAD_ARGUMENT;
    if (rows > EG_ARGMAX_NOALLOC_MAX_ROWS) return EG_NOALLOC_TOO_MANY_ROWS;
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= MAX_DEVICES) return EG_NOALLOC_BAD_ARGUMENT;
    Scratch* scratch;
    {
        // set-up, once per device, with that device current: the array's address on THIS device
        std::lock_guard<std::mutex> lock(setup_mutex);
        if (!device_scratch[device]) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, noalloc_scratch);
            if (e != cudaSuccess) return (int)e;
            device_scratch[device] = static_cast<Scratch*>(p);
        }
        scratch = device_scratch[device];
    }
    // The tickets must start at zero whatever an earlier (perhaps failed) call left; the partial results are
    // written before they are read and need no clearing.
    e = cudaMemsetAsync(scratch->counters, 0, sizeof(int) * rows, stream);
    if (e != cudaSuccess) return (int)e;
    const int blocks = vocab >= 4096 * 2 ? (vocab / 4096 < BLOCKS_PER_ROW ? vocab / 4096 : BLOCKS_PER_ROW) : 1;
    argmax_noalloc_kernel<<<dim3(rows, blocks), THREADS, 0, stream>>>(logits, ld, vocab, out, scratch);
    return (int)cudaGetLastError();
}

EG_API const char* eg_argmax_noalloc_message(int code) {
    switch (code) {
        case 0: return "ok";
        case EG_NOALLOC_TOO_MANY_ROWS:
            return "eg_argmax_noalloc takes at most 256 rows per call (EG_ARGMAX_NOALLOC_MAX_ROWS): its scratch is a "
                   "fixed device array; split the batch or use eg_argmax with scratch of your own";
        case EG_NOALLOC_BAD_ARGUMENT:
            return "eg_argmax_noalloc: null pointer, negative row count, vocabulary < 1, row stride below the "
                   "vocabulary, or a device index beyond 63";
        default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "eg_argmax_noalloc: unknown code";
    }
}
