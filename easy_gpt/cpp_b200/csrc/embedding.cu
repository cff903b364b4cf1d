// Token embedding: residual[t, :] = table[id[t], :] widened to float32.
// The reference gathers rows on the CPU with a range check that throws
// (src/models/embedding.cpp:54-76); here a bad id sets a status bit and the row
// becomes zero, so that the kernel never reads outside the table.
#include "common.cuh"

template <typename T>
__global__ void embedding_gather_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                        float* __restrict__ residual, int hidden, int vocab, int* status) {
    const int t = blockIdx.x;
    const int id = ids[t];
    float* out = residual + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, EG_STATUS_BAD_TOKEN);
        for (int j = threadIdx.x; j < hidden; j += blockDim.x) out[j] = 0.0f;
        return;
    }
    const T* row = table + (size_t)id * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) out[j] = to_f32<T>(row[j]);
}

EG_API int eg_embedding_gather(cudaStream_t stream, int dtype, const int* ids, const void* table, float* residual,
                               int tokens, int hidden, int vocab, int* status) {
    if (tokens <= 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == EG_BF16)
        embedding_gather_kernel<bf16><<<tokens, threads, 0, stream>>>(ids, (const bf16*)table, residual, hidden, vocab, status);
    else
        embedding_gather_kernel<float><<<tokens, threads, 0, stream>>>(ids, (const float*)table, residual, hidden, vocab, status);
    return eg_launch_status();
}
