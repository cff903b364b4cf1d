// SwiGLU on the fused gate/up projection: out[t, i] = up[t, i] * silu(gate[t, i]),
// silu(g) = g * 1/(1 + exp(-g)) in float32 (src/tensor.cpp:159-174,
// src/cuda/ops/mlp.cu:152-162).  The projection's rows are interleaved, so the
// input row is [gate_0, up_0, gate_1, up_1, ...]: a tile of the product holds both
// halves of every output it covers, which lets the decode kernel apply this in its epilogue.
#include "common.cuh"

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, int ld, T* __restrict__ out, int ldo, int inter) {
    const int t = blockIdx.x;
    const int i = blockIdx.y * blockDim.x + threadIdx.x;
    if (i >= inter) return;
    const T* row = gate_up + (size_t)t * ld;
    const float g = to_f32<T>(row[2 * i]);
    const float u = to_f32<T>(row[2 * i + 1]);
    const float sig = 1.0f / (1.0f + expf(-g));
    out[(size_t)t * ldo + i] = from_f32<T>(u * (g * sig));
}

EG_API int eg_swiglu(cudaStream_t stream, int dtype, const void* gate_up, int ld, void* out, int ldo, int tokens, int inter) {
    if (tokens <= 0) return 0;
    dim3 grid(tokens, (inter + 255) / 256);
    if (dtype == EG_BF16)
        swiglu_kernel<bf16><<<grid, 256, 0, stream>>>((const bf16*)gate_up, ld, (bf16*)out, ldo, inter);
    else
        swiglu_kernel<float><<<grid, 256, 0, stream>>>((const float*)gate_up, ld, (float*)out, ldo, inter);
    return eg_launch_status();
}
