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

// Four outputs per thread: one 16-byte (bfloat16) or two 16-byte (float32) loads, one vector store.
template <typename T>
__global__ void swiglu_vec4_kernel(const T* __restrict__ gate_up, int ld, T* __restrict__ out, int ldo, int inter) {
    const int t = blockIdx.x;
    const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (i >= inter) return;
    const T* row = gate_up + (size_t)t * ld + 2 * i;
    float v[8];
    if (sizeof(T) == 2) {
        const uint4 raw = *reinterpret_cast<const uint4*>(row);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            v[2 * k] = __low2float(h[k]);
            v[2 * k + 1] = __high2float(h[k]);
        }
    } else {
        const float4 a = reinterpret_cast<const float4*>(row)[0], b = reinterpret_cast<const float4*>(row)[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    float r[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float g = v[2 * k], u = v[2 * k + 1];
        r[k] = u * (g * (1.0f / (1.0f + expf(-g))));
    }
    T* o = out + (size_t)t * ldo + i;
    if (sizeof(T) == 2) {
        uint2 packed;
        __nv_bfloat162 lo = __floats2bfloat162_rn(r[0], r[1]), hi = __floats2bfloat162_rn(r[2], r[3]);
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(o) = packed;
    } else {
        *reinterpret_cast<float4*>(o) = make_float4(r[0], r[1], r[2], r[3]);
    }
}

EG_API int eg_swiglu(cudaStream_t stream, int dtype, const void* gate_up, int ld, void* out, int ldo, int tokens, int inter) {
    if (tokens <= 0) return 0;
    const size_t es = dtype == EG_BF16 ? 2 : 4;
    if (inter % 4 == 0 && ((size_t)ld * es) % 16 == 0 && ((size_t)ldo * es) % (4 * es) == 0 &&
        ((uintptr_t)gate_up % 16) == 0 && ((uintptr_t)out % (4 * es)) == 0) {
        dim3 vgrid(tokens, (inter / 4 + 127) / 128);
        if (dtype == EG_BF16)
            swiglu_vec4_kernel<bf16><<<vgrid, 128, 0, stream>>>((const bf16*)gate_up, ld, (bf16*)out, ldo, inter);
        else
            swiglu_vec4_kernel<float><<<vgrid, 128, 0, stream>>>((const float*)gate_up, ld, (float*)out, ldo, inter);
        return eg_launch_status();
    }
    dim3 grid(tokens, (inter + 255) / 256);
    if (dtype == EG_BF16)
        swiglu_kernel<bf16><<<grid, 256, 0, stream>>>((const bf16*)gate_up, ld, (bf16*)out, ldo, inter);
    else
        swiglu_kernel<float><<<grid, 256, 0, stream>>>((const float*)gate_up, ld, (float*)out, ldo, inter);
    return eg_launch_status();
}
