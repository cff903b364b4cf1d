// Residual add fused with RMSNorm.
//   residual[r, :] += delta[r, :]            (float32 residual stream, skipped when delta is null)
//   out[r, :] = gain * (residual[r, :] * 1/sqrt(mean(residual[r, :]^2) + eps))
// The formula and its order are the reference's (src/models/norm.cpp:46-60); the
// sum of squares, the mean, the square root and the division are float32 and
// correctly rounded (no fast-math).  With `rows` given, output row r is computed
// from residual row rows[r] (the final norm runs only where logits are wanted)
// and the residual is left untouched.
#include "common.cuh"

template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                   const int* __restrict__ rows, const float* __restrict__ gain,
                                   TO* __restrict__ out, int hidden, float eps) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* x = residual + (size_t)src * hidden;
    const TD* d = delta ? delta + (size_t)src * hidden : nullptr;
    const bool write_back = (rows == nullptr) && (d != nullptr);
    float ss = 0.0f;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float v = x[j];
        if (d) v += to_f32<TD>(d[j]);
        if (write_back) x[j] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float mean_sq = ss / (float)hidden;
    const float inv = 1.0f / sqrtf(mean_sq + eps);
    TO* o = out + (size_t)r * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float v = x[j];
        if (d && !write_back) v += to_f32<TD>(d[j]);
        o[j] = from_f32<TO>(gain[j] * (v * inv));
    }
}

// Rows of up to 4096 values that are a multiple of 4 wide: every thread keeps its four values in
// registers between the sum and the scaling, so the row is read once.
template <typename TD, typename TO>
__global__ void add_rmsnorm_vec4_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                        const int* __restrict__ rows, const float* __restrict__ gain,
                                        TO* __restrict__ out, int hidden, float eps) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    const int i = threadIdx.x;
    const bool active = i * 4 < hidden;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (active) {
        v = reinterpret_cast<const float4*>(residual + (size_t)src * hidden)[i];
        if (delta) {
            if (sizeof(TD) == 2) {
                const uint2 raw = reinterpret_cast<const uint2*>(delta + (size_t)src * hidden)[i];
                const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
                const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
                v.x += __low2float(a); v.y += __high2float(a); v.z += __low2float(b); v.w += __high2float(b);
            } else {
                const float4 d = reinterpret_cast<const float4*>(delta + (size_t)src * hidden)[i];
                v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
            }
            if (!rows) reinterpret_cast<float4*>(residual + (size_t)src * hidden)[i] = v;
        }
    }
    const float ss = block_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    if (active) {
        const float4 g = reinterpret_cast<const float4*>(gain)[i];
        const float y0 = g.x * (v.x * inv), y1 = g.y * (v.y * inv), y2 = g.z * (v.z * inv), y3 = g.w * (v.w * inv);
        if (sizeof(TO) == 2) {
            uint2 packed;
            __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
            packed.x = *reinterpret_cast<uint32_t*>(&lo);
            packed.y = *reinterpret_cast<uint32_t*>(&hi);
            reinterpret_cast<uint2*>(out + (size_t)r * hidden)[i] = packed;
        } else {
            reinterpret_cast<float4*>(out + (size_t)r * hidden)[i] = make_float4(y0, y1, y2, y3);
        }
    }
}

// delta_dtype / out_dtype: EG_F32 or EG_BF16.  rows may be null.  delta may be null.
EG_API int eg_add_rmsnorm(cudaStream_t stream, int delta_dtype, int out_dtype, float* residual, const void* delta,
                          const int* rows, const float* gain, void* out, int num_rows, int hidden, float eps) {
    if (num_rows <= 0) return 0;
    if (hidden % 4 == 0 && hidden <= 4096 && (uintptr_t)residual % 16 == 0 && (uintptr_t)gain % 16 == 0 &&
        (uintptr_t)out % 16 == 0 && (!delta || (uintptr_t)delta % 16 == 0)) {
        const int vthreads = ((hidden / 4 + 31) / 32) * 32;
#define EG_NORM_VEC(TD, TO) \
    add_rmsnorm_vec4_kernel<TD, TO><<<num_rows, vthreads, 0, stream>>>(residual, (const TD*)delta, rows, gain, (TO*)out, hidden, eps)
        if (delta_dtype == EG_BF16 && out_dtype == EG_BF16) EG_NORM_VEC(bf16, bf16);
        else if (delta_dtype == EG_F32 && out_dtype == EG_F32) EG_NORM_VEC(float, float);
        else if (delta_dtype == EG_BF16 && out_dtype == EG_F32) EG_NORM_VEC(bf16, float);
        else EG_NORM_VEC(float, bf16);
#undef EG_NORM_VEC
        return eg_launch_status();
    }
    int threads = 128;
    while (threads < 1024 && threads * 4 < hidden) threads <<= 1;
#define EG_NORM_LAUNCH(TD, TO) \
    add_rmsnorm_kernel<TD, TO><<<num_rows, threads, 0, stream>>>(residual, (const TD*)delta, rows, gain, (TO*)out, hidden, eps)
    if (delta_dtype == EG_BF16 && out_dtype == EG_BF16) EG_NORM_LAUNCH(bf16, bf16);
    else if (delta_dtype == EG_F32 && out_dtype == EG_F32) EG_NORM_LAUNCH(float, float);
    else if (delta_dtype == EG_BF16 && out_dtype == EG_F32) EG_NORM_LAUNCH(bf16, float);
    else EG_NORM_LAUNCH(float, bf16);
#undef EG_NORM_LAUNCH
    return eg_launch_status();
}
