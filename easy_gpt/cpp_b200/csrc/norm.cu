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

// delta_dtype / out_dtype: EG_F32 or EG_BF16.  rows may be null.  delta may be null.
EG_API int eg_add_rmsnorm(cudaStream_t stream, int delta_dtype, int out_dtype, float* residual, const void* delta,
                          const int* rows, const float* gain, void* out, int num_rows, int hidden, float eps) {
    if (num_rows <= 0) return 0;
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
