// Two elementwise kernels of the layer shapes that are not pre-norm (a norm behind a part, a norm on a part's output,
// no norm at all): adding a part's output into the float32 residual stream, and converting rows between float32 and
// the compute dtype.  The pre-norm shape needs neither: its additions ride in the norm kernels.
#include "common.cuh"

namespace {
template <typename TD>
__global__ void add_into_f32_kernel(float* __restrict__ residual, const TD* __restrict__ delta, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) residual[i] += to_f32<TD>(delta[i]);
}
template <typename TS, typename TD>
__global__ void convert_rows_kernel(const TS* __restrict__ src, TD* __restrict__ dst, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = from_f32<TD>(to_f32<TS>(src[i]));
}
}  // namespace

// residual[i] += delta[i], i < n; delta_dtype: EG_F32 or EG_BF16
EG_API int eg_add_into_f32(cudaStream_t stream, float* residual, const void* delta, int delta_dtype, long long n) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (delta_dtype == EG_BF16) add_into_f32_kernel<bf16><<<blocks, 256, 0, stream>>>(residual, (const bf16*)delta, n);
    else add_into_f32_kernel<float><<<blocks, 256, 0, stream>>>(residual, (const float*)delta, n);
    return eg_launch_status();
}

// dst[i] = src[i] converted, i < n; dtypes: EG_F32 or EG_BF16
EG_API int eg_convert_rows(cudaStream_t stream, const void* src, int src_dtype, void* dst, int dst_dtype, long long n) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (src_dtype == EG_F32 && dst_dtype == EG_BF16) convert_rows_kernel<float, bf16><<<blocks, 256, 0, stream>>>((const float*)src, (bf16*)dst, n);
    else if (src_dtype == EG_BF16 && dst_dtype == EG_F32) convert_rows_kernel<bf16, float><<<blocks, 256, 0, stream>>>((const bf16*)src, (float*)dst, n);
    else if (src_dtype == EG_F32) convert_rows_kernel<float, float><<<blocks, 256, 0, stream>>>((const float*)src, (float*)dst, n);
    else convert_rows_kernel<bf16, bf16><<<blocks, 256, 0, stream>>>((const bf16*)src, (bf16*)dst, n);
    return eg_launch_status();
}
