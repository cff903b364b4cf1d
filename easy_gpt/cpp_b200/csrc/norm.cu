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

// Rows of up to 4096 values that are a multiple of 4 wide: a warp per row, VPL float4 per lane kept in registers, so that
// the row is read once, all of its loads are in flight at once, the sum is a shuffle, and nothing waits at a barrier.
// (Measured on B200, 2,048 rows of 896: 5.6 us a launch with a block per row and a sum through shared memory.)
// The sum's order (a lane's values in order, then the lanes by halving) depends on the width alone.
template <typename TD, typename TO, int VPL>
__global__ void __launch_bounds__(256) add_rmsnorm_warp_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                                               const int* __restrict__ rows, const float* __restrict__ gain,
                                                               TO* __restrict__ out, int num_rows, int hidden, float eps) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= num_rows) return;
    const int src = rows ? rows[r] : r;
    const int quads = hidden / 4;
    float4* x = reinterpret_cast<float4*>(residual + (size_t)src * hidden);
    float4 v[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int q = i * 32 + lane;
        v[i] = q < quads ? x[q] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (delta) {
        if (sizeof(TD) == 2) {
            const uint2* d = reinterpret_cast<const uint2*>(delta + (size_t)src * hidden);
            uint2 raw[VPL];
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                const int q = i * 32 + lane;
                raw[i] = q < quads ? d[q] : make_uint2(0u, 0u);
            }
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw[i].x);
                const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw[i].y);
                v[i].x += __low2float(a); v[i].y += __high2float(a); v[i].z += __low2float(b); v[i].w += __high2float(b);
            }
        } else {
            const float4* d = reinterpret_cast<const float4*>(delta + (size_t)src * hidden);
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                const int q = i * 32 + lane;
                if (q < quads) {
                    const float4 dv = d[q];
                    v[i].x += dv.x; v[i].y += dv.y; v[i].z += dv.z; v[i].w += dv.w;
                }
            }
        }
        if (!rows) {
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                const int q = i * 32 + lane;
                if (q < quads) x[q] = v[i];
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    const float4* g = reinterpret_cast<const float4*>(gain);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int q = i * 32 + lane;
        if (q >= quads) continue;
        const float4 gv = g[q];
        const float y0 = gv.x * (v[i].x * inv), y1 = gv.y * (v[i].y * inv), y2 = gv.z * (v[i].z * inv), y3 = gv.w * (v[i].w * inv);
        if (sizeof(TO) == 2) {
            uint2 packed;
            __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
            packed.x = *reinterpret_cast<uint32_t*>(&lo);
            packed.y = *reinterpret_cast<uint32_t*>(&hi);
            reinterpret_cast<uint2*>(out + (size_t)r * hidden)[q] = packed;
        } else {
            reinterpret_cast<float4*>(out + (size_t)r * hidden)[q] = make_float4(y0, y1, y2, y3);
        }
    }
}

template <typename TD, typename TO>
static void launch_warp_norm(cudaStream_t stream, float* residual, const void* delta, const int* rows, const float* gain, void* out, int num_rows,
                             int hidden, float eps) {
    const int vpl = (hidden / 4 + 31) / 32;
    // few rows: a warp a block, so that they are spread over the SMs (64 rows: 1.72 ms a decode step with eight warps a
    // block, 1.58 with one)
    const int warps = num_rows >= 2048 ? 8 : num_rows >= 512 ? 2 : 1, blocks = (num_rows + warps - 1) / warps;
#define EG_WARP_NORM(V) \
    add_rmsnorm_warp_kernel<TD, TO, V><<<blocks, warps * 32, 0, stream>>>(residual, (const TD*)delta, rows, gain, (TO*)out, num_rows, hidden, eps)
    if (vpl <= 4) EG_WARP_NORM(4);
    else if (vpl <= 8) EG_WARP_NORM(8);
    else if (vpl <= 16) EG_WARP_NORM(16);
    else EG_WARP_NORM(32);
#undef EG_WARP_NORM
}

// delta_dtype / out_dtype: EG_F32 or EG_BF16.  rows may be null.  delta may be null.
EG_API int eg_add_rmsnorm(cudaStream_t stream, int delta_dtype, int out_dtype, float* residual, const void* delta,
                          const int* rows, const float* gain, void* out, int num_rows, int hidden, float eps) {
    if (num_rows <= 0) return 0;
    if (hidden % 4 == 0 && hidden <= 4096 && (uintptr_t)residual % 16 == 0 && (uintptr_t)gain % 16 == 0 &&
        (uintptr_t)out % 16 == 0 && (!delta || (uintptr_t)delta % 16 == 0)) {
        if (delta_dtype == EG_BF16 && out_dtype == EG_BF16) launch_warp_norm<bf16, bf16>(stream, residual, delta, rows, gain, out, num_rows, hidden, eps);
        else if (delta_dtype == EG_F32 && out_dtype == EG_F32) launch_warp_norm<float, float>(stream, residual, delta, rows, gain, out, num_rows, hidden, eps);
        else if (delta_dtype == EG_BF16 && out_dtype == EG_F32) launch_warp_norm<bf16, float>(stream, residual, delta, rows, gain, out, num_rows, hidden, eps);
        else launch_warp_norm<float, bf16>(stream, residual, delta, rows, gain, out, num_rows, hidden, eps);
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
