// Rotary position encoding of q and k, fused with the write of k and v into the
// paged cache.
//
// Input: one row per token holding [q heads | k heads | v heads], each head
// `head_dim` wide (the fused QKV projection's output), optionally still without
// its bias (then `bias` is added here in float32 first).  q is rotated in place;
// k is rotated and, like v, stored at the token's cache position.
//
// Rotation (src/ops.cpp:404-421, half rotation): for j < rotary_dim/2
//   a = float(pos) * inv_freq[j]
//   x'[j]              = x[j] cos a - x[j + rotary_dim/2] sin a
//   x'[j+rotary_dim/2] = x[j] sin a + x[j + rotary_dim/2] cos a
// The angle is a float32 product, cosf/sinf are the accurate ones; dimensions
// from rotary_dim on pass through.  inv_freq comes from the host so that every
// path shares one table.
//
// Cache layout: element (page, kv head, offset in page, d) of K lives at
//   k_cache[page * page_stride + head * head_stride + offset * head_dim + d].
// slot_map[t] = page * page_size + offset, or -1 when the token's key is not
// stored (a layer that reads another layer's cache).
#include "common.cuh"

template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, int ld, const float* __restrict__ bias,
                                  const int* __restrict__ positions, const int* __restrict__ slot_map,
                                  T* __restrict__ k_cache, T* __restrict__ v_cache, const float* __restrict__ inv_freq,
                                  int num_heads, int num_kv_heads, int head_dim, int rotary_dim, int page_size,
                                  long long page_stride, long long head_stride, long long pool_slots, int* status) {
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rotary_dim / 2;
    T* row = qkv + (size_t)t * ld;
    long long slot = slot_map ? slot_map[t] : -1;
    if (slot >= pool_slots) {
        if (threadIdx.x == 0) atomicOr(status, EG_STATUS_BAD_SLOT);
        slot = -1;
    }
    const long long page = slot >= 0 ? slot / page_size : 0;
    const int offset = slot >= 0 ? (int)(slot % page_size) : 0;

    const int rot_heads = num_heads + num_kv_heads;
    // rotated pairs of q and k
    for (int e = threadIdx.x; e < rot_heads * half; e += blockDim.x) {
        const int h = e / half, j = e % half;
        const int c0 = h * head_dim + j, c1 = c0 + half;
        float x0 = to_f32<T>(row[c0]), x1 = to_f32<T>(row[c1]);
        if (bias) { x0 += bias[c0]; x1 += bias[c1]; }
        const float a = (float)pos * inv_freq[j];
        const float c = cosf(a), s = sinf(a);
        // (one rounding of x1's product, then a fused multiply-add: spelt out so that every kernel that rotates gives
        // the same bits)
        const float y0 = __fmaf_rn(x0, c, -__fmul_rn(x1, s));
        const float y1 = __fmaf_rn(x0, s, __fmul_rn(x1, c));
        if (h < num_heads) {
            row[c0] = from_f32<T>(y0);
            row[c1] = from_f32<T>(y1);
        } else if (slot >= 0) {
            const int kh = h - num_heads;
            T* dst = k_cache + page * page_stride + kh * head_stride + (long long)offset * head_dim;
            dst[j] = from_f32<T>(y0);
            dst[j + half] = from_f32<T>(y1);
        }
    }
    // dimensions beyond the rotary part of q and k pass through (plus bias)
    const int rest = head_dim - rotary_dim;
    if (rest > 0) {
        for (int e = threadIdx.x; e < rot_heads * rest; e += blockDim.x) {
            const int h = e / rest, j = rotary_dim + e % rest;
            const int c0 = h * head_dim + j;
            float x0 = to_f32<T>(row[c0]);
            if (bias) x0 += bias[c0];
            if (h < num_heads) {
                row[c0] = from_f32<T>(x0);
            } else if (slot >= 0) {
                const int kh = h - num_heads;
                k_cache[page * page_stride + kh * head_stride + (long long)offset * head_dim + j] = from_f32<T>(x0);
            }
        }
    }
    // v: copy (plus bias)
    if (slot >= 0) {
        const int v0 = rot_heads * head_dim;
        for (int e = threadIdx.x; e < num_kv_heads * head_dim; e += blockDim.x) {
            const int kh = e / head_dim, j = e % head_dim;
            float x0 = to_f32<T>(row[v0 + e]);
            if (bias) x0 += bias[v0 + e];
            v_cache[page * page_stride + kh * head_stride + (long long)offset * head_dim + j] = from_f32<T>(x0);
        }
    }
}

// cos/sin of every (token, frequency) of a step, computed once and shared by all layers with the
// same rotary parameters: table[t][j] = (cos a, sin a), a = float(pos[t]) * inv_freq[j].
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float2* __restrict__ table, int tokens, int half) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= tokens * half) return;
    const float a = (float)positions[e / half] * inv_freq[e % half];
    table[e] = make_float2(cosf(a), sinf(a));
}

EG_API int eg_rope_table(cudaStream_t stream, const int* positions, const float* inv_freq, float* table, int tokens, int half) {
    if (tokens <= 0 || half <= 0) return 0;
    rope_table_kernel<<<(tokens * half + 255) / 256, 256, 0, stream>>>(positions, inv_freq, (float2*)table, tokens, half);
    return eg_launch_status();
}

// The same work as rope_cache_kernel for the common case (the whole head rotated, head size a multiple of 16 (bfloat16)
// or 8 (float32), cos/sin from the table, no bias left to add): a thread takes 16 bytes of the first half of a head and
// the 16 bytes of their partners in the second half; a block takes several tokens, so that the blocks are few and full.
template <typename T>
__global__ void __launch_bounds__(256) rope_cache_vec_kernel(T* __restrict__ qkv, int ld, const float2* __restrict__ table,
                                                             const int* __restrict__ slot_map, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                                             int tokens, int num_heads, int num_kv_heads, int head_dim, int page_size,
                                                             long long page_stride, long long head_stride, long long pool_slots, int* status) {
    constexpr int VEC = 16 / sizeof(T);                              // elements of a 16-byte access
    const int half = head_dim / 2, pieces = half / VEC;              // pieces of a head's first half
    const int rot_heads = num_heads + num_kv_heads;
    const int rot_work = rot_heads * pieces, v_work = num_kv_heads * head_dim / VEC;
    const int per_token = rot_work + v_work;
    for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < (long long)tokens * per_token; w += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(w / per_token), e = (int)(w % per_token);
        T* row = qkv + (size_t)t * ld;
        const bool rotated = e < rot_work;
        const int h = rotated ? e / pieces : (e - rot_work) * VEC / head_dim;
        const int j = rotated ? (e % pieces) * VEC : (e - rot_work) * VEC % head_dim;
        long long slot = -1;
        if (slot_map && (!rotated || h >= num_heads)) {
            slot = slot_map[t];
            if (slot >= pool_slots) {
                atomicOr(status, EG_STATUS_BAD_SLOT);
                slot = -1;
            }
        }
        const long long page = slot >= 0 ? slot / page_size : 0;
        const int offset = slot >= 0 ? (int)(slot % page_size) : 0;
        if (!rotated) {
            if (slot >= 0)
                *reinterpret_cast<uint4*>(v_cache + page * page_stride + (long long)h * head_stride + (long long)offset * head_dim + j) =
                    *reinterpret_cast<const uint4*>(row + (size_t)(rot_heads + h) * head_dim + j);
            continue;
        }
        T* p0 = row + (size_t)h * head_dim + j;
        T* p1 = p0 + half;
        const uint4 r0 = *reinterpret_cast<const uint4*>(p0), r1 = *reinterpret_cast<const uint4*>(p1);
        const float4* cs = reinterpret_cast<const float4*>(table + (size_t)t * half + j);       // (cos, sin) pairs, two a float4
        float x0[VEC], x1[VEC], y0[VEC], y1[VEC];
        if (sizeof(T) == 2) {
            const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&r0);
            const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&r1);
#pragma unroll
            for (int k = 0; k < VEC / 2; ++k) {
                x0[2 * k] = __low2float(a[k]); x0[2 * k + 1] = __high2float(a[k]);
                x1[2 * k] = __low2float(b[k]); x1[2 * k + 1] = __high2float(b[k]);
            }
        } else {
            const float* a = reinterpret_cast<const float*>(&r0);
            const float* b = reinterpret_cast<const float*>(&r1);
#pragma unroll
            for (int k = 0; k < VEC; ++k) { x0[k] = a[k]; x1[k] = b[k]; }
        }
#pragma unroll
        for (int k = 0; k < VEC; k += 2) {
            const float4 c = cs[k / 2];
            y0[k] = __fmaf_rn(x0[k], c.x, -__fmul_rn(x1[k], c.y));
            y1[k] = __fmaf_rn(x0[k], c.y, __fmul_rn(x1[k], c.x));
            y0[k + 1] = __fmaf_rn(x0[k + 1], c.z, -__fmul_rn(x1[k + 1], c.w));
            y1[k + 1] = __fmaf_rn(x0[k + 1], c.w, __fmul_rn(x1[k + 1], c.z));
        }
        uint4 o0, o1;
        if (sizeof(T) == 2) {
            __nv_bfloat162* a = reinterpret_cast<__nv_bfloat162*>(&o0);
            __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&o1);
#pragma unroll
            for (int k = 0; k < VEC / 2; ++k) {
                a[k] = __floats2bfloat162_rn(y0[2 * k], y0[2 * k + 1]);
                b[k] = __floats2bfloat162_rn(y1[2 * k], y1[2 * k + 1]);
            }
        } else {
            float* a = reinterpret_cast<float*>(&o0);
            float* b = reinterpret_cast<float*>(&o1);
#pragma unroll
            for (int k = 0; k < VEC; ++k) { a[k] = y0[k]; b[k] = y1[k]; }
        }
        if (h < num_heads) {
            *reinterpret_cast<uint4*>(p0) = o0;
            *reinterpret_cast<uint4*>(p1) = o1;
        } else if (slot >= 0) {
            T* dst = k_cache + page * page_stride + (long long)(h - num_heads) * head_stride + (long long)offset * head_dim + j;
            *reinterpret_cast<uint4*>(dst) = o0;
            *reinterpret_cast<uint4*>(dst + half) = o1;
        }
    }
}

EG_API int eg_rope_cache_vec(cudaStream_t stream, int dtype, void* qkv, int ld, const float* table, const int* slot_map,
                             void* k_cache, void* v_cache, int tokens, int num_heads, int num_kv_heads, int head_dim,
                             int page_size, long long page_stride, long long head_stride, long long pool_slots, int* status) {
    if (tokens <= 0) return 0;
    const size_t es = dtype == EG_BF16 ? 2 : 4;
    const int vec = (int)(16 / es);
    // every 16-byte access must be aligned: rows of qkv, heads, halves of heads, cache rows, the table's rows
    if (head_dim % (2 * vec) || ((size_t)ld * es) % 16 || (uintptr_t)qkv % 16 || !table || (uintptr_t)table % 16 ||
        (slot_map && ((uintptr_t)k_cache % 16 || (uintptr_t)v_cache % 16 || (page_stride * es) % 16 || (head_stride * es) % 16)))
        return (int)cudaErrorInvalidValue;
    const long long work = (long long)tokens * ((num_heads + num_kv_heads) * (head_dim / 2 / vec) + num_kv_heads * head_dim / vec);
    const int threads = 256;
    const int blocks = (int)((work + threads - 1) / threads < (1 << 20) ? (work + threads - 1) / threads : (1 << 20));
    if (dtype == EG_BF16)
        rope_cache_vec_kernel<bf16><<<blocks, threads, 0, stream>>>((bf16*)qkv, ld, (const float2*)table, slot_map, (bf16*)k_cache, (bf16*)v_cache,
                                                                    tokens, num_heads, num_kv_heads, head_dim, page_size, page_stride,
                                                                    head_stride, pool_slots, status);
    else
        rope_cache_vec_kernel<float><<<blocks, threads, 0, stream>>>((float*)qkv, ld, (const float2*)table, slot_map, (float*)k_cache,
                                                                     (float*)v_cache, tokens, num_heads, num_kv_heads, head_dim, page_size,
                                                                     page_stride, head_stride, pool_slots, status);
    return eg_launch_status();
}

EG_API int eg_rope_cache(cudaStream_t stream, int dtype, void* qkv, int ld, const float* bias, const int* positions,
                         const int* slot_map, void* k_cache, void* v_cache, const float* inv_freq, int tokens,
                         int num_heads, int num_kv_heads, int head_dim, int rotary_dim, int page_size,
                         long long page_stride, long long head_stride, long long pool_slots, int* status) {
    if (tokens <= 0) return 0;
    if (rotary_dim % 2 || rotary_dim > head_dim || rotary_dim < 0) return (int)cudaErrorInvalidValue;
    const int threads = 128;
    if (dtype == EG_BF16)
        rope_cache_kernel<bf16><<<tokens, threads, 0, stream>>>((bf16*)qkv, ld, bias, positions, slot_map, (bf16*)k_cache,
                                                               (bf16*)v_cache, inv_freq, num_heads, num_kv_heads, head_dim,
                                                               rotary_dim, page_size, page_stride, head_stride, pool_slots, status);
    else
        rope_cache_kernel<float><<<tokens, threads, 0, stream>>>((float*)qkv, ld, bias, positions, slot_map, (float*)k_cache,
                                                                (float*)v_cache, inv_freq, num_heads, num_kv_heads, head_dim,
                                                                rotary_dim, page_size, page_stride, head_stride, pool_slots, status);
    return eg_launch_status();
}
