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
        const float y0 = x0 * c - x1 * s;
        const float y1 = x0 * s + x1 * c;
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

// The same work as rope_cache_kernel for the common case (the whole head rotated, head size a multiple
// of 8, cos/sin from the table, no bias left to add): four rotation pairs per thread, 8-byte accesses.
template <typename T>
__global__ void rope_cache_vec_kernel(T* __restrict__ qkv, int ld, const float2* __restrict__ table,
                                      const int* __restrict__ slot_map, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                      int num_heads, int num_kv_heads, int head_dim, int page_size, long long page_stride,
                                      long long head_stride, long long pool_slots, int* status) {
    const int t = blockIdx.x;
    const int half = head_dim / 2, quads = half / 4;
    T* row = qkv + (size_t)t * ld;
    long long slot = slot_map ? slot_map[t] : -1;
    if (slot >= pool_slots) {
        if (threadIdx.x == 0) atomicOr(status, EG_STATUS_BAD_SLOT);
        slot = -1;
    }
    const long long page = slot >= 0 ? slot / page_size : 0;
    const int offset = slot >= 0 ? (int)(slot % page_size) : 0;
    const int rot_heads = num_heads + num_kv_heads;
    const float2* cs = table + (size_t)t * half;

    auto load4 = [](const T* p, float (&v)[4]) {
        if (sizeof(T) == 2) {
            const uint2 raw = *reinterpret_cast<const uint2*>(p);
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
            const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
            v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
        } else {
            const float4 f = *reinterpret_cast<const float4*>(p);
            v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        }
    };
    auto store4 = [](T* p, const float (&v)[4]) {
        if (sizeof(T) == 2) {
            uint2 raw;
            __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
            raw.x = *reinterpret_cast<uint32_t*>(&a);
            raw.y = *reinterpret_cast<uint32_t*>(&b);
            *reinterpret_cast<uint2*>(p) = raw;
        } else {
            *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        }
    };

    for (int e = threadIdx.x; e < rot_heads * quads; e += blockDim.x) {
        const int h = e / quads, j = (e % quads) * 4;
        float x0[4], x1[4], y0[4], y1[4];
        load4(row + h * head_dim + j, x0);
        load4(row + h * head_dim + j + half, x1);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 c = cs[j + k];
            y0[k] = x0[k] * c.x - x1[k] * c.y;
            y1[k] = x0[k] * c.y + x1[k] * c.x;
        }
        if (h < num_heads) {
            store4(row + h * head_dim + j, y0);
            store4(row + h * head_dim + j + half, y1);
        } else if (slot >= 0) {
            T* dst = k_cache + page * page_stride + (long long)(h - num_heads) * head_stride + (long long)offset * head_dim;
            store4(dst + j, y0);
            store4(dst + j + half, y1);
        }
    }
    if (slot >= 0) {
        const int v0 = rot_heads * head_dim;
        for (int e = threadIdx.x; e < num_kv_heads * head_dim / 4; e += blockDim.x) {
            const int kh = (e * 4) / head_dim, j = (e * 4) % head_dim;
            float x[4];
            load4(row + v0 + kh * head_dim + j, x);
            store4(v_cache + page * page_stride + (long long)kh * head_stride + (long long)offset * head_dim + j, x);
        }
    }
}

EG_API int eg_rope_cache_vec(cudaStream_t stream, int dtype, void* qkv, int ld, const float* table, const int* slot_map,
                             void* k_cache, void* v_cache, int tokens, int num_heads, int num_kv_heads, int head_dim,
                             int page_size, long long page_stride, long long head_stride, long long pool_slots, int* status) {
    if (tokens <= 0) return 0;
    const size_t es = dtype == EG_BF16 ? 2 : 4;
    if (head_dim % 8 || ((size_t)ld * es) % (4 * es) || (uintptr_t)qkv % (4 * es) || !table) return (int)cudaErrorInvalidValue;
    if (dtype == EG_BF16)
        rope_cache_vec_kernel<bf16><<<tokens, 128, 0, stream>>>((bf16*)qkv, ld, (const float2*)table, slot_map, (bf16*)k_cache,
                                                                (bf16*)v_cache, num_heads, num_kv_heads, head_dim, page_size,
                                                                page_stride, head_stride, pool_slots, status);
    else
        rope_cache_vec_kernel<float><<<tokens, 128, 0, stream>>>((float*)qkv, ld, (const float2*)table, slot_map, (float*)k_cache,
                                                                 (float*)v_cache, num_heads, num_kv_heads, head_dim, page_size,
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
