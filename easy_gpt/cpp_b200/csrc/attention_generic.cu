// Attention over the paged cache, for any mix of prompt portions and decoded
// tokens: one warp per (token, query head).
//
// The token at absolute position p of its request sees the keys at positions
// first..p of that request, first = 0 or p - window + 1 with a sliding window.
// Keys are found through the request's row of the block table:
//   page = table[seq, pos / page_size], offset = pos % page_size.
// Query head h reads KV head h / (num_heads / num_kv_heads)
// (src/cuda/ops/self_attn_detail.cuh:667-669).
//
// score = (q . k) * scale (scaled after the dot product like the reference,
// src/models/self_attn.cpp:251-253), then a running softmax in float32 over
// chunks of 32 keys (one key per lane): m, l, acc as in
// src/cuda/ops/self_attn_detail.cuh:325-382, with expf, not the fast
// approximation.  The chunks start at `first`, so the order of the sums depends
// only on the token's own position and window — not on how the request was cut
// into steps, on the batch, or on the page ids.
//
// This is the kernel of the 32-bit path and the fallback of the bfloat16 path
// for sizes the tensor-core kernels refuse.
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_DIMS_PER_LANE = 8;      // head_dim <= 256
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                         const int* __restrict__ block_table, int table_stride, const int* __restrict__ token_seq,
                         const int* __restrict__ positions, T* __restrict__ out, int ldo, int num_heads, int num_kv_heads,
                         int head_dim, int page_size, long long page_stride, long long head_stride, int num_pages,
                         int window, float scale, int* status) {
    extern __shared__ float q_shared[];              // WARPS * head_dim
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int h = blockIdx.y * WARPS + warp;
    if (h >= num_heads) return;                       // no block-wide barrier below
    const int kvh = h / (num_heads / num_kv_heads);
    const int pos = positions[t];
    const int* table = block_table + (size_t)token_seq[t] * table_stride;
    float* qs = q_shared + warp * head_dim;
    const T* qrow = q + (size_t)t * ldq + h * head_dim;
    for (int d = lane; d < head_dim; d += 32) qs[d] = to_f32<T>(qrow[d]);
    __syncwarp();

    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    float m = -INFINITY, l = 0.0f;
    float acc[MAX_DIMS_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) acc[i] = 0.0f;

    for (int base = first; base <= pos; base += 32) {
        const int kpos = base + lane;
        const bool valid = kpos <= pos;
        long long row_off = -1;
        if (valid) {
            const int page = table[kpos / page_size];
            if (page < 0 || page >= num_pages) {
                atomicOr(status, EG_STATUS_BAD_PAGE);
            } else {
                row_off = (long long)page * page_stride + kvh * head_stride + (long long)(kpos % page_size) * head_dim;
            }
        }
        float s = -INFINITY;
        if (row_off >= 0) {
            const T* krow = k_cache + row_off;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; ++d) dot = fmaf(qs[d], to_f32<T>(krow[d]), dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;              // nothing readable in this chunk (bad pages only)
        const float corr = expf(m - m_new);            // m = -inf -> 0
        const float p = (row_off >= 0) ? expf(s - m_new) : 0.0f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) acc[i] *= corr;
        const int nkeys = min(32, pos - base + 1);
        for (int j = 0; j < nkeys; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long long off_j = __shfl_sync(0xffffffffu, row_off, j);
            if (off_j < 0) continue;
            const T* vrow = v_cache + off_j;
#pragma unroll
            for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
                const int d = lane + 32 * i;
                if (d < head_dim) acc[i] = fmaf(pj, to_f32<T>(vrow[d]), acc[i]);
            }
        }
        m = m_new;
    }
    T* orow = out + (size_t)t * ldo + h * head_dim;
    const float inv_l = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) orow[d] = from_f32<T>(acc[i] * inv_l);
    }
}

// Returns cudaErrorInvalidValue for sizes this kernel does not take.
EG_API int eg_attention_generic(cudaStream_t stream, int dtype, const void* q, int ldq, const void* k_cache,
                                const void* v_cache, const int* block_table, int table_stride, const int* token_seq,
                                const int* positions, void* out, int ldo, int tokens, int num_heads, int num_kv_heads,
                                int head_dim, int page_size, long long page_stride, long long head_stride, int num_pages,
                                int window, float scale, int* status) {
    if (tokens <= 0) return 0;
    if (head_dim > 32 * MAX_DIMS_PER_LANE || head_dim <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads)
        return (int)cudaErrorInvalidValue;
    dim3 grid(tokens, (num_heads + WARPS - 1) / WARPS);
    const size_t smem = (size_t)WARPS * head_dim * sizeof(float);
    if (dtype == EG_BF16)
        attention_generic_kernel<bf16><<<grid, WARPS * 32, smem, stream>>>(
            (const bf16*)q, ldq, (const bf16*)k_cache, (const bf16*)v_cache, block_table, table_stride, token_seq, positions,
            (bf16*)out, ldo, num_heads, num_kv_heads, head_dim, page_size, page_stride, head_stride, num_pages, window, scale, status);
    else
        attention_generic_kernel<float><<<grid, WARPS * 32, smem, stream>>>(
            (const float*)q, ldq, (const float*)k_cache, (const float*)v_cache, block_table, table_stride, token_seq, positions,
            (float*)out, ldo, num_heads, num_kv_heads, head_dim, page_size, page_stride, head_stride, num_pages, window, scale, status);
    return eg_launch_status();
}
