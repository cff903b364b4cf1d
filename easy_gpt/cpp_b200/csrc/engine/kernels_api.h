// The C interface of the kernel library (libeasygpt_kernels: the hand-written sm_100a kernels of this folder), as the
// native engine calls it.  Every launcher takes raw device pointers and a stream, returns the launch's cudaError_t
// as an int (cudaErrorInvalidValue also when it refuses a size it does not take) and allocates nothing.
// (tests/test_native_build.py compares this file with the launchers' definitions.)
#pragma once
#include <cuda_runtime.h>

extern "C" {
// activation.cu
int eg_swiglu(cudaStream_t stream, int dtype, const void* gate_up, int ld, void* out, int ldo, int tokens, int inter);
// attention_generic.cu
int eg_attention_generic(cudaStream_t stream, int dtype, const void* q, int ldq, const void* k_cache,
    const void* v_cache, const int* block_table, int table_stride, const int* token_seq, const int* positions,
    void* out, int ldo, int tokens, int num_heads, int num_kv_heads, int head_dim, int page_size,
    long long page_stride, long long head_stride, int num_pages, int window, float scale, int* status);
// attention_paged.cu
int eg_attention_paged(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache,
    const int* block_table, int table_stride, const int* token_seq, const int* positions, const int* seq_context,
    void* out, int ldo, float* partial_acc, float* partial_ml, int tokens, int num_heads, int num_kv_heads,
    int head_dim, int page_size, long long page_stride, long long head_stride, int num_pages, int window, float scale,
    int splits, int* status, const void* prefetch, long long prefetch_bytes, int* counters, int use_pdl,
    unsigned long long* trace, const int* token_list);
// attention_paged.cu
int eg_attention_prefill(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache,
    const int* block_table, int table_stride, const int* positions, const int* tiles, int num_tiles, void* out,
    int ldo, int num_heads, int num_kv_heads, int head_dim, int page_size, long long page_stride,
    long long head_stride, int num_pages, int window, float scale, int* status);
// attention_tcgen05.cu
int eg_attention_prefill_tcgen05(cudaStream_t stream, const void* q, long long ldq, int total_tokens,
    const void* k_cache, const void* v_cache, const int* block_table, int table_stride, const int* positions,
    const int* tiles, int num_tiles, void* out, long long ldo, int num_heads, int num_kv_heads, int head_dim,
    int page_size, long long page_stride, long long head_stride, int num_pages, int window, float scale, int* status,
    long long* trace, int max_parts, int part_tiles, float* partial_o, float* partial_ml, int* queue);
int eg_attention_prefill_groups(int head_dim);
// embedding.cu
int eg_embedding_gather(cudaStream_t stream, int dtype, const int* ids, const void* table, float* residual, int tokens,
    int hidden, int vocab, int* status);
// engine_ops.cu
int eg_add_into_f32(cudaStream_t stream, float* residual, const void* delta, int delta_dtype, long long n);
// engine_ops.cu
int eg_convert_rows(cudaStream_t stream, const void* src, int src_dtype, void* dst, int dst_dtype, long long n);
// gemm_f32.cu
int eg_gemm_f32_nt(cudaStream_t stream, const float* A, int lda, const float* W, int ldw, const float* bias, float* C,
    int ldc, int M, int N, int K);
// gemm_skinny.cu
int eg_gemm_skinny(cudaStream_t stream, int epilogue, int norm, int use_pdl, const void* W, long long ldw,
    const float* bias, int M, int N, int K, const void* x, long long ldx, const float* resid_in, float* resid_out,
    const void* delta, const float* gain, float eps, void* out, long long ldo, int row_blocks, int k_slices,
    int k_split, float* scratch, int* counters, int num_heads, int num_kv_heads, int head_dim, const int* positions,
    const int* slot_map, void* k_cache, void* v_cache, const float* inv_freq, int page_size, long long page_stride,
    long long head_stride, long long pool_slots, int* status, const void* prefetch, long long prefetch_bytes,
    unsigned long long* trace, const float* ss_in, int ss_parts, float* resid_inout, const float* gain_out,
    void* xn_out, float* ss_out);
// gemm_tcgen05.cu
int eg_gemm_tcgen05(cudaStream_t stream, int epilogue, const void* A, long long lda, const void* W, long long ldw,
    const float* bias, void* out, long long ldo, int M, int N, int K, int* status);
// gemm_tcgen05.cu
int eg_gemm_tcgen05_pair(cudaStream_t stream, int epilogue, const void* A, long long lda, const void* W, long long ldw,
    const float* bias, void* out, long long ldo, int M, int N, int K, int tile_n, int* status, long long* trace);
// norm.cu
int eg_add_rmsnorm(cudaStream_t stream, int delta_dtype, int out_dtype, float* residual, const void* delta,
    const int* rows, const float* gain, void* out, int num_rows, int hidden, float eps);
// rope_cache.cu
int eg_rope_table(cudaStream_t stream, const int* positions, const float* inv_freq, float* table, int tokens,
    int half);
// rope_cache.cu
int eg_rope_cache_vec(cudaStream_t stream, int dtype, void* qkv, int ld, const float* table, const int* slot_map,
    void* k_cache, void* v_cache, int tokens, int num_heads, int num_kv_heads, int head_dim, int page_size,
    long long page_stride, long long head_stride, long long pool_slots, int* status);
// rope_cache.cu
int eg_rope_cache(cudaStream_t stream, int dtype, void* qkv, int ld, const float* bias, const int* positions,
    const int* slot_map, void* k_cache, void* v_cache, const float* inv_freq, int tokens, int num_heads,
    int num_kv_heads, int head_dim, int rotary_dim, int page_size, long long page_stride, long long head_stride,
    long long pool_slots, int* status);
// sampling.cu
int eg_argmax(cudaStream_t stream, const float* logits, long long ld, int rows, int vocab, int* out,
    int blocks_per_row, float* part_val, int* part_idx, int* counters);
// sampling.cu
int eg_sample(cudaStream_t stream, const float* logits, long long ld, int rows, int vocab, const float* temperature,
    const int* top_k, const float* top_p, const float* uniform, int* out);
// decode_fused.cu
int eg_decode_fused_smem(int stages, int xs_bytes, int num_ops, int num_tmpls);
// decode_fused.cu
int eg_decode_fused(cudaStream_t stream, const void* tmpls, int num_tmpls, const void* ops, int num_ops, int tokens, int stages, int xs_bytes, int ctas,
    unsigned* sync, int* status, unsigned long long* trace);
}  // extern "C"
