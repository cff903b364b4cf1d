// Launch plans and size rules of the kernel library, as the native engine uses them: which kernel takes
// which sizes, how the CTAs of a launch share the work.  The numbers were measured on B200; they hang off
// the device's SM count, never off a model's sizes.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdlib>

#include "device.hpp"
#include "kernels_api.h"

namespace easygpt::engine::plans {

constexpr int QUERY_TILE = 128;            // tokens per listed tile of a prompt portion
constexpr int SMALL_ENTRY_TOKENS = 4;      // entries of up to this many tokens go through the decode attention kernel
// Up to where the decode product beats the library product.  (Measured again, ms a decode step with the limit at 16 / 32 /
// 64 tokens: batch 24 1.29 / 1.38 / 1.40, batch 32 1.35 / 1.51 / 1.47, batch 64 1.60 / 1.61 / 2.87.)
constexpr int SKINNY_MAX_TOKENS = 16;
constexpr int FUSED_NORM_MAX_TOKENS = 16;  // every CTA repeats the norm prologue: worth it only for a few tokens
constexpr int MAX_HEAD_DIM = 256;          // the generic attention kernel keeps up to eight dimensions of a head per lane
constexpr int TCGEN05_ATTENTION_MIN_QUERY = 33;
constexpr size_t PREFILL_PARTS_SCRATCH_BYTES = 64u << 20;   // most memory for the partial results of a prompt attention whose key ranges are cut
// When a decode kernel lets the next one start: 2 once it has passed its own wait (the fastest measured), 1 at once,
// 0 never, i.e. no programmatic dependent launch (EASY_GPT_PDL, for measurements)
inline int use_pdl() {
    static int mode = -1;
    if (mode < 0) {
        const char* forced = std::getenv("EASY_GPT_PDL");
        mode = forced ? std::atoi(forced) : 2;
    }
    return mode;
}
enum Epilogue { EPI_STORE = 0, EPI_F32 = 1, EPI_SWIGLU = 2, EPI_QKV_ROPE = 3, EPI_RESID_NORM = 4 };

inline int sm_count() {
    static int count = 0;
    if (!count) {
        if (const char* forced = std::getenv("EASY_GPT_SM_COUNT")) count = std::atoi(forced);
        if (count <= 0) {
            int device = 0;
            cudaDeviceProp prop;
            if (cudaGetDevice(&device) == cudaSuccess && cudaGetDeviceProperties(&prop, device) == cudaSuccess) count = prop.multiProcessorCount;
        }
        if (count <= 0) count = 148;
    }
    return count;
}

inline bool attention_paged_takes(DType dtype, int head_dim, int page_size) {
    return dtype == DType::BF16 && (head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256) && page_size % 16 == 0;
}
inline bool attention_prefill_takes(DType dtype, int head_dim, int page_size) {
    return dtype == DType::BF16 && (head_dim == 32 || head_dim == 64 || head_dim == 128) && page_size % 16 == 0;
}
inline bool attention_prefill_tcgen05_takes(DType dtype, int head_dim, int page_size) {
    return dtype == DType::BF16 && (head_dim == 64 || head_dim == 128) && page_size % 16 == 0;
}

// How many CTAs share one (token, KV head).  Up to 16 tokens the kernel is fastest with one wave of 128 to 256
// CTAs that walk about eight key tiles of 64 each; with more tokens with about four CTAs per SM.  A power of two,
// at least four tiles per CTA.
inline int attention_paged_splits(int tokens, int num_heads, int num_kv_heads, long long max_context, int head_dim = 64) {
    const long long base = (long long)tokens * num_kv_heads * ((num_heads / num_kv_heads + 15) / 16);
    const long long tiles = std::max<long long>(1, (max_context + 63) / 64);
    // (measured with 2 / 4 / 8 CTAs per SM as the most, ms a step at context 4096: batch 24 1.43 / 1.31 / -, batch 32
    // 1.35 / 1.40 / 1.54, batch 48 1.78 / 1.54 / -, batch 64 1.81 / 1.65 / 1.75)
    // heads of more than 64: the kernel's three stages are 96 KB, two CTAs an SM (1.5B sizes, ms a step with 2 / 4 CTAs an
    // SM as the most: batch 32 2.27 / 2.62, batch 64 3.20 / 3.35; 7B sizes, batch 64: 9.18 / 9.47)
    const long long most = tokens <= SKINNY_MAX_TOKENS ? 256 : (head_dim > 64 ? 2LL : 4LL) * sm_count();
    int splits = 1;
    while ((long long)splits * 2 * base <= most && tiles / (splits * 2) >= 4 && splits < 128) splits *= 2;
    return splits;
}

// (parts, part_tiles): the most parts a query tile's keys are cut into and the fewest key tiles (of 64) of a part; the
// kernel cuts a tile's keys into min(parts, key tiles / part_tiles) parts.  A part costs its CTA a start-up of some
// microseconds and a pass of the merge kernel, which pays only while there are fewer (tile, head) pairs than CTAs (one
// per SM for heads of 64, whose CTAs share a unit's keys between two softmax groups already; two per SM else): the
// kernel is bound by what an SM gets through, not by its longest unit.  (Measured on B200, 14 heads of 64: a portion of
// 512 tokens on a context of 3,584, 56 pairs, takes 68 us uncut with one softmax group a CTA and 34 us in 4 parts; a
// prompt of 2,048 tokens, 224 pairs, 41 us uncut and 40 to 62 us however it is cut, with two groups a CTA 30 us.)
inline void attention_prefill_parts(int num_tiles, int num_heads, int head_dim, long long longest_context, int* parts, int* part_tiles) {
    const int ctas = sm_count() * (eg_attention_prefill_groups(head_dim) == 2 ? 1 : 2);
    const int wanted = std::min(ctas / std::max(1, num_tiles * num_heads), 8);
    if (wanted >= 2) { *parts = wanted; *part_tiles = 4; return; }
    *parts = 1;
    *part_tiles = 1 << 20;
    // Many units, but some with long key ranges (portions of prompts deep in their contexts, beside each other in a step
    // of a serving run): ranges of 48 key tiles and more are cut into parts of 24 at least (64 requests with prompts of
    // up to 4,096 tokens in portions of 512: 1.078 s with that, 1.093 without; parts of 12: 1.125).
    constexpr int long_from = 48, long_part = 24, long_most = 4;
    const long long key_tiles = (longest_context + 63) / 64;
    if (long_most > 1 && key_tiles >= long_from) { *parts = (int)std::min<long long>(long_most, key_tiles / long_part); *part_tiles = long_part; }
}

// Up to how many tokens a step's add + RMSNorm over rows of `width` can ride in the decode product's prologue
// (the rows of a token tile must fit the kernel's 200 KB of shared memory); 0: the norm runs on its own.
inline int fused_norm_max_tokens(int width) {
    if (width % 16) return 0;
    for (int tile : {16, 8}) {
        const long long row = (2LL * width + 127) / 128 * 128 + 64;
        const long long need = tile * row + tile * 4 + width * 4LL + tile * 32 + (width + 15) / 16 * tile * 4LL;
        if (need <= 200 * 1024) return std::min(tile, FUSED_NORM_MAX_TOKENS);
    }
    return 0;
}

struct SkinnyPlan {
    int row_blocks, k_slices, k_split;
};
// How the warps of a CTA and the CTAs of the grid share a [n_rows, in_features] weight matrix.
inline SkinnyPlan skinny_plan(int n_rows, int in_features, int head_dim = 0) {
    const int chunks = (in_features + 63) / 64;
    if (head_dim) {                                    // fused QKV: one CTA per head
        const int rb = head_dim / 16;
        int ks = 1;
        while (ks * 2 * rb <= 16 && chunks > 4 * ks) ks *= 2;
        // A head of a larger model is more than one SM should stream alone (7B sizes: 917 KB): its K range is cut across
        // up to 8 CTAs (a cluster) of about 128 KB each, at least four chunks a warp.  (1.5B sizes, three parts: 1.28 ms a
        // decode step at batch 1 against 1.36; 7B sizes, seven parts, 252 CTAs: 3.80 against 3.58.)
        const long long bytes = (long long)head_dim * in_features * 2;
        const int heads = std::max(1, n_rows / head_dim);
        int split = (int)std::max<long long>(1, std::min<long long>(8, (bytes + (64 << 10)) / (128 << 10)));
        split = std::max(1, std::min(split, sm_count() / heads));      // no more CTAs than SMs: every CTA stages the input rows
        if (heads * 8 > sm_count()) split = 1;                         // only where the heads leave most SMs idle (7B sizes, 36 heads in 4 parts: 4.11 ms against 4.04)
        while (split > 1 && chunks < 4 * ks * split) --split;
        return {rb, ks, split};
    }
    // wide matrices (gate/up, the head): 64 rows per CTA.  (Measured, ms a decode step at batch 8: 4 x 2 warps 0.737;
    // for the head alone 2 x 4 0.744, 4 x 1 0.733, 8 x 1 0.740, 2 x 2 0.735, 8 x 2 0.747; for both 2 x 4 0.803, 8 x 1 0.819.)
    if (n_rows >= 64 * sm_count()) return {4, 2, 1};
    const int rb = 1, ks = 8;
    // (Python's round() sends halves to the even neighbour; so does nearbyint in the default rounding mode)
    int split = (int)std::max(1.0, std::min(8.0, std::nearbyint(chunks / (ks * 2.5))));
    // No more CTAs than are on the GPU at once, two an SM (their registers): a second wave starts when the first is done
    // (1.5B sizes, down product, 96 row groups in 6 parts: the last CTAs started 15 us after the kernel in front had
    // ended).  No split where the row groups alone fill the SMs (7B sizes, down product, 224 row groups: 4.04 ms a step
    // at batch 8 unsplit, 4.24 in two parts).
    const long long groups = (n_rows + 15) / 16;
    if (groups >= sm_count()) split = 1;
    while (split > 1 && groups * split > 2LL * sm_count()) --split;
    return {rb, ks, split};
}
inline bool gemm_skinny_takes(DType dtype, int tokens, int in_features) {
    return dtype == DType::BF16 && tokens > 0 && tokens <= SKINNY_MAX_TOKENS && in_features % 16 == 0;
}
inline int skinny_padded_tokens(int tokens) { return tokens <= 8 ? 8 : tokens <= 16 ? 16 : tokens <= 32 ? 32 : 64; }

// Products wide and tall enough for the persistent tcgen05 kernel on CTA pairs (one tile per SM at least).
inline bool gemm_tcgen05_wide_takes(DType dtype, int tokens, int out_features, int in_features) {
    // (with fewer tiles the library product and a SwiGLU kernel are faster: a decode step at batch 64 takes 1.74 ms with
    // the pair kernel for gate/up, 38 tiles, against 1.67)
    return dtype == DType::BF16 && tokens > SKINNY_MAX_TOKENS && out_features % 256 == 0 && in_features % 64 == 0 &&
           (long long)((tokens + 127) / 128) * (out_features / 256) >= sm_count();
}

}  // namespace easygpt::engine::plans
