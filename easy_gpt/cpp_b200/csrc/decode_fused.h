// The program of a fused decode step: what eg_decode_fused runs as ONE persistent kernel.
//
// A decode step of a few tokens is a chain of small dependent operations; as separate kernels every link costs a
// launch boundary and a cold start (profiles: 33 us a layer where the memory needs 7).  Here the step is a list of
// operations that all CTAs of one cooperative launch walk together, with a barrier across the grid between
// operations.  A warp of every CTA streams the weights that its CTA will need, operation after operation, into a
// ring in shared memory, and is never held up by the barriers: weights do not depend on the step's data.
//
// An operation is described by a template (sizes, epilogue, the step's buffers) and a short record (the weights and
// caches of one layer).  The parts of a model emit them; a model whose parts cannot say what they do as such
// operations runs the kernels one by one instead.
#pragma once
#include <stdint.h>

enum { EGF_LINEAR = 1, EGF_ATTENTION = 2 };
// what a linear operation multiplies: rows of bfloat16; gain * (residual), scaled by the rows' 1/rms afterwards;
// the same with the residual taken from the embedding table (and written back by one CTA)
enum { EGF_IN_ROWS = 0, EGF_IN_NORM = 1, EGF_IN_EMBED_NORM = 2 };
// what happens to its result: rounded to bfloat16 and added to the float32 residual; stored as float32; rows interleaved
// (gate, up): up * silu(gate) to bfloat16; one head's rows (+ bias), q and k rotated, q stored, k and v into the cache
enum { EGF_OUT_RESIDUAL = 0, EGF_OUT_F32 = 1, EGF_OUT_SWIGLU = 2, EGF_OUT_QKV_ROPE = 3 };

typedef struct {
    int32_t type, input, output;
    int32_t N, K;
    // A unit of work is one or two tiles of 8 weight rows: unit u starts at row (u / units_per_group) * group_rows +
    // (u % units_per_group) * 8, its second tile pair_offset rows further (the partner rows of a rotation, or the next 8).
    int32_t tiles_per_unit, group_rows, units_per_group, pair_offset, num_units;
    int32_t warp_units;         // 1: every warp takes whole units of its own (one tile, K within a stage; outputs F32, SWIGLU)
    float eps;
    const void* x;              // EGF_IN_ROWS: bfloat16 [M, K]
    int64_t ldx;
    float* residual;            // float32 [M, K] (input) or [M, N] (EGF_OUT_RESIDUAL)
    const void* embed_table;    // EGF_IN_EMBED_NORM: bfloat16 [vocab, K]
    const int32_t* token_ids;
    int32_t vocab;
    void* out;                  // float32 [M, N] / bfloat16 [M, N/2] / bfloat16 q [M, num_heads * head_dim]
    int64_t ldo;
    // rotation, cache and attention
    int32_t num_heads, num_kv_heads, head_dim, page_size, num_pages, window;
    const int32_t* positions;
    const int32_t* slot_map;
    const float* inv_freq;      // null: no rotation
    int64_t page_stride, head_stride, pool_slots;
    const void* q;
    int32_t ldq;
    const int32_t* block_table;
    int32_t table_stride;
    const int32_t* seq_context; // keys cached before this step, per token of the step
    float scale;
    int32_t splits;             // CTAs that share the keys of one (token, KV head)
    float* partial_acc;         // [M, num_heads, splits, head_dim]
    float* partial_ml;          // [M, num_heads, splits, 2]
    int32_t* tickets;           // [M * num_kv_heads], zero before and after
    void* attn_out;             // bfloat16 [M, num_heads * head_dim]
    int32_t ld_attn;
} EgFusedTemplate;

typedef struct {
    int32_t tmpl;
    int32_t unit_offset;        // the CTA that takes the operation's first unit (small operations go to different SMs)
    const void* W;              // bfloat16 [N, K]
    int64_t ldw;
    const float* bias;          // float32 [N] or null
    const float* gain;          // float32 [K], EGF_IN_NORM / EGF_IN_EMBED_NORM
    void* k_cache;
    void* v_cache;
} EgFusedOp;

enum { EGF_MAX_TOKENS = 8, EGF_STAGE_BYTES = 16384, EGF_STAGE_COLS = 896, EGF_KV_BYTES = 65536 };
