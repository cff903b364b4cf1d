// A whole decode step of up to 8 tokens as ONE persistent kernel (see decode_fused.h for the program it runs).
//
// One CTA per SM, launched cooperatively, so that all of them are on the GPU together and may meet at barriers.
// Each CTA has eight warps that compute and one that loads:
//
//   the loader   walks the program ahead of everybody else and brings the weight tiles of this CTA's units into a
//                ring of stages in shared memory with bulk copies (cp.async.bulk, completion counted on an mbarrier).
//                Weights never depend on the step's data, so the loader is not held up by the barriers between
//                operations: while the compute warps wait for each other across the grid, HBM keeps streaming.
//   the compute  warps take the operations in order.  A linear operation's unit is one or two tiles of 8 weight rows
//   warps        over the whole K: the eight warps share the K range of every stage (mma.m16n8k16, the tokens are the
//                M side, the weight rows the N side, both operands read with 16-byte shared-memory loads under the
//                same permutation of k), sum their parts through shared memory in a fixed order and run the
//                epilogue.  No unit is shared between CTAs, so nothing is summed across CTAs and every result has one
//                order of summation.  The attention operation is the split-KV kernel's body (attention_paged.cu) on
//                eight warps: two key tiles of 64 at a time, partial results to scratch memory, the CTA that
//                finishes a (token, KV head) last merges its splits; cached keys that were there before the step are
//                fetched before the barrier that the fresh ones wait for.
//   barriers     between operations: a counter in global memory, release-add on arrival, acquire loads while waiting,
//                bounded (after the limit the CTA raises an abort flag and a status bit; from then on every wait
//                returns at once, every CTA runs through the rest of the program without touching data, and the
//                kernel ends).
//
// Softmax, norms, rotation angles and the residual sum are float32 (src/models/norm.cpp:46-60,
// src/ops.cpp:404-421, src/cuda/ops/self_attn_detail.cuh:325-382).
#include "decode_fused.h"
#include "mbarrier.cuh"
#include "mma_utils.cuh"

namespace {

constexpr int COMPUTE_WARPS = 8;
constexpr int COMPUTE_THREADS = COMPUTE_WARPS * 32;
constexpr int THREADS = COMPUTE_THREADS + 128;              // the loader's warp group: one warp loads, three only give their registers away
constexpr int COMPUTE_REGS = 232, LOADER_REGS = 40;          // per thread, after the groups have re-balanced the register file
constexpr int MT = EGF_MAX_TOKENS;
constexpr int KC = EGF_STAGE_COLS;                     // weight columns of a stage
constexpr int W_STRIDE = KC * 2 + 64;                  // bytes between the 8 rows of a stage: rows alternate between the halves of a 128-byte line
constexpr int TILE_KEYS = 64;
constexpr int QUARTER_TILES = 64;
constexpr unsigned WAIT_LIMIT = 1u << 22;
constexpr unsigned GRID_WAIT_LIMIT = 1u << 22;
static_assert(8 * W_STRIDE <= EGF_STAGE_BYTES, "a stage holds 8 rows");
static_assert(COMPUTE_THREADS == 256, "the barrier of the compute warps is written for 256 threads");

__host__ __device__ inline int xs_stride_bytes(int K) { return ((K * 2 + 127) / 128) * 128 + 64; }

struct Layout {                                        // offsets into dynamic shared memory
    int ring, xs, red, vals, factor, quarters, ops, tmpls, bars, flags, total;
};
__host__ __device__ inline Layout layout_for(int stages, int xs_bytes, int num_ops, int num_tmpls) {
    Layout l;
    int at = 0;
    auto take = [&](int bytes, int align) {
        at = (at + align - 1) / align * align;
        const int here = at;
        at += bytes;
        return here;
    };
    l.ring = take(stages * EGF_STAGE_BYTES, 1024);
    l.xs = take(xs_bytes, 1024);
    l.red = take(COMPUTE_WARPS * 2 * MT * 8 * 4, 16);
    l.vals = take(2 * MT * 8 * 4, 16);
    l.factor = take(MT * 4, 16);
    l.quarters = take(QUARTER_TILES * 4 * 8, 16);
    l.ops = take(num_ops * (int)sizeof(EgFusedOp), 16);
    l.tmpls = take(num_tmpls * (int)sizeof(EgFusedTemplate), 16);
    l.bars = take(2 * stages * 8, 8);
    l.flags = take(16, 16);
    l.total = at;
    return l;
}

struct Params {
    const EgFusedTemplate* tmpls;
    const EgFusedOp* ops;
    int num_tmpls, num_ops, M, stages, xs_bytes;
    unsigned* sync_counter;      // zero at launch
    int* abort_flag;             // zero at launch
    int* status;
    unsigned long long* trace;   // optional: [num_ops][4] latest stamps: operation entered, input staged, products done, left
};

__device__ __forceinline__ void compute_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(COMPUTE_THREADS) : "memory"); }
__device__ __forceinline__ uint4 lds128(const void* p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
    return v;
}
__device__ __forceinline__ void bulk_to_smem(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}


struct Shared {
    unsigned char* ring;
    unsigned char* xs;
    float* red;        // [warp][tile][m][n]
    float* vals;       // [tile][m][n]
    float* factor;     // [m]
    long long* quarters;
    const EgFusedOp* ops;
    const EgFusedTemplate* tmpls;
    uint64_t* full;
    uint64_t* empty;
    volatile int* abort;   // [0]: this CTA has given up
    int* is_last;
    int* decision;         // a flag that all compute threads read the same value of (written by one, between barriers)
};

// Whether this CTA has given up, as ONE answer for all its compute threads (the flag may be raised at any moment,
// and branches that hold barriers must not split the CTA).
__device__ __forceinline__ bool given_up(const Shared& s) {
    if (threadIdx.x == 0) *s.decision = *s.abort;
    asm volatile("bar.sync 1, 256;\n" ::: "memory");
    const bool yes = *s.decision != 0;
    asm volatile("bar.sync 1, 256;\n" ::: "memory");
    return yes;
}

// ---- the barrier across the grid (compute warps only) -------------------------------------------------------------
// Arrivals are counted on one word; the CTA that arrives last writes the barrier's number to another word (in a cache
// line of its own), which is what everybody else reads while waiting: the counter's line is not polled.
__device__ __forceinline__ void grid_barrier(const Params& p, const Shared& s, unsigned number) {
    compute_sync();
    if (threadIdx.x == 0) {
        unsigned* flag = p.sync_counter + 32;
        unsigned old;
        // release: everything this CTA wrote (ordered before by the barrier above) is visible to whoever acquires the count
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;\n" : "=r"(old) : "l"(p.sync_counter) : "memory");
        if (old + 1 == number * gridDim.x) {
            asm volatile("st.release.gpu.global.u32 [%0], %1;\n" ::"l"(flag), "r"(number) : "memory");
        } else if (!*s.abort) {
            unsigned polls = 0;
            unsigned seen;
            for (;;) {
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(flag) : "memory");
                if (seen >= number) break;
                ++polls;
                if ((polls & 63u) == 0 && *(volatile int*)p.abort_flag) {
                    *s.abort = 1;
                    break;
                }
                if (polls > GRID_WAIT_LIMIT) {
                    atomicOr(p.status, EG_STATUS_WAIT_TIMEOUT);
                    atomicExch(p.abort_flag, 1);
                    *s.abort = 1;
                    break;
                }
            }
            asm volatile("fence.acq_rel.gpu;\n" ::: "memory");
        }
    }
    compute_sync();
}

// A tile whose 8 rows are whole rows of W, one behind the other in memory, comes in one copy and keeps W's row pitch in
// shared memory (two rows then share the banks of a 16-byte read: a two-way conflict, paid for by seven copies fewer).
__device__ __forceinline__ bool dense_rows(const EgFusedTemplate& t, const EgFusedOp& op) { return t.K <= KC && op.ldw == t.K; }

// where a walker of the ring stands: the slot of its next stage and the parity of that slot's current use
struct RingPlace {
    unsigned slot = 0, parity = 0;
    __device__ __forceinline__ void advance(int stages) {
        if (++slot == (unsigned)stages) {
            slot = 0;
            parity ^= 1u;
        }
    }
};

__device__ __forceinline__ int first_unit_of(const EgFusedOp& op) {
    const int G = (int)gridDim.x;
    return ((int)blockIdx.x + G - op.unit_offset % G) % G;
}

// ---- the loader warp ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void loader(const Params& p, const Shared& s) {
    const int lane = threadIdx.x & 31;
    const int G = (int)gridDim.x;
    unsigned fill = 0;
    RingPlace place;
    bool ok = true;
    for (int i = 0; i < p.num_ops && ok; ++i) {
        const EgFusedOp& op = s.ops[i];
        const EgFusedTemplate& t = s.tmpls[op.tmpl];
        if (t.type != EGF_LINEAR) continue;
        const bf16* W = static_cast<const bf16*>(op.W);
        const bool dense = dense_rows(t, op);
        for (int u = first_unit_of(op); u < t.num_units && ok; u += G) {
            const int row0 = (u / t.units_per_group) * t.group_rows + (u % t.units_per_group) * 8;
            for (int tile = 0; tile < t.tiles_per_unit && ok; ++tile) {
                const int r0 = row0 + tile * t.pair_offset;
                for (int k0 = 0; k0 < t.K && ok; k0 += KC) {
                    const int cols = min(KC, t.K - k0);
                    const unsigned slot = place.slot;
                    int got = 1;
                    if (lane == 0) got = mbar_wait_bounded(&s.empty[slot], place.parity ^ 1u, s.abort, p.status, WAIT_LIMIT) ? 1 : 0;
                    got = __shfl_sync(0xffffffffu, got, 0);
                    if (!got) {
                        ok = false;
                        break;
                    }
                    unsigned char* stage = s.ring + (size_t)slot * EGF_STAGE_BYTES;
                    if (lane == 0) mbar_expect_tx(&s.full[slot], 8u * (unsigned)cols * 2u);
                    __syncwarp();
                    if (dense) {                                        // the tile's 8 rows lie one behind the other: one copy
                        if (lane == 0) bulk_to_smem(stage, W + (size_t)r0 * op.ldw, 8u * (unsigned)cols * 2u, &s.full[slot]);
                    } else if (lane < 8) {
                        bulk_to_smem(stage + lane * W_STRIDE, W + (size_t)(r0 + lane) * op.ldw + k0, (unsigned)cols * 2u, &s.full[slot]);
                    }
                    ++fill;
                    place.advance(p.stages);
                }
            }
        }
    }
    if (!ok && lane == 0) {
        // given up: the copies already issued must land before this CTA's shared memory goes away
        const unsigned from = fill > (unsigned)p.stages ? fill - (unsigned)p.stages : 0u;
        for (unsigned j = from; j < fill; ++j) {
            uint64_t* bar = &s.full[j % (unsigned)p.stages];
            const unsigned parity = (j / (unsigned)p.stages) & 1u;
            for (unsigned n = 0; n < WAIT_LIMIT && !mbar_try_wait(bar, parity); ++n) {}
        }
    }
}

// ---- linear operations ------------------------------------------------------------------------------------------------
// The input of an operation with a norm in front, into shared memory: bfloat16 [MT][K] of gain * v, rows past M zero, and
// the rows' 1/rms to s.factor.  (Plain bfloat16 rows are read from global memory by the warps that need them.)
__device__ __forceinline__ void stage_input(const Params& p, const Shared& s, const EgFusedTemplate& t, const EgFusedOp& op, bool writes_residual) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int K = t.K, stride = xs_stride_bytes(K);
    // a warp per token row: v = residual (or the token's embedding), sum of squares, bfloat16(gain * v)
    const int m = warp;                                             // COMPUTE_WARPS == MT
    const int quads = K / 4;
    uint2* dst = reinterpret_cast<uint2*>(s.xs + (size_t)m * stride);
    if (m >= p.M) {
        for (int i = lane; i < quads; i += 32) dst[i] = make_uint2(0u, 0u);
        if (lane == 0) s.factor[m] = 0.f;
        return;
    }
    const float4* g = reinterpret_cast<const float4*>(op.gain);
    float ss = 0.f;
    constexpr int BATCH = 8;
    if (t.input == EGF_IN_NORM) {
        const float4* r = reinterpret_cast<const float4*>(t.residual + (size_t)m * K);
        for (int i0 = lane; i0 < quads; i0 += 32 * BATCH) {
            float4 rv[BATCH], gv[BATCH];
#pragma unroll
            for (int b = 0; b < BATCH; ++b) {
                const int i = i0 + 32 * b;
                if (i < quads) {
                    rv[b] = __ldcg(r + i);
                    gv[b] = __ldg(g + i);
                }
            }
#pragma unroll
            for (int b = 0; b < BATCH; ++b) {
                const int i = i0 + 32 * b;
                if (i < quads) {
                    const float4 v = rv[b];
                    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                    dst[i] = make_uint2(pack_bf16(gv[b].x * v.x, gv[b].y * v.y), pack_bf16(gv[b].z * v.z, gv[b].w * v.w));
                }
            }
        }
    } else {
        int id = t.token_ids[m];
        if (id < 0 || id >= t.vocab) {
            if (lane == 0) atomicOr(p.status, EG_STATUS_BAD_TOKEN);
            id = 0;
        }
        const uint2* row = reinterpret_cast<const uint2*>(static_cast<const bf16*>(t.embed_table) + (size_t)id * K);
        float4* ro = writes_residual ? reinterpret_cast<float4*>(t.residual + (size_t)m * K) : nullptr;
        for (int i0 = lane; i0 < quads; i0 += 32 * BATCH) {
            uint2 ev[BATCH];
            float4 gv[BATCH];
#pragma unroll
            for (int b = 0; b < BATCH; ++b) {
                const int i = i0 + 32 * b;
                if (i < quads) {
                    ev[b] = __ldg(row + i);
                    gv[b] = __ldg(g + i);
                }
            }
#pragma unroll
            for (int b = 0; b < BATCH; ++b) {
                const int i = i0 + 32 * b;
                if (i < quads) {
                    const __nv_bfloat162 e01 = *reinterpret_cast<const __nv_bfloat162*>(&ev[b].x);
                    const __nv_bfloat162 e23 = *reinterpret_cast<const __nv_bfloat162*>(&ev[b].y);
                    const float4 v = make_float4(__low2float(e01), __high2float(e01), __low2float(e23), __high2float(e23));
                    if (ro) ro[i] = v;
                    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                    dst[i] = make_uint2(pack_bf16(gv[b].x * v.x, gv[b].y * v.y), pack_bf16(gv[b].z * v.z, gv[b].w * v.w));
                }
            }
        }
    }
    ss = warp_sum(ss);
    if (lane == 0) s.factor[m] = 1.0f / sqrtf(ss / (float)K + t.eps);
}

__device__ __forceinline__ void linear_epilogue(const Params& p, const Shared& s, const EgFusedTemplate& t, const EgFusedOp& op, int row0) {
    const int tid = threadIdx.x;
    const bool normed = t.input != EGF_IN_ROWS;
    // vals[tile][m][n] holds the products; row n of tile k is weight row row0 + k * pair_offset + n
    auto value = [&](int tile, int m, int n) -> float {
        float v = s.vals[(tile * MT + m) * 8 + n];
        if (normed) v *= s.factor[m];
        if (op.bias) v += op.bias[row0 + tile * t.pair_offset + n];
        return v;
    };
    if (t.output == EGF_OUT_RESIDUAL || t.output == EGF_OUT_F32) {
        for (int e = tid; e < t.tiles_per_unit * 8 * p.M; e += COMPUTE_THREADS) {
            const int n = e % 8, tile = (e / 8) % t.tiles_per_unit, m = e / (8 * t.tiles_per_unit);
            const int row = row0 + tile * t.pair_offset + n;
            const float v = value(tile, m, n);
            if (t.output == EGF_OUT_F32) {
                static_cast<float*>(t.out)[(size_t)m * t.ldo + row] = v;
            } else {
                // (another CTA wrote this element in the operation before: read it past the L1)
                float* r = t.residual + (size_t)m * t.N + row;
                *r = __ldcg(r) + __bfloat162float(__float2bfloat16_rn(v));      // what a stored bfloat16 delta would add
            }
        }
    } else if (t.output == EGF_OUT_SWIGLU) {
        const int pairs = t.tiles_per_unit * 4;                       // (gate, up) pairs of this unit: rows 2i, 2i + 1
        for (int e = tid; e < pairs * p.M; e += COMPUTE_THREADS) {
            const int i = e % pairs, m = e / pairs;
            const int tile = i / 4, n = (i % 4) * 2;
            const float g = value(tile, m, n), u = value(tile, m, n + 1);
            const float sig = 1.0f / (1.0f + expf(-g));
            const int col = (row0 + tile * t.pair_offset + n) >> 1;
            static_cast<bf16*>(t.out)[(size_t)m * t.ldo + col] = __float2bfloat16_rn(u * (g * sig));
        }
    } else {   // EGF_OUT_QKV_ROPE: tile 0 holds rows j .. j+7 of a head, tile 1 their partners j + head_dim/2 ..
        const int HD = t.head_dim, half = HD / 2;
        const int head = row0 / HD, j0 = row0 % HD;
        const bool is_q = head < t.num_heads, is_k = !is_q && head < t.num_heads + t.num_kv_heads;
        for (int e = tid; e < 8 * p.M; e += COMPUTE_THREADS) {
            const int n = e % 8, m = e / 8, j = j0 + n;
            const float x0 = value(0, m, n), x1 = value(1, m, n);
            float y0 = x0, y1 = x1;
            if ((is_q || is_k) && t.inv_freq) {
                const float a = (float)t.positions[m] * t.inv_freq[j];
                const float cs = cosf(a), sn = sinf(a);
                y0 = x0 * cs - x1 * sn;
                y1 = x0 * sn + x1 * cs;
            }
            if (is_q) {
                bf16* o = static_cast<bf16*>(t.out) + (size_t)m * t.ldo + (size_t)head * HD;
                o[j] = __float2bfloat16_rn(y0);
                o[j + half] = __float2bfloat16_rn(y1);
            } else {
                const long long slot = t.slot_map[m];
                if (slot < 0 || slot >= t.pool_slots) {
                    if (slot >= t.pool_slots) atomicOr(p.status, EG_STATUS_BAD_SLOT);
                    continue;
                }
                const int kvh = is_k ? head - t.num_heads : head - t.num_heads - t.num_kv_heads;
                bf16* o = static_cast<bf16*>(is_k ? op.k_cache : op.v_cache) + (slot / t.page_size) * t.page_stride + (long long)kvh * t.head_stride +
                          (slot % t.page_size) * HD;
                o[j] = __float2bfloat16_rn(y0);
                o[j + half] = __float2bfloat16_rn(y1);
            }
        }
    }
}

// Many small units (gate/up, the head): every warp takes whole units of its own, one tile of 8 rows over all of K in one
// stage, and finishes them from its registers; the warps meet only once, when the input rows are staged.
__device__ __forceinline__ void linear_warp_units(const Params& p, const Shared& s, const EgFusedTemplate& t, const EgFusedOp& op, RingPlace& ring, int first) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    const int G = (int)gridDim.x;
    const int stride = xs_stride_bytes(t.K);
    const int wstride = dense_rows(t, op) ? t.K * 2 : W_STRIDE;
    const int chunks = (t.K + 31) / 32;
    const unsigned char* xrow = s.xs + (size_t)gid * stride + tig * 16;
    const float factor = gid < p.M ? s.factor[gid] : 0.f;
    int j = 0;
    for (int u = first; u < t.num_units; u += G, ++j) {
        const unsigned slot = ring.slot, parity = ring.parity;
        ring.advance(p.stages);
        // Every warp sees every stage arrive, in order, also those of the other warps' units: a wait by parity is only
        // right for the barrier's next phase, never for one further ahead.
        int got = 1;
        if (lane == 0) got = mbar_wait_bounded(&s.full[slot], parity, s.abort, p.status, WAIT_LIMIT) ? 1 : 0;
        got = __shfl_sync(0xffffffffu, got, 0);
        if ((j & (COMPUTE_WARPS - 1)) != warp) {
            if (lane == 0) mbar_arrive(&s.empty[slot]);
            continue;
        }
        float acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        if (got) {
            const unsigned char* wrow = s.ring + (size_t)slot * EGF_STAGE_BYTES + gid * wstride + tig * 16;
#pragma unroll 4
            for (int c = 0; c < chunks; ++c) {
                uint4 w = make_uint4(0u, 0u, 0u, 0u), x = make_uint4(0u, 0u, 0u, 0u);
                if (c * 32 + tig * 8 < t.K) {
                    w = lds128(wrow + c * 64);
                    x = lds128(xrow + c * 64);
                }
                const uint32_t a0[4] = {x.x, 0u, x.y, 0u}, a1[4] = {x.z, 0u, x.w, 0u};
                mma_bf16_16816(acc[(c & 1) * 2], a0, w.x, w.y);          // four accumulators: no product waits for the one before it
                mma_bf16_16816(acc[(c & 1) * 2 + 1], a1, w.z, w.w);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.empty[slot]);
        if (!got || gid >= p.M) continue;
        // this thread holds token gid, weight rows row0 + 2 tig and row0 + 2 tig + 1
        const int row = u * 8 + 2 * tig;                                 // one tile per unit, units in row order
        float v0 = ((acc[0][0] + acc[1][0]) + (acc[2][0] + acc[3][0])) * factor;
        float v1 = ((acc[0][1] + acc[1][1]) + (acc[2][1] + acc[3][1])) * factor;
        if (op.bias) {
            v0 += op.bias[row];
            v1 += op.bias[row + 1];
        }
        if (t.output == EGF_OUT_F32) {
            *reinterpret_cast<float2*>(static_cast<float*>(t.out) + (size_t)gid * t.ldo + row) = make_float2(v0, v1);
        } else {                                                          // rows (gate, up) of one pair
            const float sig = 1.0f / (1.0f + expf(-v0));
            static_cast<bf16*>(t.out)[(size_t)gid * t.ldo + (row >> 1)] = __float2bfloat16_rn(v1 * (v0 * sig));
        }
    }
}

__device__ __forceinline__ void linear_op(const Params& p, const Shared& s, const EgFusedTemplate& t, const EgFusedOp& op, RingPlace& ring, unsigned long long* stamps) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
    const int G = (int)gridDim.x;
    const int first = first_unit_of(op);
    if (first >= t.num_units) return;                                 // nothing for this CTA (and nothing in its ring)
    const bool staged = t.input != EGF_IN_ROWS;                       // rows of bfloat16 are read straight from global memory instead
    if (staged) {
        if (!*s.abort) stage_input(p, s, t, op, first == 0);
        compute_sync();
    }
    if (stamps && tid == 0) atomicMax(stamps + 1, now_ns());
    if (t.warp_units) {
        linear_warp_units(p, s, t, op, ring, first);
        if (stamps && tid == 0) atomicMax(stamps + 2, now_ns());
        compute_sync();                                               // the input rows are free for the next operation
        return;
    }
    const int stride = xs_stride_bytes(t.K);
    const int wstride = dense_rows(t, op) ? t.K * 2 : W_STRIDE;
    const bf16* xg = static_cast<const bf16*>(t.x) + (size_t)gid * t.ldx + tig * 8;
    for (int u = first; u < t.num_units; u += G) {
        const int row0 = (u / t.units_per_group) * t.group_rows + (u % t.units_per_group) * 8;
        float acc[2][2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int k = 0; k < 2; ++k) acc[i][k][0] = acc[i][k][1] = acc[i][k][2] = acc[i][k][3] = 0.f;
#pragma unroll
        for (int tile = 0; tile < 2; ++tile) {
            if (tile >= t.tiles_per_unit) break;
            for (int k0 = 0; k0 < t.K; k0 += KC) {
                const int cols = min(KC, t.K - k0);
                const int chunks = (cols + 31) / 32;
                // this warp's chunks of the stage: warp, warp + 8, ...: at most four (KC / 32 / 8 rounded up)
                uint4 xr[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c = warp + COMPUTE_WARPS * i;
                    xr[i] = make_uint4(0u, 0u, 0u, 0u);
                    if (c < chunks && c * 32 + tig * 8 < cols) {
                        if (staged) xr[i] = lds128(s.xs + (size_t)gid * stride + (size_t)(k0 + c * 32 + tig * 8) * 2);
                        else if (gid < p.M) xr[i] = __ldcg(reinterpret_cast<const uint4*>(xg + k0 + c * 32));   // written by other CTAs: past the L1
                    }
                }
                const unsigned slot = ring.slot, parity = ring.parity;
                ring.advance(p.stages);
                int got = 1;
                if (lane == 0) got = mbar_wait_bounded(&s.full[slot], parity, s.abort, p.status, WAIT_LIMIT) ? 1 : 0;
                got = __shfl_sync(0xffffffffu, got, 0);
                if (got) {
                    const unsigned char* wrow = s.ring + (size_t)slot * EGF_STAGE_BYTES + gid * wstride + tig * 16;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int c = warp + COMPUTE_WARPS * i;
                        if (c < chunks) {                              // the same for the whole warp
                            uint4 w = make_uint4(0u, 0u, 0u, 0u);
                            if (c * 32 + tig * 8 < cols) w = lds128(wrow + c * 64);
                            // two k-steps of 16; both operands use elements 4s .. 4s+3 of the lane's 8 in step s
                            const uint32_t a0[4] = {xr[i].x, 0u, xr[i].y, 0u}, a1[4] = {xr[i].z, 0u, xr[i].w, 0u};
                            mma_bf16_16816(acc[tile][0], a0, w.x, w.y);
                            mma_bf16_16816(acc[tile][1], a1, w.z, w.w);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&s.empty[slot]);
            }
        }
        // sum the warps' parts: rows gid (tokens), columns 2 tig, 2 tig + 1 (weight rows of the tile)
#pragma unroll
        for (int tile = 0; tile < 2; ++tile) {
            float* mine = s.red + ((size_t)(warp * 2 + tile) * MT + gid) * 8 + 2 * tig;
            mine[0] = acc[tile][0][0] + acc[tile][1][0];
            mine[1] = acc[tile][0][1] + acc[tile][1][1];
        }
        compute_sync();
        for (int e = tid; e < t.tiles_per_unit * MT * 8; e += COMPUTE_THREADS) {
            const int tile = e / (MT * 8), rest = e % (MT * 8);
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < COMPUTE_WARPS; ++w) v += s.red[(size_t)(w * 2 + tile) * MT * 8 + rest];      // fixed order
            s.vals[e] = v;
        }
        compute_sync();
        if (!*s.abort) linear_epilogue(p, s, t, op, row0);
    }
    if (stamps && tid == 0) atomicMax(stamps + 2, now_ns());
}

// ---- attention ------------------------------------------------------------------------------------------------------
template <int HD>
struct KvLayout {
    static constexpr int CHUNKS = HD / 8;
    static constexpr int SWZ = CHUNKS >= 8 ? 7 : CHUNKS - 1;
    static constexpr int TILE_BYTES = TILE_KEYS * HD * 2;
    static constexpr int BUF_BYTES = 2 * TILE_BYTES;                 // keys, then values
    __device__ static __forceinline__ int offset(int row, int chunk) { return (row * CHUNKS + (chunk ^ (row & SWZ))) * 16; }
};

struct AttnUnit {
    int m, kvh, split, pos, fresh_from, first, my_lo, my_hi, ntiles;
    const int* table;
};
__device__ __forceinline__ AttnUnit attn_unit(const EgFusedTemplate& t, int u) {
    AttnUnit a;
    a.split = u % t.splits;
    a.kvh = (u / t.splits) % t.num_kv_heads;
    a.m = u / (t.splits * t.num_kv_heads);
    a.pos = t.positions[a.m];
    a.fresh_from = t.seq_context ? t.seq_context[a.m] : 0;
    a.first = (t.window > 0 && a.pos - t.window + 1 > 0) ? a.pos - t.window + 1 : 0;
    a.table = t.block_table + (size_t)a.m * t.table_stride;
    const int tile_lo = a.first / TILE_KEYS, tile_hi = a.pos / TILE_KEYS;
    const int per = (tile_hi - tile_lo + 1 + t.splits - 1) / t.splits;
    a.my_lo = tile_lo + a.split * per;
    a.my_hi = min(tile_hi, a.my_lo + per - 1);
    a.ntiles = a.my_hi - a.my_lo + 1;
    return a;
}

template <int HD>
struct Attention {
    using L = KvLayout<HD>;
    const Params& p;
    const Shared& s;
    const EgFusedTemplate& t;
    const EgFusedOp& op;
    int quarter_tile0 = 0;

    __device__ __forceinline__ Attention(const Params& p, const Shared& s, const EgFusedTemplate& t, const EgFusedOp& op) : p(p), s(s), t(t), op(op) {}

    __device__ __forceinline__ void fill_quarters(const AttnUnit& a, int tile0) {
        quarter_tile0 = tile0;
        const int count = min(QUARTER_TILES, a.my_hi - tile0 + 1);
        for (int e = threadIdx.x; e < count * 4; e += COMPUTE_THREADS) {
            const int kpos0 = (tile0 + e / 4) * TILE_KEYS + (e % 4) * 16;
            long long base = -1;
            if (kpos0 <= a.pos && kpos0 + 15 >= a.first) {
                const int page = a.table[kpos0 / t.page_size];
                if (page < 0 || page >= t.num_pages) atomicOr(p.status, EG_STATUS_BAD_PAGE);
                else base = (long long)page * t.page_stride + (long long)a.kvh * t.head_stride + (long long)(kpos0 % t.page_size) * HD;
            }
            s.quarters[e] = base;
        }
    }
    // mode 0: every row; 1 (before the barrier): all but the fresh keys; 2 (after it): the fresh keys only
    __device__ __forceinline__ void load_tile(const AttnUnit& a, int tile, int buf, int mode) {
        unsigned char* ks = s.xs + (size_t)buf * L::BUF_BYTES;
        unsigned char* vs = ks + L::TILE_BYTES;
        const long long* qb = s.quarters + (tile - quarter_tile0) * 4;
        const bf16* kc = static_cast<const bf16*>(op.k_cache);
        const bf16* vc = static_cast<const bf16*>(op.v_cache);
        for (int e = threadIdx.x; e < TILE_KEYS * L::CHUNKS; e += COMPUTE_THREADS) {
            const int row = e / L::CHUNKS, chunk = e % L::CHUNKS;
            const int kpos = tile * TILE_KEYS + row;
            const long long base = qb[row >> 4];
            const bool valid = kpos >= a.first && kpos <= a.pos && base >= 0;
            const bool fresh = kpos >= a.first && kpos <= a.pos && kpos >= a.fresh_from;
            if ((mode == 1 && fresh) || (mode == 2 && !fresh)) continue;
            const long long off = valid ? base + (long long)(row & 15) * HD + chunk * 8 : 0;
            cp_async_16(ks + L::offset(row, chunk), kc + off, valid);
            cp_async_16(vs + L::offset(row, chunk), vc + off, valid);
        }
    }
    // pairs 0 and 1 of the unit's tiles (buffers 0..3): what does not depend on this step; two commit groups
    __device__ __forceinline__ void prefetch(const AttnUnit& a) {
        if (a.ntiles > 0) fill_quarters(a, a.my_lo);
        compute_sync();
        for (int pr = 0; pr < 2; ++pr) {
            for (int h = 0; h < 2; ++h)
                if (2 * pr + h < a.ntiles) load_tile(a, a.my_lo + 2 * pr + h, 2 * pr + h, 1);
            cp_async_commit();
        }
    }

    __device__ __forceinline__ void run(const AttnUnit& a, bool prefetched) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
        const int G = t.num_heads / t.num_kv_heads;
        const float scale_log2 = t.scale * 1.4426950408889634f;
        if (!prefetched) prefetch(a);
        for (int pr = 0; pr < 2; ++pr)
            for (int h = 0; h < 2; ++h) {
                const int i = 2 * pr + h;
                if (i < a.ntiles && (a.my_lo + i + 1) * TILE_KEYS > a.fresh_from) load_tile(a, a.my_lo + i, i, 2);
            }
        cp_async_commit();

        // query rows as A fragments: row r <-> head kvh * G + r
        uint32_t qf[HD / 16][4];
        {
            const bf16* q = static_cast<const bf16*>(t.q);
            const bf16* q0 = q + (size_t)a.m * t.ldq + (size_t)(a.kvh * G + gid) * HD;
            const bf16* q1 = q + (size_t)a.m * t.ldq + (size_t)(a.kvh * G + gid + 8) * HD;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                const int d = ks * 16 + 2 * tig;
                qf[ks][0] = gid < G ? __ldcg(reinterpret_cast<const uint32_t*>(q0 + d)) : 0u;       // written by other CTAs: past the L1
                qf[ks][1] = gid + 8 < G ? __ldcg(reinterpret_cast<const uint32_t*>(q1 + d)) : 0u;
                qf[ks][2] = gid < G ? __ldcg(reinterpret_cast<const uint32_t*>(q0 + d + 8)) : 0u;
                qf[ks][3] = gid + 8 < G ? __ldcg(reinterpret_cast<const uint32_t*>(q1 + d + 8)) : 0u;
            }
        }
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
        float acc[HD / 8][4];
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;

        const int pairs = (a.ntiles + 1) / 2;
        const int half = warp >> 2, quarter = warp & 3;              // which tile of the pair, which 16 keys of it
        for (int pr = 0; pr < pairs; ++pr) {
            if (pr == 0) cp_async_wait<0>();                             // the first two pairs and their fresh rows
            else cp_async_wait<1>();                                      // all but the pair asked for last
            compute_sync();
            const int it = 2 * pr + half;
            if (it < a.ntiles) {
                const int buf = (2 * pr + half) & 3;
                const unsigned char* ks = s.xs + (size_t)buf * L::BUF_BYTES;
                const unsigned char* vs = ks + L::TILE_BYTES;
                const int key_base = (a.my_lo + it) * TILE_KEYS + quarter * 16;
                if (!(key_base > a.pos || key_base + 15 < a.first)) {
                    float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                    for (int kk = 0; kk < HD / 16; ++kk) {
                        uint32_t b[4];
                        const int mi = lane >> 3, r = lane & 7;
                        ldmatrix_x4(b, ks + L::offset(quarter * 16 + (mi >> 1) * 8 + r, kk * 2 + (mi & 1)));
                        mma_bf16_16816(sc[0], qf[kk], b[0], b[1]);
                        mma_bf16_16816(sc[1], qf[kk], b[2], b[3]);
                    }
                    float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
                    for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int kpos = key_base + j * 8 + 2 * tig + (e & 1);
                            const bool ok = kpos >= a.first && kpos <= a.pos;
                            sc[j][e] = ok ? sc[j][e] * scale_log2 : -INFINITY;
                            if (e < 2) tmax0 = fmaxf(tmax0, sc[j][e]);
                            else tmax1 = fmaxf(tmax1, sc[j][e]);
                        }
                    tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 1));
                    tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 2));
                    tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 1));
                    tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 2));
                    const float mn0 = fmaxf(m0, tmax0), mn1 = fmaxf(m1, tmax1);
                    const float c0 = exp2f(m0 - mn0), c1 = exp2f(m1 - mn1);
                    m0 = mn0;
                    m1 = mn1;
                    const float e00 = exp2f(sc[0][0] - mn0), e01 = exp2f(sc[0][1] - mn0), e02 = exp2f(sc[0][2] - mn1), e03 = exp2f(sc[0][3] - mn1);
                    const float e10 = exp2f(sc[1][0] - mn0), e11 = exp2f(sc[1][1] - mn0), e12 = exp2f(sc[1][2] - mn1), e13 = exp2f(sc[1][3] - mn1);
                    const uint32_t pf[4] = {pack_bf16(e00, e01), pack_bf16(e02, e03), pack_bf16(e10, e11), pack_bf16(e12, e13)};
                    l0 = l0 * c0 + (e00 + e01 + e10 + e11);
                    l1 = l1 * c1 + (e02 + e03 + e12 + e13);
#pragma unroll
                    for (int i = 0; i < HD / 8; ++i) {
                        acc[i][0] *= c0;
                        acc[i][1] *= c0;
                        acc[i][2] *= c1;
                        acc[i][3] *= c1;
                    }
#pragma unroll
                    for (int nt = 0; nt < HD / 8; nt += 2) {
                        uint32_t b[4];
                        const int mi = lane >> 3, r = lane & 7;
                        ldmatrix_x4_trans(b, vs + L::offset(quarter * 16 + (mi & 1) * 8 + r, nt + (mi >> 1)));
                        mma_bf16_16816(acc[nt], pf, b[0], b[1]);
                        mma_bf16_16816(acc[nt + 1], pf, b[2], b[3]);
                    }
                }
            }
            compute_sync();                                               // everyone is done with this pair's buffers
            {
                const int nxt = 2 * (pr + 2);
                if (nxt < a.ntiles && nxt % QUARTER_TILES == 0) {
                    fill_quarters(a, a.my_lo + nxt);
                    compute_sync();
                }
                for (int h = 0; h < 2; ++h)
                    if (nxt + h < a.ntiles) load_tile(a, a.my_lo + nxt + h, (nxt + h) & 3, 0);
                cp_async_commit();
            }
        }
        cp_async_wait<0>();
        compute_sync();

        // ---- merge the eight warps
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        float* wm = reinterpret_cast<float*>(s.xs);                      // [8][16]
        float* wl = wm + COMPUTE_WARPS * 16;
        float* wacc = wl + COMPUTE_WARPS * 16;                           // [8][16][HD]
        if (tig == 0) {
            wm[warp * 16 + gid] = m0;
            wm[warp * 16 + gid + 8] = m1;
            wl[warp * 16 + gid] = l0;
            wl[warp * 16 + gid + 8] = l1;
        }
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            const int d = i * 8 + 2 * tig;
            float* a0 = wacc + ((warp * 16 + gid) * HD + d);
            float* a1 = wacc + ((warp * 16 + gid + 8) * HD + d);
            a0[0] = acc[i][0];
            a0[1] = acc[i][1];
            a1[0] = acc[i][2];
            a1[1] = acc[i][3];
        }
        compute_sync();
        const int rows = min(16, G);
        for (int e = threadIdx.x; e < rows * HD; e += COMPUTE_THREADS) {
            const int r = e / HD, d = e % HD;
            float m = -INFINITY;
#pragma unroll
            for (int w = 0; w < COMPUTE_WARPS; ++w) m = fmaxf(m, wm[w * 16 + r]);
            float l = 0.f, av = 0.f;
            if (m > -INFINITY) {
#pragma unroll
                for (int w = 0; w < COMPUTE_WARPS; ++w) {
                    const float f = exp2f(wm[w * 16 + r] - m);
                    l += wl[w * 16 + r] * f;
                    av += wacc[(w * 16 + r) * HD + d] * f;
                }
            }
            const int h = a.kvh * G + r;
            if (t.splits == 1) {
                static_cast<bf16*>(t.attn_out)[(size_t)a.m * t.ld_attn + (size_t)h * HD + d] = __float2bfloat16_rn(l > 0.f ? av / l : 0.f);
            } else {
                const size_t slot = ((size_t)a.m * t.num_heads + h) * t.splits + a.split;
                t.partial_acc[slot * HD + d] = av;
                if (d == 0) {
                    t.partial_ml[slot * 2] = m;
                    t.partial_ml[slot * 2 + 1] = l;
                }
            }
        }
        if (t.splits == 1) {
            compute_sync();
            return;
        }
        // ---- the last CTA of this (token, KV head) merges the splits, in order
        __threadfence();
        compute_sync();
        if (threadIdx.x == 0) {
            int* counter = t.tickets + a.m * t.num_kv_heads + a.kvh;
            const int ticket = atomicAdd(counter, 1);
            *s.is_last = ticket == t.splits - 1;
            if (*s.is_last) *counter = 0;
        }
        compute_sync();
        if (!*s.is_last) return;
        __threadfence();
        constexpr int QUADS = HD / 4;
        constexpr int MERGE_BATCH = 8;
        float* fac = reinterpret_cast<float*>(s.xs);                      // [rows][splits]
        float* lpart = fac + 16 * t.splits;
        float* inv_l = lpart + 16 * t.splits;
        const size_t head0 = (size_t)a.m * t.num_heads + a.kvh * G;
        for (int e = threadIdx.x; e < rows * t.splits; e += COMPUTE_THREADS) {
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(t.partial_ml) + head0 * t.splits + e);
            fac[e] = ml.x;
            lpart[e] = ml.y;
        }
        for (int q0 = 0; q0 < rows * QUADS; q0 += COMPUTE_THREADS) {
            const int q = q0 + threadIdx.x;
            const bool mine = q < rows * QUADS;
            const int r = mine ? q / QUADS : 0, dq = mine ? q % QUADS : 0;
            const float4* src = reinterpret_cast<const float4*>(t.partial_acc + (head0 + r) * t.splits * HD) + dq;
            float4 part[MERGE_BATCH];
#pragma unroll
            for (int i = 0; i < MERGE_BATCH; ++i)
                if (mine && i < t.splits) part[i] = __ldcg(src + (size_t)i * QUADS);
            if (q0 == 0) {
                compute_sync();
                if (threadIdx.x < rows) {
                    float* f = fac + threadIdx.x * t.splits;
                    const float* lp = lpart + threadIdx.x * t.splits;
                    float m = -INFINITY;
                    for (int s2 = 0; s2 < t.splits; ++s2) m = fmaxf(m, f[s2]);
                    float l = 0.f;
                    for (int s2 = 0; s2 < t.splits; ++s2) {
                        const float w = m > -INFINITY ? exp2f(f[s2] - m) : 0.f;
                        f[s2] = w;
                        l += lp[s2] * w;
                    }
                    inv_l[threadIdx.x] = l > 0.f ? 1.0f / l : 0.f;
                }
                compute_sync();
            }
            if (!mine) continue;
            const float* f = fac + r * t.splits;
            float4 av = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int i = 0; i < MERGE_BATCH; ++i)
                if (i < t.splits) {
                    const float w = f[i];
                    av.x += part[i].x * w; av.y += part[i].y * w; av.z += part[i].z * w; av.w += part[i].w * w;
                }
            for (int s0 = MERGE_BATCH; s0 < t.splits; s0 += MERGE_BATCH) {
#pragma unroll
                for (int i = 0; i < MERGE_BATCH; ++i)
                    if (s0 + i < t.splits) part[i] = __ldcg(src + (size_t)(s0 + i) * QUADS);
#pragma unroll
                for (int i = 0; i < MERGE_BATCH; ++i)
                    if (s0 + i < t.splits) {
                        const float w = f[s0 + i];
                        av.x += part[i].x * w; av.y += part[i].y * w; av.z += part[i].z * w; av.w += part[i].w * w;
                    }
            }
            const float il = inv_l[r];
            const int h = a.kvh * G + r;
            *reinterpret_cast<uint2*>(static_cast<bf16*>(t.attn_out) + (size_t)a.m * t.ld_attn + (size_t)h * HD + dq * 4) =
                make_uint2(pack_bf16(av.x * il, av.y * il), pack_bf16(av.z * il, av.w * il));
        }
        compute_sync();
    }
};

template <int HD>
__device__ __forceinline__ void attention_prefetch(const Params& p, const Shared& s, const EgFusedTemplate& t, const EgFusedOp& op) {
    const int first = first_unit_of(op);
    const int units = p.M * t.num_kv_heads * t.splits;
    if (first >= units) return;
    if (given_up(s)) return;
    Attention<HD> att(p, s, t, op);
    att.prefetch(attn_unit(t, first));
}
template <int HD>
__device__ __forceinline__ void attention_op(const Params& p, const Shared& s, const EgFusedTemplate& t, const EgFusedOp& op, bool prefetched) {
    const int G = (int)gridDim.x;
    const int units = p.M * t.num_kv_heads * t.splits;
    const int first = first_unit_of(op);
    if (first >= units) return;
    if (given_up(s)) {
        cp_async_wait<0>();                                              // copies in flight must land before the memory is used again
        compute_sync();
        return;
    }
    Attention<HD> att(p, s, t, op);
    att.quarter_tile0 = 0;
    for (int u = first; u < units; u += G) {
        const AttnUnit a = attn_unit(t, u);
        if (u == first && prefetched) att.quarter_tile0 = a.my_lo;
        att.run(a, u == first && prefetched);
    }
}

__global__ void __launch_bounds__(THREADS, 1) decode_fused_kernel(const Params p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const Layout l = layout_for(p.stages, p.xs_bytes, p.num_ops, p.num_tmpls);
    Shared s;
    s.ring = smem + l.ring;
    s.xs = smem + l.xs;
    s.red = reinterpret_cast<float*>(smem + l.red);
    s.vals = reinterpret_cast<float*>(smem + l.vals);
    s.factor = reinterpret_cast<float*>(smem + l.factor);
    s.quarters = reinterpret_cast<long long*>(smem + l.quarters);
    s.ops = reinterpret_cast<const EgFusedOp*>(smem + l.ops);
    s.tmpls = reinterpret_cast<const EgFusedTemplate*>(smem + l.tmpls);
    s.full = reinterpret_cast<uint64_t*>(smem + l.bars);
    s.empty = s.full + p.stages;
    s.abort = reinterpret_cast<volatile int*>(smem + l.flags);
    s.is_last = reinterpret_cast<int*>(smem + l.flags) + 1;
    s.decision = reinterpret_cast<int*>(smem + l.flags) + 2;

    // the program into shared memory, the barriers of the ring
    {
        const int op_words = p.num_ops * (int)sizeof(EgFusedOp) / 4, tmpl_words = p.num_tmpls * (int)sizeof(EgFusedTemplate) / 4;
        const uint32_t* src_ops = reinterpret_cast<const uint32_t*>(p.ops);
        const uint32_t* src_tmpls = reinterpret_cast<const uint32_t*>(p.tmpls);
        uint32_t* dst_ops = reinterpret_cast<uint32_t*>(smem + l.ops);
        uint32_t* dst_tmpls = reinterpret_cast<uint32_t*>(smem + l.tmpls);
        for (int i = threadIdx.x; i < op_words; i += THREADS) dst_ops[i] = __ldg(src_ops + i);
        for (int i = threadIdx.x; i < tmpl_words; i += THREADS) dst_tmpls[i] = __ldg(src_tmpls + i);
        if (threadIdx.x == 0) {
            for (int i = 0; i < p.stages; ++i) {
                mbar_init(&s.full[i], 1);
                mbar_init(&s.empty[i], COMPUTE_WARPS);
            }
            *s.abort = 0;
            *s.is_last = 0;
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        }
    }
    __syncthreads();

    if (threadIdx.x >= COMPUTE_THREADS) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(LOADER_REGS));
        if (threadIdx.x < COMPUTE_THREADS + 32) loader(p, s);
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(COMPUTE_REGS));
        RingPlace ring;
        bool prefetched = false;
        for (int i = 0; i < p.num_ops; ++i) {
            const EgFusedOp& op = s.ops[i];
            const EgFusedTemplate& t = s.tmpls[op.tmpl];
            unsigned long long* stamps = p.trace ? p.trace + (size_t)i * 4 : nullptr;
            if (stamps && threadIdx.x == 0) atomicMax(stamps, now_ns());
            if (t.type == EGF_LINEAR) {
                linear_op(p, s, t, op, ring, stamps);
            } else {
                attention_op<64>(p, s, t, op, prefetched);               // (the launcher's caller offers head size 64 only)
                prefetched = false;
            }
            if (stamps && threadIdx.x == 0) atomicMax(stamps + 3, now_ns());
            if (i + 1 < p.num_ops) {
                // what the next operation can fetch before the others have finished this one
                const EgFusedOp& nop = s.ops[i + 1];
                const EgFusedTemplate& nt = s.tmpls[nop.tmpl];
                if (nt.type == EGF_ATTENTION) {
                    compute_sync();                                      // this operation's shared memory is free
                    attention_prefetch<64>(p, s, nt, nop);
                    prefetched = true;
                }
                grid_barrier(p, s, (unsigned)(i + 1));
            }
        }
        cp_async_wait<0>();
    }
    __syncthreads();
}

}  // namespace

// Shared memory a launch needs; 0 if the program does not fit (the caller then runs the step kernel by kernel).
EG_API int eg_decode_fused_smem(int stages, int xs_bytes, int num_ops, int num_tmpls) {
    return layout_for(stages, xs_bytes, num_ops, num_tmpls).total;
}

// `sync` points at 64 words (the barrier's counter, the abort flag, and in a cache line of its own the barrier's flag);
// the launcher zeroes them on the stream.
EG_API int eg_decode_fused(cudaStream_t stream, const void* tmpls, int num_tmpls, const void* ops, int num_ops, int tokens, int stages, int xs_bytes, int ctas,
                           unsigned* sync, int* status, unsigned long long* trace) {
    if (tokens <= 0 || tokens > EGF_MAX_TOKENS || stages < 2 || num_ops <= 0 || ctas <= 0) return (int)cudaErrorInvalidValue;
    const Layout l = layout_for(stages, xs_bytes, num_ops, num_tmpls);
    static int configured = 0;
    if (l.total > configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, l.total);
        if (e != cudaSuccess) return (int)e;
        configured = l.total;
    }
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_fused_kernel, THREADS, l.total);
    if (e != cudaSuccess) return (int)e;
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (per_sm < 1 || ctas > per_sm * sms) return (int)cudaErrorCooperativeLaunchTooLarge;
    e = cudaMemsetAsync(sync, 0, 256, stream);
    if (e != cudaSuccess) return (int)e;
    Params p;
    p.tmpls = static_cast<const EgFusedTemplate*>(tmpls);
    p.ops = static_cast<const EgFusedOp*>(ops);
    p.num_tmpls = num_tmpls;
    p.num_ops = num_ops;
    p.M = tokens;
    p.stages = stages;
    p.xs_bytes = xs_bytes;
    p.sync_counter = sync;
    p.abort_flag = reinterpret_cast<int*>(sync + 1);
    p.status = status;
    p.trace = trace;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = l.total;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, decode_fused_kernel, p);
    return (int)e;
}
