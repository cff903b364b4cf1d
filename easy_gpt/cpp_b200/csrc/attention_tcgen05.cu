// Attention for prompt portions on the 5th-generation tensor cores.
//
// One CTA takes up to 128 consecutive query tokens of one request and one query head, and walks the
// request's keys in the paged cache in tiles of 64 (the portion's own keys were stored there just before):
//
//   S = Q K^T      tcgen05.mma  M 128, N 64, K = head size     Q and K tiles K-major in shared memory, S in TMEM
//   P = softmax    four warps, one query row per thread: the row of S comes out of TMEM with tcgen05.ld, the
//                  reference maximum and the sum stay in registers, P goes back into TMEM as bfloat16 pairs
//                  (tcgen05.st) over the first half of the S buffer it came from
//   O += P V       tcgen05.mma  M 128, N = head size, K 64     P from TMEM, the V tile as it lies in the cache
//                  (N-major operand in shared memory), accumulated in TMEM over all key tiles
// The exponents are taken against a reference that follows the row's maximum lazily: only when the maximum has
// grown by more than 2^8 since the reference was set does the row's thread move the reference, and then it scales
// its row of O in TMEM (tcgen05.ld, multiply, tcgen05.st) and its sum; O / sum stays the same.
//
// Warp roles, in two forms.  With ONE softmax group a CTA has 256 threads of 128 registers and at most 113 KB of shared
// memory, so that two CTAs share an SM and one fills the other's waits; each allocates 256 of the 512 TMEM columns.
// With TWO groups (heads of 64) a CTA has 384 threads and the SM to itself: the groups take the unit's even and odd
// key tiles, each with a reference, a sum, score buffers and an O of its own, and the second hands its rows to the
// first through shared memory when the unit ends.  An SM runs the softmax of two key tiles at a time either way; with
// two groups the longest unit of a prompt, which is what a prompt of a few thousand tokens waits for, takes half as long.
//   warp 0     TMA loads: Q once; per key tile boxes of 64 keys x 64 columns (32 or 16 keys where the pages are no
//              multiple of 64), K and V, 128-byte swizzled, into a ring of stages; every box of a tile has its own
//              lane.  Block-table entries are fetched 32 pieces at a time, a batch ahead.
//   warp 1     allocates TMEM; one thread issues the score products (descriptors ready before it waits: the
//              arithmetic of a descriptor costs more than the issue of the MMA)
//   warps 2-5  the softmax rows (warps 8-11: the second group's)
//   warp 6     one thread issues the output products
// S has three TMEM buffers (two for head size 128): the tensor core computes the scores of later key tiles while
// the rows work on this one.  S_j goes where S and P of three tiles before were, once the output product of that
// tile is done.  Everything is handed over with mbarriers; a barrier's parity tells two phases apart, so every set
// of barriers has as many members as its buffers, and nobody waits on one from further than a phase away.
// Scale, maximum, exponent and sums are 32-bit; the exponent is the hardware's base-2 approximation with the scale
// folded into its multiply-add.
//
// A step with fewer (query tile, head) pairs than CTAs cuts the tiles' key ranges into parts, which are units of
// their own: each writes its unnormalised O, reference and sum, and a small kernel behind this one (launched early; it
// waits for this one by itself) adds a tile's parts up in order.
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT polls the thread raises the CTA's abort flag and
// EG_STATUS_WAIT_TIMEOUT; every role then leaves its loop, the loader waits (bounded again) for the copies it
// still has in flight, and the TMEM is freed as usual.
//
// Takes head sizes 64 and 128, pages of a multiple of 16 tokens, 16-byte aligned rows.  Anything else:
// cudaErrorInvalidValue, and the caller uses the warp-level kernel.
#define EG_NEEDS_TENSOR_MAPS

#include "common.cuh"
#include "mbarrier.cuh"

namespace {

constexpr int BM = 128, BN = 64;
constexpr unsigned WAIT_LIMIT = 1u << 24;
constexpr float REFERENCE_SLACK = 8.f;                            // the exponents' reference may lag the maximum by 2^8
constexpr int SUB_ROW_BYTES = 128;                                // 64 bfloat16: one swizzle row

template <int HD, int WGS>
struct Shape {
    static constexpr int SUBS = HD / 64;                          // 64-column sub-tiles of Q, K, V
    static constexpr int STAGES = WGS == 1 ? (HD == 64 ? 5 : 2) : (HD == 64 ? 8 : 3);
    static constexpr int SCORE_BUFFERS = HD == 64 ? 3 : 2;        // TMEM buffers of S_j / P_j of one softmax group
    static constexpr int THREADS = WGS == 1 ? 256 : 384;          // loader warp, two MMA warps (1 and 6), four softmax warps a group (2-5, 8-11)
    static constexpr int CTAS_PER_SM = WGS == 1 ? 2 : 1;
    static constexpr int Q_SUB_BYTES = BM * SUB_ROW_BYTES;        // 16 KB
    static constexpr int KV_SUB_BYTES = BN * SUB_ROW_BYTES;       // 8 KB
    static constexpr int Q_BYTES = SUBS * Q_SUB_BYTES;
    static constexpr int K_BYTES = SUBS * KV_SUB_BYTES;
    static constexpr int STAGE_BYTES = 2 * K_BYTES;               // K then V
    // where the second softmax group hands its rows to the first at the end of a unit: O as [column][row], then reference and sum
    static constexpr int HANDOVER_BYTES = (WGS - 1) * (HD + 2) * BM * 4;
    static constexpr int SMEM_BYTES = Q_BYTES + STAGES * STAGE_BYTES + HANDOVER_BYTES + 1024;
    // TMEM: the score buffers of group 0, of group 1, then O of either
    static constexpr int O_COL = WGS * SCORE_BUFFERS * BN;
    static constexpr int TMEM_COLS = WGS == 1 ? 256 : 512;        // two CTAs share the SM's 512 columns, or one has them all
    static_assert(O_COL + WGS * HD <= TMEM_COLS, "TMEM columns");
    static_assert(WGS == 1 || WGS == 2, "one or two softmax groups");
};


// Bounded wait: false if it gave up (or another role already did).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status) {
    return mbar_wait_bounded(bar, parity, abort_flag, status, WAIT_LIMIT);
}

// Bounded wait that does not look at the abort flag (for copies in flight at the end).
__device__ __forceinline__ void mbar_wait_plain(uint64_t* bar, uint32_t parity) {
    for (unsigned i = 0; i < WAIT_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return;
}

__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(smem_dst), "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; ACCUMULATE false overwrites D
template <bool ACCUMULATE>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "n"(ACCUMULATE ? 1 : 0) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
template <bool ACCUMULATE>
__device__ __forceinline__ void tc_mma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "n"(ACCUMULATE ? 1 : 0) : "memory");
}
// 32 consecutive columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// Shared-memory matrix descriptors, 128-byte swizzle, rows of 128 bytes, groups of 8 rows 1024 bytes apart.
//   K-major (Q, K, P): 16 elements of K further = 32 bytes further in the row; the leading offset is unused.
//   N-major (V as [key][column]): the 8 x 128-byte group holds 8 keys x 64 columns; 8 keys further = the stride
//   offset (1024 bytes), 64 columns further = the leading offset (the next sub-tile).
__device__ __forceinline__ uint64_t desc_k_major(uint32_t address) {
    uint64_t d = 0;
    d |= (uint64_t)((address & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ uint64_t desc_n_major(uint32_t address, uint32_t leading_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((address & 0x3FFFF) >> 4);
    d |= (uint64_t)((leading_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16 instruction descriptor: D float32, A and B bfloat16, M 128.
__device__ __forceinline__ uint32_t idesc(int n, bool b_n_major) {
    uint32_t d = 0;
    d |= 1u << 4;
    d |= 1u << 7;
    d |= 1u << 10;
    if (b_n_major) d |= 1u << 16;
    d |= (uint32_t)(n >> 3) << 17;
    d |= (uint32_t)(BM >> 4) << 24;
    return d;
}

__device__ __forceinline__ float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// two float32 in a 64-bit register, for the packed instructions
__device__ __forceinline__ uint64_t pair_of(float lo, float hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ void split_pair(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma_pair(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add_pair(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

struct Params {
    const int* block_table;
    int table_stride;
    const int* positions;      // [T]
    const int* tiles;          // [num_tiles][3]: row of the block table, first token, tokens in the tile (<= 128)
    bf16* out;
    long long ldo;
    int num_heads, num_kv_heads, page_size, num_pages, window;
    long long page_rows, head_rows;           // in rows of the cache maps: per page, per KV head
    float scale;
    int* status;
    long long* trace;          // optional (profiling): [32][8] clock stamps of the first CTA's first softmax warp, then per unit
                               // [4]: start, end (ns), SM, key tiles
    // for key ranges cut into parts: per (tile, head, part) 128 rows of unnormalised O, and of (reference, sum)
    float* partial_o;
    float* partial_ml;
    // work queue of the persistent CTAs: [0] next unit, [1] CTAs that have left; both zero before and after a launch
    int* queue;
    int num_tiles, max_parts, part_tiles;
    int piece_rows;            // keys a TMA box of K or V holds: 64, 32 or 16, a divisor of the page size
};

// The 64-bit shared-memory descriptor from its constant high word and a low word (start address, leading offset).
__device__ __forceinline__ uint64_t desc_from(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}
template <int HD, int WGS>
__global__ void __launch_bounds__((Shape<HD, WGS>::THREADS), (Shape<HD, WGS>::CTAS_PER_SM))
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                 const __grid_constant__ CUtensorMap map_v, const Params p) {
    using S = Shape<HD, WGS>;
    constexpr int STAGES = S::STAGES, SCORE_BUFFERS = S::SCORE_BUFFERS, ALL_BUFFERS = WGS * S::SCORE_BUFFERS;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t q_full, k_full[STAGES], v_full[STAGES], kv_empty[STAGES], s_full[ALL_BUFFERS], p_full[ALL_BUFFERS], o_done[ALL_BUFFERS];
    __shared__ int unit_slot[2];                                  // the unit the CTA works on, by round parity
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_addr = base, ring_addr = base + S::Q_BYTES;
    float* const handover = reinterpret_cast<float*>(smem_raw + (base - smem_addr(smem_raw)) + S::Q_BYTES + STAGES * S::STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&kv_empty[s], 1);
        }
        for (int b = 0; b < ALL_BUFFERS; ++b) {
            mbar_init(&s_full[b], 1);
            mbar_init(&p_full[b], 4);                             // one arrival per softmax warp
            mbar_init(&o_done[b], 1);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(&tmem_base_slot)), "r"(S::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    // A unit of work: (query tile, head, part of its key range).  Units are numbered so that the query tiles listed
    // last (of a prompt: those that see most keys) come first, and dealt out through a counter: a CTA that is done
    // with a unit takes the next one, which evens out the SMs' loads.
    // Every role counts alike: gt key tiles before this unit (stage indices and their barriers' phases run on), the
    // key tiles that either softmax group had before this unit (its score buffers and their barriers), units before
    // this one (phase of q_full).  Key tile j of a unit belongs to group j % WGS, as that group's tile j / WGS.
    const int total_units = p.num_tiles * p.num_heads * p.max_parts;
    int gt = 0, units_done = 0, group_tiles[WGS] = {};
    for (int round = 0;; ++round) {
        if (threadIdx.x == 0) {
            int u;
            for (bool own = round == 0;; own = false) {          // the next unit that has keys (at most total_units probes)
                // a CTA's first unit is the one of its own number (no trip to the counter before the CTA's longest unit);
                // the counter deals out the units behind the grid's
                u = own ? (int)blockIdx.x : (int)gridDim.x + atomicAdd(&p.queue[0], 1);
                if (u >= total_units) break;
                const int u_tile = p.num_tiles - 1 - u / (p.max_parts * p.num_heads);
                const int u_t0 = p.tiles[u_tile * 3 + 1], u_count = p.tiles[u_tile * 3 + 2];
                const int u_lo = p.positions[u_t0], u_hi = u_lo + u_count - 1;
                const int u_first = (p.window > 0 && u_lo - p.window + 1 > 0) ? u_lo - p.window + 1 : 0;
                const int u_tiles = u_hi / BN - u_first / BN + 1;
                if (u % p.max_parts < min(p.max_parts, (u_tiles + p.part_tiles - 1) / p.part_tiles)) break;
            }
            unit_slot[round & 1] = u;
        }
        __syncthreads();
        const int unit = unit_slot[round & 1];
        if (unit >= total_units || abort_flag) break;
        const int part = unit % p.max_parts;
        const int h = (unit / p.max_parts) % p.num_heads;
        const int tile = p.num_tiles - 1 - unit / (p.max_parts * p.num_heads);
        const int kvh = h / (p.num_heads / p.num_kv_heads);
        const int seq = p.tiles[tile * 3], t0 = p.tiles[tile * 3 + 1], count = p.tiles[tile * 3 + 2];
        const int pos_lo = p.positions[t0], pos_hi = pos_lo + count - 1;        // positions in a tile are consecutive
        const int first = (p.window > 0 && pos_lo - p.window + 1 > 0) ? pos_lo - p.window + 1 : 0;
        // the key tiles of this query tile, and this unit's part of them
        const int all_lo = first / BN, all_tiles = pos_hi / BN - all_lo + 1;
        const int parts = min(p.max_parts, (all_tiles + p.part_tiles - 1) / p.part_tiles);
        const int part_begin = (int)((long long)all_tiles * part / parts), part_end = (int)((long long)all_tiles * (part + 1) / parts);
        const int tile_lo = all_lo + part_begin, ntiles = part_end - part_begin;
        if (p.trace && threadIdx.x == 0) {                      // profiling: per unit start, end (ns), SM, key tiles
            unsigned long long now;
            unsigned smid;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
            p.trace[256 + unit * 4] = (long long)now;
            p.trace[256 + unit * 4 + 2] = smid;
            p.trace[256 + unit * 4 + 3] = ntiles;
        }

        if (warp == 0) {                                         // ---- TMA loader: one lane per box of a key tile
            // A key tile comes as boxes of `piece_rows` keys (64 where the pages allow it, else 32 or 16) x 64 columns:
            // lane = (sub * 2 + kv) * pieces + g for the 64-column sub-tile, K or V, and the piece.  Issuing a TMA copy
            // costs the issuing thread about ninety cycles and the lanes of a warp take turns at it (measured: eight boxes
            // 700 cycles of the 1,700 that the loader took per tile, more than the softmax rows), so the boxes are as tall
            // as the pages allow.
            const int pieces = BN / p.piece_rows;
            const int g = lane % pieces, is_v = (lane / pieces) & 1, sub = lane / (2 * pieces);
            const bool loads = lane < 2 * pieces * S::SUBS;
            if (lane == 0) {
                mbar_expect_tx(&q_full, S::Q_BYTES);
#pragma unroll
                for (int qs = 0; qs < S::SUBS; ++qs) tma_load_2d(q_addr + qs * S::Q_SUB_BYTES, &map_q, &q_full, h * HD + qs * 64, t0);
            }
            const int* table = p.block_table + (size_t)seq * p.table_stride;
            // The pieces of the unit, numbered through (piece f of the unit is piece f % pieces of key tile f / pieces), are
            // looked up 32 at a time, one by each lane, a batch ahead: the block-table entry, and from it the piece's row in
            // the cache maps.  A piece outside the visible keys reads the last page.
            auto entry_of = [&](int f) {
                const int kpos0 = (tile_lo + f / pieces) * BN + (f % pieces) * p.piece_rows;
                if (f / pieces >= ntiles || kpos0 > pos_hi || kpos0 + p.piece_rows - 1 < first) return p.num_pages - 1;
                return __ldg(table + kpos0 / p.page_size);
            };
            auto row_of = [&](int page, int f) {
                if (page < 0 || page >= p.num_pages) {
                    atomicOr(p.status, EG_STATUS_BAD_PAGE);
                    page = p.num_pages - 1;
                }
                const int kpos0 = (tile_lo + f / pieces) * BN + (f % pieces) * p.piece_rows;
                return (int)((long long)page * p.page_rows + (long long)kvh * p.head_rows + (kpos0 % p.page_size));
            };
            int rows = row_of(entry_of(lane), lane), ahead = entry_of(32 + lane);
            const CUtensorMap* map = is_v ? &map_v : &map_k;
            int issued = 0;
            for (int j = 0; j < ntiles; ++j, ++issued) {
                const int s = (gt + j) % STAGES, use = (gt + j) / STAGES, f0 = j * pieces;
                if (j > 0 && (f0 & 31) == 0) {                   // the next batch of pieces (a tile's pieces lie in one batch)
                    rows = row_of(ahead, f0 + lane);
                    ahead = entry_of(f0 + 32 + lane);
                }
                // one lane polls, the others wait for it at the vote
                if (use > 0 && !__all_sync(0xffffffffu, lane != 0 || mbar_wait(&kv_empty[s], (use - 1) & 1, &abort_flag, p.status))) break;
                if (lane == 0) {
                    mbar_expect_tx(&k_full[s], S::K_BYTES);
                    mbar_expect_tx(&v_full[s], S::K_BYTES);
                }
                const int row = __shfl_sync(0xffffffffu, rows, (f0 + g) & 31);
                __syncwarp();
                if (loads) {
                    const uint32_t dst = ring_addr + s * S::STAGE_BYTES + is_v * S::K_BYTES + sub * S::KV_SUB_BYTES + g * p.piece_rows * SUB_ROW_BYTES;
                    tma_load_2d(dst, map, is_v ? &v_full[s] : &k_full[s], sub * 64, row);
                }
            }
            // every copy has to land before the CTA gives up its shared memory, also when a role has given up
            if (lane == 0 && abort_flag) {
                mbar_wait_plain(&q_full, units_done & 1);
                for (int j = issued > STAGES ? issued - STAGES : 0; j < issued; ++j) {
                    mbar_wait_plain(&k_full[(gt + j) % STAGES], ((gt + j) / STAGES) & 1);
                    mbar_wait_plain(&v_full[(gt + j) % STAGES], ((gt + j) / STAGES) & 1);
                }
            }
        } else if (warp == 1) {
            if (lane == 0) {                                     // ---- issuer of the score products S_j = Q K_j^T
                const uint32_t idesc_s = idesc(BN, false);
                // descriptors differ in their low word only (start address): build the words once
                const uint32_t desc_hi = (uint32_t)(desc_k_major(0) >> 32);
                const uint32_t q_lo = (uint32_t)desc_k_major(q_addr);
                const uint32_t k_lo = (uint32_t)desc_k_major(ring_addr);
                bool ok = mbar_wait(&q_full, units_done & 1, &abort_flag, p.status);
                for (int j = 0; j < ntiles && ok; ++j) {
                    const int n = gt + j;
                    const int g = j % WGS, ng = (g ? group_tiles[WGS - 1] : group_tiles[0]) + j / WGS;    // the group's running tile
                    const int sb = g * SCORE_BUFFERS + ng % SCORE_BUFFERS;
                    const uint32_t stage_lo = k_lo + (uint32_t)(((n % STAGES) * S::STAGE_BYTES) >> 4);
                    const uint32_t d = tmem_base + (uint32_t)(sb * BN);
                    uint64_t a[HD / 16], b[HD / 16];
#pragma unroll
                    for (int kk = 0; kk < HD / 16; ++kk) {
                        a[kk] = desc_from(q_lo + (uint32_t)(((kk / 4) * S::Q_SUB_BYTES + (kk % 4) * 32) >> 4), desc_hi);
                        b[kk] = desc_from(stage_lo + (uint32_t)(((kk / 4) * S::KV_SUB_BYTES + (kk % 4) * 32) >> 4), desc_hi);
                    }
                    // S goes where the group's S and P of SCORE_BUFFERS tiles before were: the product that read that P must be done
                    if (ng >= SCORE_BUFFERS) {
                        ok = mbar_wait(&o_done[sb], (ng / SCORE_BUFFERS - 1) & 1, &abort_flag, p.status);
                        if (!ok) break;
                        tc_fence_after();
                    }
                    ok = mbar_wait(&k_full[n % STAGES], (n / STAGES) & 1, &abort_flag, p.status);
                    if (!ok) break;
                    tc_mma<false>(d, a[0], b[0], idesc_s);
#pragma unroll
                    for (int kk = 1; kk < HD / 16; ++kk) tc_mma<true>(d, a[kk], b[kk], idesc_s);
                    tc_commit(&s_full[sb]);
                }
            }
        } else if (warp == 6) {
            if (lane == 0) {                                     // ---- issuer of the output products O += P_j V_j
                const uint32_t idesc_o = idesc(HD, true);
                const uint32_t desc_hi = (uint32_t)(desc_k_major(0) >> 32);
                const uint32_t v_lo = (uint32_t)desc_n_major(ring_addr + S::K_BYTES, S::KV_SUB_BYTES);
                bool ok = true;
                for (int j = 0; j < ntiles && ok; ++j) {
                    const int n = gt + j;
                    const int g = j % WGS, ng = (g ? group_tiles[WGS - 1] : group_tiles[0]) + j / WGS;
                    const int sb = g * SCORE_BUFFERS + ng % SCORE_BUFFERS;
                    const uint32_t d = tmem_base + (uint32_t)(S::O_COL + g * HD);                  // the group's own O
                    const uint32_t stage_lo = v_lo + (uint32_t)(((n % STAGES) * S::STAGE_BYTES) >> 4);
                    const uint32_t pa = tmem_base + (uint32_t)(sb * BN);                             // P_j: 32 columns of bfloat16 pairs
                    uint64_t b[BN / 16];
#pragma unroll
                    for (int kk = 0; kk < BN / 16; ++kk) b[kk] = desc_from(stage_lo + (uint32_t)((kk * 2048) >> 4), desc_hi);
                    ok = mbar_wait(&v_full[n % STAGES], (n / STAGES) & 1, &abort_flag, p.status) &&
                         mbar_wait(&p_full[sb], (ng / SCORE_BUFFERS) & 1, &abort_flag, p.status);
                    if (!ok) break;
                    tc_fence_after();
                    if (j < WGS) tc_mma_a_tmem<false>(d, pa, b[0], idesc_o);                         // the group's first tile of the unit
                    else tc_mma_a_tmem<true>(d, pa, b[0], idesc_o);
#pragma unroll
                    for (int kk = 1; kk < BN / 16; ++kk) tc_mma_a_tmem<true>(d, pa + (uint32_t)(kk * 8), b[kk], idesc_o);
                    tc_commit(&o_done[sb]);
                    tc_commit(&kv_empty[n % STAGES]);            // K and V of this stage have been read
                }
            }
        } else if ((warp >= 2 && warp < 6) || (WGS > 1 && warp >= 8)) {      // ---- softmax rows, warps 2..5 (and 8..11)
            // With two groups the first takes the unit's even key tiles and the second the odd ones, each with a
            // reference, a sum and an O of its own; at the end of the unit the second hands its rows to the first.
            const int g = (WGS > 1 && warp >= 8) ? 1 : 0;
            const int my_tiles = (ntiles + WGS - 1 - g) / WGS, my_before = g ? group_tiles[WGS - 1] : group_tiles[0];
            const int quad = warp & 3;                           // a warp may touch TMEM lanes 32 * (warp % 4) ..
            const int row = quad * 32 + lane;
            const bool valid = row < count;
            const int qpos = pos_lo + row;
            const int warp_lo = pos_lo + quad * 32, warp_hi = pos_lo + min(count - 1, quad * 32 + 31);
            const int warp_first = (p.window > 0 && warp_lo - p.window + 1 > 0) ? warp_lo - p.window + 1 : 0;
            const bool warp_has_rows = quad * 32 < count;
            const float scale_log2 = p.scale * 1.4426950408889634f;
            const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
            const uint32_t o_lane = lane_base + (uint32_t)(S::O_COL + g * HD);

            // m: the reference of the exponents, a maximum the row has seen (in scaled base-2 units); l: the sum against it
            float m = -INFINITY, l = 0.f;
            bool ok = true;
            const bool tracing = p.trace && blockIdx.x == 0 && round == 0 && threadIdx.x == 64;
#define STAMP(k) if (tracing && i < 32) p.trace[i * 8 + (k)] = clock64();
            for (int i = 0; i < my_tiles; ++i) {
                const int j = g + i * WGS, n = my_before + i, b = g * SCORE_BUFFERS + n % SCORE_BUFFERS;
                STAMP(0)
                ok = __all_sync(0xffffffffu, mbar_wait(&s_full[b], (n / SCORE_BUFFERS) & 1, &abort_flag, p.status));   // the warp stays together
                if (!ok) break;
                tc_fence_after();
                STAMP(1)
                const int key_base = (tile_lo + j) * BN;
                // a key tile that lies wholly behind or before this warp's rows contributes nothing
                const bool skip = !warp_has_rows || key_base > warp_hi || key_base + BN - 1 < warp_first;
                float c = 1.f, ref = 0.f;
                float s[64];
                if (!skip) {
                    {
                        uint32_t r0[32], r1[32];
                        tmem_ld32(lane_base + (uint32_t)(b * BN), r0);
                        tmem_ld32(lane_base + (uint32_t)(b * BN + 32), r1);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            s[e] = __uint_as_float(r0[e]);
                            s[32 + e] = __uint_as_float(r1[e]);
                        }
                    }
                    STAMP(2)
                    // only a tile that crosses the diagonal, the window's far edge or the end of the portion needs limits
                    const bool limits = key_base + BN - 1 > warp_lo || quad * 32 + 31 >= count ||
                                        (p.window > 0 && key_base <= warp_lo + 31 - p.window);
                    if (limits) {
#pragma unroll
                        for (int e = 0; e < 64; ++e) {
                            const int kpos = key_base + e;
                            const bool see = valid && kpos <= qpos && (p.window <= 0 || kpos > qpos - p.window);
                            if (!see) s[e] = -INFINITY;
                        }
                    }
                    // the row's maximum with the three-input instruction: 64 -> 22 -> 8 -> 3 -> 1
                    float t[22];
#pragma unroll
                    for (int e = 0; e < 21; ++e) t[e] = max3(s[3 * e], s[3 * e + 1], s[3 * e + 2]);
                    t[21] = s[63];
#pragma unroll
                    for (int e = 0; e < 7; ++e) t[e] = max3(t[3 * e], t[3 * e + 1], t[3 * e + 2]);
                    t[7] = t[21];
                    t[0] = max3(t[0], t[1], t[2]);
                    t[1] = max3(t[3], t[4], t[5]);
                    t[0] = max3(t[0], t[1], fmaxf(t[6], t[7]));
                    const float mn = t[0] * scale_log2;
                    if (mn > m + REFERENCE_SLACK) {               // also the first finite maximum (m = -inf)
                        c = exp2_approx(m - mn);                 // 0 for the first
                        m = mn;
                    }
                    // a row that has seen nothing keeps m = -inf: 0 as the reference makes exp(-inf - 0) = 0
                    ref = m == -INFINITY ? 0.f : m;
                }
                STAMP(3)
                // Rows whose reference moved scale what they have accumulated so far: the product of the tile before
                // must be done.  (The barriers take turns like the score buffers: a parity tells two phases apart, not
                // more, and nobody who waits on one of them is ever further than one phase from it.)
                if (i > 0 && __any_sync(0xffffffffu, c != 1.f)) {
                    ok = __all_sync(0xffffffffu, mbar_wait(&o_done[g * SCORE_BUFFERS + (n - 1) % SCORE_BUFFERS], ((n - 1) / SCORE_BUFFERS) & 1, &abort_flag, p.status));
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int c0 = 0; c0 < HD; c0 += 16) {
                        uint32_t r[16];
                        tmem_ld16(o_lane + (uint32_t)c0, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 16; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * c);
                        tmem_st16(o_lane + (uint32_t)c0, r);
                    }
                }
                STAMP(4)
                // P_j over the first 32 columns of S_j, element pairs (2e, 2e + 1) of this row, sixteen columns at a time
                // (Multiply-adds and sums on pairs: the packed float32 instructions halve their count.  With two softmax warps
                // on an SM sub-core this loop runs at the exponent unit's rate, 4 results a clock: 1,100 cycles for the two.
                // Measured with every second or every fourth pair's exponent as a polynomial of degree 4 on the
                // multiply-add pipe instead, eleven instructions a pair: 2,100 and 1,600 cycles.  Measured with the next
                // tile's maximum taken inside this loop, from a second read of its scores: 1,780 cycles against 1,100 + 290.  Measured
                // with the two warps of a sub-core taking turns at this loop: 830 cycles each, one after the other, which is
                // no better than 1,100 together; a warp alone does not fill the unit.)
                uint64_t sums = 0;
                const uint64_t scale2 = pair_of(scale_log2, scale_log2), shift2 = pair_of(-ref, -ref);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t packed[16];
                    if (skip) {
#pragma unroll
                        for (int e = 0; e < 16; ++e) packed[e] = 0u;
                    } else {
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            float x0, x1;
                            split_pair(fma_pair(pair_of(s[32 * half + 2 * e], s[32 * half + 2 * e + 1]), scale2, shift2), x0, x1);
                            const float e0 = exp2_approx(x0), e1 = exp2_approx(x1);
                            sums = add_pair(sums, pair_of(e0, e1));
                            packed[e] = pack2(e0, e1);
                        }
                    }
                    tmem_st16(lane_base + (uint32_t)(b * BN + 16 * half), packed);
                }
                float sum0, sum1;
                split_pair(sums, sum0, sum1);
                l = l * c + (sum0 + sum1);
                STAMP(5)
                tmem_st_wait();
                STAMP(6)
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_full[b]);
                STAMP(7)
            }
#undef STAMP
            const int last = my_before + my_tiles - 1;
            if (ok && my_tiles > 0)
                ok = __all_sync(0xffffffffu, mbar_wait(&o_done[g * SCORE_BUFFERS + last % SCORE_BUFFERS], (last / SCORE_BUFFERS) & 1, &abort_flag, p.status));
            // what the groups hold together: the first group's rows take in the second group's
            float o_scale = 1.f;                                 // of this group's O in TMEM
            float other_scale = 0.f;                             // of the other group's O in shared memory (0: nothing there)
            if constexpr (WGS > 1) {
                float* const other_o = handover;                                  // [HD][BM]
                float* const other_ml = handover + HD * BM;                       // [2][BM]
                if (g == 1) {
                    const bool have = ok && my_tiles > 0;
                    other_ml[row] = have ? m : -INFINITY;
                    other_ml[BM + row] = have ? l : 0.f;
                    if (have) {
                        tc_fence_after();
#pragma unroll
                        for (int c0 = 0; c0 < HD; c0 += 32) {
                            uint32_t r[32];
                            tmem_ld32(o_lane + (uint32_t)c0, r);
                            tmem_ld_wait();
#pragma unroll
                            for (int e = 0; e < 32; ++e) other_o[(c0 + e) * BM + row] = __uint_as_float(r[e]);
                        }
                    }
                }
                // both groups, whatever happened before: a wait that gave up must not leave the others at this barrier
                asm volatile("bar.sync 1, %0;\n" ::"n"(WGS * 128) : "memory");
                if (g == 0) {
                    const float m1 = other_ml[row], l1 = other_ml[BM + row];
                    if (m1 != -INFINITY) {
                        const float top = fmaxf(m, m1);
                        o_scale = m == -INFINITY ? 0.f : exp2f(m - top);
                        other_scale = exp2f(m1 - top);
                        l = l * o_scale + l1 * other_scale;
                        m = top;
                    }
                }
            }
            // this row's columns c0 .. c0 + 31 of O, unnormalised: the group's own and, where there is one, the other's
            auto load_o = [&](int c0, float (&v)[32]) {
                uint32_t r[32];
                tmem_ld32(o_lane + (uint32_t)c0, r);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(r[e]);
                if constexpr (WGS > 1) {
                    if (other_scale != 0.f) {
#pragma unroll
                        for (int e = 0; e < 32; ++e) v[e] = fmaf(handover[(c0 + e) * BM + row], other_scale, v[e] * o_scale);
                    }
                }
            };
            if (g != 0) {
                // the second group's rows are with the first
            } else if (ok && parts == 1) {
                tc_fence_after();
                const float inv = l > 0.f ? 1.0f / l : 0.f;
                uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)(t0 + row) * p.ldo + (size_t)h * HD);
#pragma unroll
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    float o[32];
                    load_o(c0, o);
                    if (valid) {
#pragma unroll
                        for (int ch = 0; ch < 4; ++ch) {
                            float v[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e] = o[8 * ch + e] * inv;
                            dst[c0 / 8 + ch] = make_uint4(pack2(v[0], v[1]), pack2(v[2], v[3]), pack2(v[4], v[5]), pack2(v[6], v[7]));
                        }
                    }
                }
            } else if (ok) {
                // One of several parts: the row's unnormalised O, reference and sum go to global memory; a kernel behind
                // this one adds the parts up.
                tc_fence_after();
                const size_t slot0 = ((size_t)tile * p.num_heads + h) * p.max_parts;
                float* my_o = p.partial_o + ((slot0 + part) * BM + row) * HD;
#pragma unroll
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    float o[32];
                    load_o(c0, o);
                    if (valid) {
#pragma unroll
                        for (int e = 0; e < 32; e += 4)
                            *reinterpret_cast<float4*>(my_o + c0 + e) = make_float4(o[e], o[e + 1], o[e + 2], o[e + 3]);
                    }
                }
                if (valid) *reinterpret_cast<float2*>(p.partial_ml + ((slot0 + part) * BM + row) * 2) = make_float2(m, l);
            }
        }
        // the unit is done when its rows are: O in TMEM and Q in shared memory may be overwritten
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        if (p.trace && threadIdx.x == 0) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            p.trace[256 + unit * 4 + 1] = (long long)now;
        }
        gt += ntiles;
#pragma unroll
        for (int w = 0; w < WGS; ++w) group_tiles[w] += (ntiles + WGS - 1 - w) / WGS;
        ++units_done;
    }
    // the last CTA to leave puts the queue back to zero for the next launch
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&p.queue[1], 1) == (int)gridDim.x - 1) {
            p.queue[0] = 0;
            p.queue[1] = 0;
        }
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(S::TMEM_COLS) : "memory");
    }
}

// Adds up the parts of the query tiles whose key ranges were cut: one CTA per (query tile, head), a thread per
// (row, 16 columns); every part's numbers are requested before the first is used.
constexpr int MERGE_MAX_PARTS = 8;
template <int HD>
__global__ void __launch_bounds__(256)
attention_merge_parts_kernel(const Params p) {
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const int tile = blockIdx.x, h = blockIdx.y;
    const int t0 = p.tiles[tile * 3 + 1], count = p.tiles[tile * 3 + 2];
    const int pos_lo = p.positions[t0], pos_hi = pos_lo + count - 1;
    const int first = (p.window > 0 && pos_lo - p.window + 1 > 0) ? pos_lo - p.window + 1 : 0;
    const int all_tiles = pos_hi / BN - first / BN + 1;
    const int parts = min(p.max_parts, (all_tiles + p.part_tiles - 1) / p.part_tiles);
    if (parts <= 1) return;
    const size_t slot0 = ((size_t)tile * p.num_heads + h) * p.max_parts;
    constexpr int GROUPS = HD / 16;
    for (int item = threadIdx.x; item < BM * GROUPS; item += blockDim.x) {
        const int row = item / GROUPS, c0 = (item % GROUPS) * 16;
        if (row >= count) continue;
        float2 ml[MERGE_MAX_PARTS];
#pragma unroll
        for (int i = 0; i < MERGE_MAX_PARTS; ++i)
            ml[i] = i < parts ? __ldcg(reinterpret_cast<const float2*>(p.partial_ml + ((slot0 + i) * BM + row) * 2)) : make_float2(-INFINITY, 0.f);
        float4 v[MERGE_MAX_PARTS][4];
#pragma unroll
        for (int i = 0; i < MERGE_MAX_PARTS; ++i) {
            const float4* src = reinterpret_cast<const float4*>(p.partial_o + ((slot0 + (i < parts ? i : 0)) * BM + row) * HD + c0);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[i][e] = i < parts ? __ldcg(src + e) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float big = -INFINITY;
#pragma unroll
        for (int i = 0; i < MERGE_MAX_PARTS; ++i) big = fmaxf(big, ml[i].x);
        float total = 0.f, w[MERGE_MAX_PARTS];
#pragma unroll
        for (int i = 0; i < MERGE_MAX_PARTS; ++i) {
            w[i] = ml[i].x == -INFINITY ? 0.f : exp2f(ml[i].x - big);                     // -inf: that part saw no key of this row
            total += w[i] * ml[i].y;
        }
        const float inv = total > 0.f ? 1.0f / total : 0.f;
        float acc[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) acc[e] = 0.f;
#pragma unroll
        for (int i = 0; i < MERGE_MAX_PARTS; ++i) {                                       // in order: the sum is the same every time
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc[4 * e] = fmaf(w[i], v[i][e].x, acc[4 * e]);
                acc[4 * e + 1] = fmaf(w[i], v[i][e].y, acc[4 * e + 1]);
                acc[4 * e + 2] = fmaf(w[i], v[i][e].z, acc[4 * e + 2]);
                acc[4 * e + 3] = fmaf(w[i], v[i][e].w, acc[4 * e + 3]);
            }
        }
        uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)(t0 + row) * p.ldo + (size_t)h * HD + c0);
        dst[0] = make_uint4(pack2(acc[0] * inv, acc[1] * inv), pack2(acc[2] * inv, acc[3] * inv), pack2(acc[4] * inv, acc[5] * inv), pack2(acc[6] * inv, acc[7] * inv));
        dst[1] = make_uint4(pack2(acc[8] * inv, acc[9] * inv), pack2(acc[10] * inv, acc[11] * inv), pack2(acc[12] * inv, acc[13] * inv), pack2(acc[14] * inv, acc[15] * inv));
    }
}

// A [rows, cols] bfloat16 matrix with row stride ld (elements), cut into boxes of [box_rows x 64], 128-byte swizzled.
int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    const eg_encode_tiled_fn encode = eg_encode_tiled();
    if (!encode) return (int)cudaErrorNotSupported;
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int HD, int WGS>
int launch(cudaStream_t stream, const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v, const Params& p, int sm_count) {
    using S = Shape<HD, WGS>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tcgen05_kernel<HD, WGS>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const long long units = (long long)p.num_tiles * p.num_heads * p.max_parts, places = (long long)S::CTAS_PER_SM * sm_count;
    const int ctas = (int)(units < places ? units : places);
    attention_prefill_tcgen05_kernel<HD, WGS><<<ctas, S::THREADS, S::SMEM_BYTES, stream>>>(map_q, map_k, map_v, p);
    return eg_launch_status();
}

}  // namespace

// How many softmax groups a CTA of the kernel has for this head size (with two the CTAs have an SM each, with one
// they share it in pairs): what a caller needs to know to count the CTAs.
EG_API int eg_attention_prefill_groups(int head_dim) { return head_dim == 64 ? 2 : 1; }

// q: [total_tokens, >= num_heads * head_dim] bfloat16 with row stride ldq; k_cache / v_cache: [num_pages][num_kv_heads]
// [page_size][head_dim] with the same strides (in elements); the last page must hold finite numbers (pieces of a
// key tile that no query sees are read from it); tiles as in the warp-level prefill kernel, of up to 128 tokens.
// A query tile's keys are cut into parts of about part_tiles key tiles (of 64), at most max_parts (<= 8): partial_o
// takes num_tiles * num_heads * max_parts * 128 * head_dim floats, partial_ml * 128 * 2; queue: two zeroed ints
// (left zero).
EG_API int eg_attention_prefill_tcgen05(cudaStream_t stream, const void* q, long long ldq, int total_tokens, const void* k_cache,
                                        const void* v_cache, const int* block_table, int table_stride, const int* positions,
                                        const int* tiles, int num_tiles, void* out, long long ldo, int num_heads, int num_kv_heads,
                                        int head_dim, int page_size, long long page_stride, long long head_stride, int num_pages,
                                        int window, float scale, int* status, long long* trace, int max_parts, int part_tiles, float* partial_o, float* partial_ml,
                                        int* queue) {
    if (num_tiles <= 0) return 0;
    if (max_parts < 1 || max_parts > MERGE_MAX_PARTS || part_tiles < 1 || !queue || (max_parts > 1 && (!partial_o || !partial_ml)))
        return (int)cudaErrorInvalidValue;
    if ((head_dim != 64 && head_dim != 128) || page_size <= 0 || page_size % 16 || num_kv_heads <= 0 || num_heads % num_kv_heads ||
        num_heads > 65535 || num_pages <= 0 || total_tokens <= 0 || !status)
        return (int)cudaErrorInvalidValue;
    if (ldq % 8 || ldo % 8 || (uintptr_t)q % 16 || (uintptr_t)out % 16 || (uintptr_t)k_cache % 16 || (uintptr_t)v_cache % 16 ||
        page_stride % head_dim || head_stride % head_dim || page_stride <= 0 || head_stride <= 0)
        return (int)cudaErrorInvalidValue;
    Params p{};
    p.block_table = block_table;
    p.table_stride = table_stride;
    p.positions = positions;
    p.tiles = tiles;
    p.out = (bf16*)out;
    p.ldo = ldo;
    p.num_heads = num_heads;
    p.num_kv_heads = num_kv_heads;
    p.page_size = page_size;
    p.num_pages = num_pages;
    p.window = window;
    p.page_rows = page_stride / head_dim;
    p.head_rows = head_stride / head_dim;
    p.scale = scale;
    p.status = status;
    p.trace = trace;
    p.partial_o = partial_o;
    p.partial_ml = partial_ml;
    p.queue = queue;
    p.num_tiles = num_tiles;
    p.max_parts = max_parts;
    p.part_tiles = part_tiles;
    p.piece_rows = page_size % 64 == 0 ? 64 : page_size % 32 == 0 ? 32 : 16;
    // rows of head_dim elements that the cache maps cover: up to the last row of the last page
    const long long kv_rows = (long long)(num_pages - 1) * p.page_rows + (long long)(num_kv_heads - 1) * p.head_rows + page_size;
    if (kv_rows >= (1ll << 31)) return (int)cudaErrorInvalidValue;
    CUtensorMap map_q, map_k, map_v;
    if (make_map(&map_q, q, total_tokens, (long long)num_heads * head_dim, ldq, BM) ||
        make_map(&map_k, k_cache, kv_rows, head_dim, head_dim, p.piece_rows) || make_map(&map_v, v_cache, kv_rows, head_dim, head_dim, p.piece_rows))
        return (int)cudaErrorInvalidValue;
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 148;
    }
    // Persistent CTAs that deal the units out among themselves: one per SM with two softmax groups, which share a
    // unit's key tiles between them, or two per SM with one group each.  Either way an SM runs the softmax of two key
    // tiles at a time, and the tensor core works under it; with two groups the longest unit of a prompt takes half as
    // long.  EASY_GPT_PREFILL_GROUPS=1 or 2 sets the form for a measurement.
    static const int asked = getenv("EASY_GPT_PREFILL_GROUPS") ? atoi(getenv("EASY_GPT_PREFILL_GROUPS")) : 0;
    const int groups = asked == 1 || asked == 2 ? asked : eg_attention_prefill_groups(head_dim);
    int code;
    if (groups == 1) code = head_dim == 64 ? launch<64, 1>(stream, map_q, map_k, map_v, p, sm_count) : launch<128, 1>(stream, map_q, map_k, map_v, p, sm_count);
    else code = head_dim == 64 ? launch<64, 2>(stream, map_q, map_k, map_v, p, sm_count) : launch<128, 2>(stream, map_q, map_k, map_v, p, sm_count);
    if (code || max_parts == 1) return code;
    // the parts are added up behind the main kernel (launched early: it waits for it by itself)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_tiles, num_heads);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)(head_dim == 64 ? cudaLaunchKernelEx(&cfg, attention_merge_parts_kernel<64>, p)
                                : cudaLaunchKernelEx(&cfg, attention_merge_parts_kernel<128>, p));
}
