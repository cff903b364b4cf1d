// Paged grouped-query attention on the warp-level tensor cores (bfloat16), for
// every token of a step: decoded tokens and, until a tiled prefill kernel takes
// them, the tokens of prompt portions too.
//
// One CTA works on (token, KV head, split): the G = NH/NKV query heads that share
// the KV head are the rows of the MMA (padded to 16), so a key tile is read once
// for all of them.  The token's visible keys [first, pos] are cut into tiles of
// 64 keys (aligned to 64, so a tile's 16-key quarters never straddle a page of
// 16, 32, 64, ... tokens); the tiles are dealt to `splits` CTAs in contiguous
// runs, each CTA streams its run through a cp.async pipeline, its four warps take
// a quarter of every tile each, and keep a running softmax (m, l, acc) in
// float32 (src/cuda/ops/self_attn_detail.cuh:325-382).  The warps' states are
// merged in shared memory; with one split the result is written at once, else a
// partial (m, l, acc) goes to scratch memory and the CTA of that (token, KV head)
// that finishes last (a ticket counter; nobody waits) merges the splits in order.
//
// score = (q . k) * scale in float32; the running softmax works in base 2 (scores times
// log2 e, exp2f: one hardware instruction, 2 ulp); P is rounded to bfloat16 for the
// P V product (as V is bfloat16 anyway); sums and the accumulator stay float32.
#include <cstdlib>

#include "mma_utils.cuh"

namespace {

constexpr int TILE_KEYS = 64;
constexpr int THREADS = 128;
constexpr int QUARTER_TILES = 64;      // tiles whose cache addresses are kept in shared memory at a time

// DEEP: as many stages as fit about 96 KB (up to five tiles in flight per CTA, two CTAs per SM): for steps with few
// CTAs, where each has to keep its own loads going.  Otherwise three stages, so that four CTAs share an SM: with
// many CTAs it is their number in flight that hides a tile's latency.
constexpr int MAX_SPLITS = 128;

// TPI: the CTA's warps in fours; TI: key tiles that they work on at a time (a warp takes 16 or 32 keys of a tile)
template <int HD, bool DEEP = true, int TPI = 1, int TI = TPI>
struct Layout {
    static constexpr int CHUNKS = HD / 8;                         // 16-byte chunks per key row
    static constexpr int SWZ = CHUNKS >= 8 ? 7 : CHUNKS - 1;
    static constexpr int TILE_BYTES = TILE_KEYS * HD * 2;          // K or V
    static constexpr int GROUP_BYTES = 2 * TILE_BYTES;             // K and V of one tile
    static constexpr int STAGE_BYTES = TI * GROUP_BYTES;
    // up to five tiles in flight per CTA, within about 96 KB of shared memory (two stages at least)
    static constexpr int DEEP_STAGES = (TPI * 96 * 1024 / STAGE_BYTES) >= 5 ? 5 : ((TPI * 96 * 1024 / STAGE_BYTES) >= 2 ? (TPI * 96 * 1024 / STAGE_BYTES) : 2);
    static constexpr int STAGES = DEEP ? DEEP_STAGES : (DEEP_STAGES < 3 ? DEEP_STAGES : 3);
    static constexpr int WARP_MERGE_BYTES = TPI * 4 * 16 * (HD + 2) * 4;      // the warps' partial results
    static constexpr int SPLIT_MERGE_BYTES = (2 * 16 * MAX_SPLITS + 16) * 4;  // (m, l) of every row and split, 1/l per row
    static constexpr int MERGE_BYTES = WARP_MERGE_BYTES > SPLIT_MERGE_BYTES ? WARP_MERGE_BYTES : SPLIT_MERGE_BYTES;
    static constexpr int SMEM = (STAGES * STAGE_BYTES > MERGE_BYTES) ? STAGES * STAGE_BYTES : MERGE_BYTES;
    __device__ static __forceinline__ int offset(int row, int chunk) {      // bytes inside a K or V tile
        return (row * CHUNKS + (chunk ^ (row & SWZ))) * 16;
    }
};

struct Params {
    const bf16* q;
    int ldq;
    const bf16* k_cache;
    const bf16* v_cache;
    long long page_stride, head_stride;
    const int* block_table;
    int table_stride;
    const int* token_seq;
    const int* positions;
    const int* seq_context;   // [sequences] keys cached before this step (those from it on are written by the kernel in front); may be null
    bf16* out;
    int ldo;
    float* partial_acc;       // [T, NH, splits, HD]
    float* partial_ml;        // [T, NH, splits, 2]
    int num_heads, num_kv_heads, page_size, num_pages, window, splits;
    float scale;
    int* status;
    const void* prefetch;         // weights of a kernel that runs soon: pulled into L2 meanwhile
    long long prefetch_bytes;
    int* counters;                // [tokens of this launch * gridDim.y] tickets, zero before and after every launch
    int use_pdl;
    unsigned long long* trace;    // optional: [2] earliest start / latest end of this launch's CTAs (%globaltimer, ns)
    const int* token_list;        // optional: the tokens this launch works on (blockIdx.x indexes it); null: all, in order
    int cluster_merge;            // the splits of a (token, KV head) are one cluster and are merged in its first CTA's shared memory
};

template <int HD, bool DEEP, int TPI, int KW>
__global__ void __launch_bounds__(TPI * THREADS) attention_paged_kernel(const Params p) {
    constexpr int TI = TPI * KW / 16;                                // key tiles of an iteration
    constexpr int KB = KW / 16;                                      // blocks of 16 keys a warp takes of its tile
    using L = Layout<HD, DEEP, TPI, TI>;
    constexpr int NT = TPI * THREADS;                                // threads of the CTA
    constexpr int WARPS = TPI * 4;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int is_last;
    TraceScope trace_scope(p.trace);
    const int t = p.token_list ? p.token_list[blockIdx.x] : blockIdx.x;
    const int G = p.num_heads / p.num_kv_heads;
    const int gblocks = (G + 15) / 16;
    const int kvh = blockIdx.y / gblocks;
    const int g0 = (blockIdx.y % gblocks) * 16;                   // first query head of the group handled here
    const int split = blockIdx.z;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;

    if (p.prefetch) {
        constexpr long long PIECE = 4096;
        const long long pieces = (p.prefetch_bytes + PIECE - 1) / PIECE;
        const long long cta = ((long long)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
        const long long ctas = (long long)gridDim.x * gridDim.y * gridDim.z;
        for (long long i = cta * NT + threadIdx.x; i < pieces; i += ctas * NT) {
            const long long off = i * PIECE;
            const long long n = p.prefetch_bytes - off < PIECE ? p.prefetch_bytes - off : PIECE;
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(static_cast<const char*>(p.prefetch) + off),
                         "r"((unsigned)(n & ~15LL)) : "memory");
        }
    }
    // Positions and block tables were uploaded before the step and the cached keys were written by earlier
    // steps, so everything up to the first fresh key can be fetched before the kernel in front has finished.
    if (p.use_pdl == 1) asm volatile("griddepcontrol.launch_dependents;\n" ::);
    const int pos = p.positions[t];
    const int fresh_from = p.seq_context ? p.seq_context[p.token_seq[t]] : 0;
    const int first = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const int* table = p.block_table + (size_t)p.token_seq[t] * p.table_stride;
    const int tile_lo = first / TILE_KEYS, tile_hi = pos / TILE_KEYS;           // inclusive
    const int per = (tile_hi - tile_lo + 1 + p.splits - 1) / p.splits;
    const int my_lo = tile_lo + split * per;
    const int my_hi = min(tile_hi, my_lo + per - 1);
    const int ntiles = my_hi - my_lo + 1;                                       // may be <= 0

    // Where every 16-key quarter of this CTA's tiles starts in the cache (element offset, -1: nothing to read):
    // looked up once through the block table, so that the tile loads below touch no global metadata.
    __shared__ long long quarter_base[QUARTER_TILES * 4];
    int quarter_tile0 = my_lo;
    auto fill_quarters = [&](int tile0) {
        quarter_tile0 = tile0;
        const int count = min(QUARTER_TILES, my_hi - tile0 + 1);
        for (int e = threadIdx.x; e < count * 4; e += NT) {
            const int kpos0 = (tile0 + e / 4) * TILE_KEYS + (e % 4) * 16;
            long long base = -1;
            if (kpos0 <= pos && kpos0 + 15 >= first) {
                const int page = table[kpos0 / p.page_size];
                if (page < 0 || page >= p.num_pages) atomicOr(p.status, EG_STATUS_BAD_PAGE);
                else base = (long long)page * p.page_stride + (long long)kvh * p.head_stride + (long long)(kpos0 % p.page_size) * HD;
            }
            quarter_base[e] = base;
        }
    };
    if (ntiles > 0) fill_quarters(my_lo);
    __syncthreads();

    // mode 0: every row; 1 (before the wait): all but the fresh keys; 2 (after it): the fresh keys only
    auto load_one = [&](int tile, unsigned char* ks, int mode) {
        unsigned char* vs = ks + L::TILE_BYTES;
        const long long* qb = quarter_base + (tile - quarter_tile0) * 4;
        for (int e = threadIdx.x; e < TILE_KEYS * L::CHUNKS; e += NT) {
            const int row = e / L::CHUNKS, chunk = e % L::CHUNKS;
            const int kpos = tile * TILE_KEYS + row;
            const long long base = qb[row >> 4];
            const bool valid = kpos >= first && kpos <= pos && base >= 0;
            const bool fresh = kpos >= first && kpos <= pos && kpos >= fresh_from;
            if ((mode == 1 && fresh) || (mode == 2 && !fresh)) continue;
            const long long off = valid ? base + (long long)(row & 15) * HD + chunk * 8 : 0;
            cp_async_16(ks + L::offset(row, chunk), p.k_cache + off, valid);
            cp_async_16(vs + L::offset(row, chunk), p.v_cache + off, valid);
        }
    };
    // the TPI tiles of iteration `it` into stage `stage` (those that exist); fresh_only: only tiles that hold fresh keys
    auto load_tile = [&](int it_tile0, int stage, int mode) {
#pragma unroll
        for (int g = 0; g < TI; ++g) {
            const int tile = it_tile0 + g;
            if (tile > my_hi) break;
            if (mode == 2 && (tile + 1) * TILE_KEYS <= fresh_from) continue;
            load_one(tile, smem + stage * L::STAGE_BYTES + g * L::GROUP_BYTES, mode);
        }
    };
    const int niter = ntiles > 0 ? (ntiles + TI - 1) / TI : 0;

    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;                 // rows gid and gid + 8
    float acc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;

#pragma unroll
    for (int s = 0; s < L::STAGES - 1; ++s) {
        if (s < niter) load_tile(my_lo + s * TI, s, 1);
        cp_async_commit();
    }
    trace_scope.mark(0);
    if (p.use_pdl) asm volatile("griddepcontrol.wait;\n" ::: "memory");     // q and the fresh keys come from the kernel in front
    if (p.use_pdl == 2) asm volatile("griddepcontrol.launch_dependents;\n" ::);
    trace_scope.mark(1);
#pragma unroll
    for (int s = 0; s < L::STAGES - 1; ++s)
        if (s < niter) load_tile(my_lo + s * TI, s, 2);
    cp_async_commit();

    // ---- query rows as A fragments: row r <-> head kvh*G + g0 + r
    uint32_t qf[HD / 16][4];
    {
        const int r0 = g0 + gid, r1 = g0 + gid + 8;
        const bf16* q0 = p.q + (size_t)t * p.ldq + (size_t)(kvh * G + r0) * HD;
        const bf16* q1 = p.q + (size_t)t * p.ldq + (size_t)(kvh * G + r1) * HD;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            const int d = ks * 16 + 2 * tig;
            qf[ks][0] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0 + d) : 0u;
            qf[ks][1] = r1 < G ? *reinterpret_cast<const uint32_t*>(q1 + d) : 0u;
            qf[ks][2] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0 + d + 8) : 0u;
            qf[ks][3] = r1 < G ? *reinterpret_cast<const uint32_t*>(q1 + d + 8) : 0u;
        }
    }


    constexpr int WARPS_PER_TILE = TILE_KEYS / KW;
    const int group = warp / WARPS_PER_TILE, key0 = (warp % WARPS_PER_TILE) * KW;   // which tile of the iteration, which keys of it
    for (int it = 0; it < niter; ++it) {
        if (it == 0) cp_async_wait<0>();                                          // the first tiles and their fresh rows
        else cp_async_wait<L::STAGES - 2>();
        __syncthreads();
        if (it == 0) trace_scope.mark(2);
        {   // prefetch the tile STAGES-1 ahead into the stage freed by the previous iteration
            const int nxt = it + L::STAGES - 1;
            if (nxt < niter && (nxt * TI) % QUARTER_TILES == 0) {                 // the next stretch of the block table
                fill_quarters(my_lo + nxt * TI);
                __syncthreads();
            }
            if (nxt < niter) load_tile(my_lo + nxt * TI, nxt % L::STAGES, 0);
            cp_async_commit();
        }
        const unsigned char* ks = smem + (it % L::STAGES) * L::STAGE_BYTES + group * L::GROUP_BYTES;
        const unsigned char* vs = ks + L::TILE_BYTES;
        if (it * TI + group >= ntiles) continue;                                  // the run has no tile for this group of warps any more
        const int key_base = (my_lo + it * TI + group) * TILE_KEYS + key0;        // this warp's KW keys
        if (key_base > pos || key_base + KW - 1 < first) continue;                // nothing visible in them

        // S = Q K^T for 16 rows x KW keys
        float s[2 * KB][4];
#pragma unroll
        for (int j = 0; j < 2 * KB; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                uint32_t b[4];
                const int mi = lane >> 3, r = lane & 7;
                ldmatrix_x4(b, ks + L::offset(key0 + kb * 16 + (mi >> 1) * 8 + r, kk * 2 + (mi & 1)));
                mma_bf16_16816(s[2 * kb], qf[kk], b[0], b[1]);
                mma_bf16_16816(s[2 * kb + 1], qf[kk], b[2], b[3]);
            }
        }
        // scale, mask, running softmax
        float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2 * KB; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kpos = key_base + j * 8 + 2 * tig + (e & 1);
                const bool ok = kpos >= first && kpos <= pos;
                s[j][e] = ok ? s[j][e] * scale_log2 : -INFINITY;
                if (e < 2) tmax0 = fmaxf(tmax0, s[j][e]); else tmax1 = fmaxf(tmax1, s[j][e]);
            }
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 1));
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 2));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 1));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 2));
        const float mn0 = fmaxf(m0, tmax0), mn1 = fmaxf(m1, tmax1);               // finite: a key of these is visible
        const float c0 = exp2f(m0 - mn0), c1 = exp2f(m1 - mn1);
        m0 = mn0;
        m1 = mn1;
        uint32_t pf[KB][4];
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
            const float (&sa)[4] = s[2 * kb];
            const float (&sb)[4] = s[2 * kb + 1];
            const float e00 = exp2f(sa[0] - mn0), e01 = exp2f(sa[1] - mn0), e02 = exp2f(sa[2] - mn1), e03 = exp2f(sa[3] - mn1);
            const float e10 = exp2f(sb[0] - mn0), e11 = exp2f(sb[1] - mn0), e12 = exp2f(sb[2] - mn1), e13 = exp2f(sb[3] - mn1);
            ps0 += (e00 + e01) + (e10 + e11);
            ps1 += (e02 + e03) + (e12 + e13);
            pf[kb][0] = pack_bf16(e00, e01);
            pf[kb][1] = pack_bf16(e02, e03);
            pf[kb][2] = pack_bf16(e10, e11);
            pf[kb][3] = pack_bf16(e12, e13);
        }
        l0 = l0 * c0 + ps0;
        l1 = l1 * c1 + ps1;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            acc[i][0] *= c0;
            acc[i][1] *= c0;
            acc[i][2] *= c1;
            acc[i][3] *= c1;
        }
        // acc += P V
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
            for (int nt = 0; nt < HD / 8; nt += 2) {
                uint32_t b[4];
                const int mi = lane >> 3, r = lane & 7;
                ldmatrix_x4_trans(b, vs + L::offset(key0 + kb * 16 + (mi & 1) * 8 + r, nt + (mi >> 1)));
                mma_bf16_16816(acc[nt], pf[kb], b[0], b[1]);
                mma_bf16_16816(acc[nt + 1], pf[kb], b[2], b[3]);
            }
    }
    cp_async_wait<0>();
    trace_scope.mark(3, true);
    __syncthreads();                                                              // the pipeline's memory is free now

    // ---- merge the four warps: rows r = gid, gid + 8
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    float* wm = reinterpret_cast<float*>(smem);                                   // [WARPS][16]
    float* wl = wm + WARPS * 16;                                                  // [WARPS][16]
    float* wacc = wl + WARPS * 16;                                                // [WARPS][16][HD]
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
    // Splits as a cluster: every CTA of it is past its key tiles here, so the first CTA's pipeline memory is free for
    // the others' results (behind the part that its own warps' merge still uses).
    unsigned cluster_rank = 0;
    uint32_t incoming = 0;                                                         // [splits][rows][HD + 2] in the first CTA
    if (p.cluster_merge) {
        asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(cluster_rank));
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(incoming) : "r"(smem_u32(smem + L::WARP_MERGE_BYTES)), "r"(0));
        asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    } else {
        __syncthreads();
    }
    const int rows = min(16, G - g0);
    for (int e = threadIdx.x; e < rows * HD; e += NT) {
        const int r = e / HD, d = e % HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, wm[w * 16 + r]);
        float l = 0.f, a = 0.f;
        if (m > -INFINITY) {
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float f = exp2f(wm[w * 16 + r] - m);                          // -inf -> 0
                l += wl[w * 16 + r] * f;
                a += wacc[(w * 16 + r) * HD + d] * f;
            }
        }
        const int h = kvh * G + g0 + r;
        if (p.splits == 1) {
            p.out[(size_t)t * p.ldo + (size_t)h * HD + d] = __float2bfloat16_rn(l > 0.f ? a / l : 0.f);
        } else if (p.cluster_merge) {
            const uint32_t at = incoming + (uint32_t)((cluster_rank * rows + r) * (HD + 2)) * 4u;
            asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(at + (uint32_t)d * 4u), "f"(a) : "memory");
            if (d == 0) {
                asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(at + (uint32_t)HD * 4u), "f"(m) : "memory");
                asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(at + (uint32_t)(HD + 1) * 4u), "f"(l) : "memory");
            }
        } else {
            const size_t slot = ((size_t)t * p.num_heads + h) * p.splits + split;
            p.partial_acc[slot * HD + d] = a;
            if (d == 0) {
                p.partial_ml[slot * 2] = m;
                p.partial_ml[slot * 2 + 1] = l;
            }
        }
    }
    trace_scope.mark(4);
    if (p.splits == 1) return;
    if (p.cluster_merge) {
        asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
        trace_scope.mark(5);
        if (cluster_rank != 0) return;
        // out = sum_s acc_s e^{m_s - m} / sum_s l_s e^{m_s - m}, the splits in order, from this CTA's own shared memory
        const float* inc = reinterpret_cast<const float*>(smem + L::WARP_MERGE_BYTES);
        constexpr int QUADS = HD / 4;
        for (int q = threadIdx.x; q < rows * QUADS; q += NT) {
            const int r = q / QUADS, dq = q % QUADS;
            float m = -INFINITY;
            for (int s2 = 0; s2 < p.splits; ++s2) m = fmaxf(m, inc[(size_t)(s2 * rows + r) * (HD + 2) + HD]);
            float l = 0.f;
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s2 = 0; s2 < p.splits; ++s2) {
                const float* part = inc + (size_t)(s2 * rows + r) * (HD + 2);
                const float w = m > -INFINITY ? exp2f(part[HD] - m) : 0.f;
                l += part[HD + 1] * w;
                const float2 lo = *reinterpret_cast<const float2*>(part + dq * 4), hi = *reinterpret_cast<const float2*>(part + dq * 4 + 2);
                a.x += lo.x * w; a.y += lo.y * w; a.z += hi.x * w; a.w += hi.y * w;
            }
            const float il = l > 0.f ? 1.0f / l : 0.f;
            const int h = kvh * G + g0 + r;
            *reinterpret_cast<uint2*>(p.out + (size_t)t * p.ldo + (size_t)h * HD + dq * 4) =
                make_uint2(pack_bf16(a.x * il, a.y * il), pack_bf16(a.z * il, a.w * il));
        }
        return;
    }

    // ---- the last CTA of this (token, KV head) to get here merges the splits, in order:
    // out = sum_s acc_s e^{m_s - m} / sum_s l_s e^{m_s - m}
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* counter = p.counters + (size_t)blockIdx.x * gridDim.y + blockIdx.y;   // by the token's place in this launch
        const int ticket = atomicAdd(counter, 1);
        is_last = ticket == p.splits - 1;
        if (is_last) *counter = 0;                                                // all have arrived: ready for the next launch
    }
    __syncthreads();
    trace_scope.mark(5);
    if (!is_last) return;
    __threadfence();
    // Every load of the merge is issued before anything waits: (m, l) of all (row, split) pairs, and the first
    // MERGE_BATCH splits of the accumulators, a float4 of one row per thread.  One trip to the L2 instead of several.
    constexpr int MERGE_BATCH = 16;
    constexpr int QUADS = HD / 4;
    float* fac = reinterpret_cast<float*>(smem);                                  // [rows][splits]: m_s, then e^{m_s - m}
    float* lpart = fac + 16 * p.splits;                                            // [rows][splits]: l_s
    float* inv_l = lpart + 16 * p.splits;                                          // [rows]
    const size_t head0 = (size_t)t * p.num_heads + kvh * G + g0;
    for (int e = threadIdx.x; e < rows * p.splits; e += NT) {
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.partial_ml) + head0 * p.splits + e);   // rows are consecutive heads
        fac[e] = ml.x;
        lpart[e] = ml.y;
    }
    for (int q0 = 0; q0 < rows * QUADS; q0 += NT) {
        const int q = q0 + threadIdx.x;
        const bool mine = q < rows * QUADS;
        const int r = mine ? q / QUADS : 0, dq = mine ? q % QUADS : 0;
        const float4* src = reinterpret_cast<const float4*>(p.partial_acc + (head0 + r) * p.splits * HD) + dq;
        float4 part[MERGE_BATCH];
#pragma unroll
        for (int i = 0; i < MERGE_BATCH; ++i)
            if (mine && i < p.splits) part[i] = __ldcg(src + (size_t)i * QUADS);
        if (q0 == 0) {
            __syncthreads();
            if (threadIdx.x < rows) {
                float* f = fac + threadIdx.x * p.splits;
                const float* lp = lpart + threadIdx.x * p.splits;
                float m = -INFINITY;
                for (int s2 = 0; s2 < p.splits; ++s2) m = fmaxf(m, f[s2]);
                float l = 0.f;
                for (int s2 = 0; s2 < p.splits; ++s2) {                             // in order
                    const float w = m > -INFINITY ? exp2f(f[s2] - m) : 0.f;
                    f[s2] = w;
                    l += lp[s2] * w;
                }
                inv_l[threadIdx.x] = l > 0.f ? 1.0f / l : 0.f;
            }
            __syncthreads();
        }
        if (!mine) continue;
        const float* f = fac + r * p.splits;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < MERGE_BATCH; ++i)
            if (i < p.splits) {
                const float w = f[i];
                a.x += part[i].x * w; a.y += part[i].y * w; a.z += part[i].z * w; a.w += part[i].w * w;
            }
        for (int s0 = MERGE_BATCH; s0 < p.splits; s0 += MERGE_BATCH) {             // further splits, a batch in flight at a time
#pragma unroll
            for (int i = 0; i < MERGE_BATCH; ++i)
                if (s0 + i < p.splits) part[i] = __ldcg(src + (size_t)(s0 + i) * QUADS);
#pragma unroll
            for (int i = 0; i < MERGE_BATCH; ++i)
                if (s0 + i < p.splits) {
                    const float w = f[s0 + i];
                    a.x += part[i].x * w; a.y += part[i].y * w; a.z += part[i].z * w; a.w += part[i].w * w;
                }
        }
        const float il = inv_l[r];
        const int h = kvh * G + g0 + r;
        *reinterpret_cast<uint2*>(p.out + (size_t)t * p.ldo + (size_t)h * HD + dq * 4) =
            make_uint2(pack_bf16(a.x * il, a.y * il), pack_bf16(a.z * il, a.w * il));
    }
}

template <int HD, bool DEEP, int TPI = 1, int KW = 16>
int launch_with(cudaStream_t stream, const Params& p, dim3 grid, bool must_cluster = false) {
    using L = Layout<HD, DEEP, TPI, TPI * KW / 16>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_paged_kernel<HD, DEEP, TPI, KW>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(TPI * THREADS);
    cfg.dynamicSmemBytes = L::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int nattr = 0;
    if (p.use_pdl) {
        attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[nattr].val.programmaticStreamSerializationAllowed = 1;
        ++nattr;
    }
    // The splits of a (token, KV head) as one cluster (up to 16 CTAs, which needs the kernel's leave for a cluster of
    // more than 8), merged through the first CTA's shared memory instead of scratch memory and a ticket: for the
    // launches of fewer CTAs than SMs, and for those of many small CTAs.
    Params q = p;
    static const bool cluster_allowed = !(getenv("EASY_GPT_CLUSTER_MERGE") && atoi(getenv("EASY_GPT_CLUSTER_MERGE")) == 0);
    const int G = p.num_heads / p.num_kv_heads;
    const size_t incoming_bytes = (size_t)p.splits * (G < 16 ? G : 16) * (HD + 2) * sizeof(float);
    // (Measured on B200, 16 splits, context 4096: at batch 1 the step takes 0.708 ms with it against 0.749, at batch 4
    // 0.753 against 0.777; at batch 8, 256 CTAs in 16 clusters, 0.966 against 0.826: so many clusters of 16 find room
    // only when the kernel in front has left the SMs, and the early start is lost.)
    int sms = 0, device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const long long ctas = (long long)grid.x * grid.y * grid.z;
    // Launches of many CTAs (four an SM): clusters of up to 8 (batch 24 / 32 / 64: 1.288 / 1.370 / 1.604 ms a step with
    // them, 1.307 / 1.394 / 1.65 without).
    if (cluster_allowed && ((DEEP && ctas <= sms) || (!DEEP && p.splits <= 8)) && p.splits > 1 && p.splits <= 16 &&
        L::WARP_MERGE_BYTES + incoming_bytes <= (size_t)L::SMEM) {
        static int leave = 0;                                                      // 0 not asked yet, 1 given, -1 refused
        if (!leave) leave = cudaFuncSetAttribute(attention_paged_kernel<HD, DEEP, TPI, KW>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess ? 1 : -1;
        if (p.splits <= 8 || leave == 1) {
            attr[nattr].id = cudaLaunchAttributeClusterDimension;
            attr[nattr].val.clusterDim.x = 1;
            attr[nattr].val.clusterDim.y = 1;
            attr[nattr].val.clusterDim.z = (unsigned)p.splits;
            cfg.attrs = attr;
            cfg.numAttrs = nattr + 1;
            int clusters = 0;
            // all clusters have to be on the GPU together, or the last ones run as a second wave (measured: batch 8, 16
            // clusters of 8 CTAs, of which 15 found room: the step took 0.92 ms instead of 0.80)
            if (cudaOccupancyMaxActiveClusters(&clusters, attention_paged_kernel<HD, DEEP, TPI, KW>, &cfg) == cudaSuccess &&
                clusters >= (int)(grid.x * grid.y)) {
                q.cluster_merge = 1;
                ++nattr;
            } else {
                (void)cudaGetLastError();
            }
        }
    }
    if (must_cluster && !q.cluster_merge) return -1;                              // the caller has another way
    cfg.attrs = attr;
    cfg.numAttrs = nattr;
    return (int)cudaLaunchKernelEx(&cfg, attention_paged_kernel<HD, DEEP, TPI, KW>, q);
}

template <int HD>
int launch(cudaStream_t stream, const Params& p, int tokens) {
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 148;
    }
    const int G = p.num_heads / p.num_kv_heads;
    const dim3 grid(tokens, p.num_kv_heads * ((G + 15) / 16), p.splits);
    const long long ctas = (long long)grid.x * grid.y * grid.z;
    // Up to twice as many CTAs as SMs: eight warps a CTA take two key tiles at a time and half as many splits (the same
    // warps, tiles in flight and trips through the keys as with four warps), so that the splits of a (token, KV head)
    // are at most 8 CTAs, one an SM, and can be merged as a cluster.  All clusters have to find room at once; if they
    // do not, a split or two fewer may.  (Measured on B200, context 4096, ms a decode step with / without: batch 1
    // 0.681 / 0.749, batch 4 0.702 / 0.777, batch 7 0.732; batch 8: 16 clusters of 8 do not find room.)
    // A long run of key tiles is a stream, and streams want all SMs: at the 0.5B sizes, batch 8, context 32k, 7 splits in
    // 16 clusters are 112 CTAs and the step takes 1.59 ms with them, 1.45 with 256 four-warp CTAs.
    constexpr int WIDE_KEYS = HD <= 64 ? 32 : 16;                                // keys a warp of the eight-warp form takes of a tile
    const long long most_tiles = ((long long)p.table_stride * p.page_size + TILE_KEYS - 1) / TILE_KEYS;
    if constexpr (HD <= 128) if (ctas <= 2ll * sm_count && p.splits >= 4 && p.splits % 2 == 0) {
        for (int fewer = 0; fewer <= 2; ++fewer) {
            Params half = p;
            half.splits = p.splits / 2 - fewer;
            if (half.splits < 2) break;
            // long runs: only if the clusters still cover most of the SMs (7B sizes, batch 8, context 8k: 4.05 ms a step with
            // 32 clusters of 4, 5.08 with 256 four-warp CTAs and tickets)
            if (most_tiles > 16ll * half.splits && (long long)grid.x * grid.y * half.splits * 100 < 85ll * sm_count) break;
            const int rc = launch_with<HD, true, 2, WIDE_KEYS>(stream, half, dim3(grid.x, grid.y, half.splits), true);
            if (rc != -1) return rc;
        }
    }
    return ctas <= 2ll * sm_count ? launch_with<HD, true>(stream, p, grid) : launch_with<HD, false>(stream, p, grid);
}


// ---------------------------------------------------------------------------
// Prompt portions: 64 consecutive query tokens of one request (half of a listed
// tile) and one query head per CTA (four warps of 16 rows), against key tiles of 64 from the
// paged cache — the portion's own keys were stored there just before.  The K/V
// tiles of a KV head are read by the CTAs of its G query heads at about the same
// time and come from the L2 after the first.  Causal and window limits are
// applied per element; the running softmax is the same as above.
// ---------------------------------------------------------------------------

// 2^x by the hardware's approximation (relative error about 2^-22; results below 2^-126 become 0, and -inf gives 0).
__device__ __forceinline__ float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct PrefillParams {
    const bf16* q;
    int ldq;
    const bf16* k_cache;
    const bf16* v_cache;
    long long page_stride, head_stride;
    const int* block_table;
    int table_stride;
    const int* positions;      // [T]
    const int* tiles;          // [num_tiles][3]: sequence (row of the block table), first token, tokens in the tile (<= 128)
    bf16* out;
    int ldo;
    int num_heads, num_kv_heads, page_size, num_pages, window;
    float scale;
    int* status;
};

template <int HD>
struct PrefillLayout {
    static constexpr int CHUNKS = HD / 8;
    static constexpr int TILE_BYTES = TILE_KEYS * HD * 2;
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    static constexpr int STAGES = 3;
    static constexpr int SMEM = STAGES * STAGE_BYTES;
};

template <int HD>
__global__ void __launch_bounds__(THREADS, HD <= 64 ? 4 : 2) attention_prefill_kernel(const PrefillParams p) {
    using L = Layout<HD>;
    using PL = PrefillLayout<HD>;
    extern __shared__ __align__(128) unsigned char smem[];
    // later tiles of a request see more keys: start them first
    const int item = gridDim.x - 1 - blockIdx.x;
    const int tile = item >> 1, half = item & 1;                 // a listed tile has up to 128 tokens: two CTAs
    const int h = blockIdx.y;
    const int kvh = h / (p.num_heads / p.num_kv_heads);
    const float scale_log2 = p.scale * 1.4426950408889634f;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int seq = p.tiles[tile * 3], t0 = p.tiles[tile * 3 + 1] + half * TILE_KEYS;
    const int count = min(TILE_KEYS, p.tiles[tile * 3 + 2] - half * TILE_KEYS);
    if (count <= 0) return;
    const int* table = p.block_table + (size_t)seq * p.table_stride;
    const int pos_lo = p.positions[t0], pos_hi = pos_lo + count - 1;           // positions in a tile are consecutive
    const int first = (p.window > 0 && pos_lo - p.window + 1 > 0) ? pos_lo - p.window + 1 : 0;
    const int tile_lo = first / TILE_KEYS, ntiles = pos_hi / TILE_KEYS - tile_lo + 1;

    // rows of this warp: r0 = warp*16 + gid, r1 = r0 + 8
    const int r0 = warp * 16 + gid, r1 = r0 + 8;
    const bool v0 = r0 < count, v1 = r1 < count;
    const int qp0 = pos_lo + r0, qp1 = pos_lo + r1;
    uint32_t qf[HD / 16][4];
    {
        const bf16* q0 = p.q + (size_t)(t0 + (v0 ? r0 : 0)) * p.ldq + (size_t)h * HD;
        const bf16* q1 = p.q + (size_t)(t0 + (v1 ? r1 : 0)) * p.ldq + (size_t)h * HD;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            const int d = ks * 16 + 2 * tig;
            qf[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + d) : 0u;
            qf[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + d) : 0u;
            qf[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + d + 8) : 0u;
            qf[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + d + 8) : 0u;
        }
    }

    __shared__ long long quarter_base[QUARTER_TILES * 4];         // as in the decode kernel
    int quarter_tile0 = tile_lo;
    auto fill_quarters = [&](int tile0) {
        quarter_tile0 = tile0;
        const int count = min(QUARTER_TILES, tile_lo + ntiles - tile0);
        for (int e = threadIdx.x; e < count * 4; e += THREADS) {
            const int kpos0 = (tile0 + e / 4) * TILE_KEYS + (e % 4) * 16;
            long long base = -1;
            if (kpos0 <= pos_hi && kpos0 + 15 >= first) {
                const int page = table[kpos0 / p.page_size];
                if (page < 0 || page >= p.num_pages) atomicOr(p.status, EG_STATUS_BAD_PAGE);
                else base = (long long)page * p.page_stride + (long long)kvh * p.head_stride + (long long)(kpos0 % p.page_size) * HD;
            }
            quarter_base[e] = base;
        }
    };
    fill_quarters(tile_lo);
    __syncthreads();

    auto load_tile = [&](int kt, int stage) {
        unsigned char* ks = smem + stage * PL::STAGE_BYTES;
        unsigned char* vs = ks + PL::TILE_BYTES;
        const long long* qb = quarter_base + (kt - quarter_tile0) * 4;
        for (int e = threadIdx.x; e < TILE_KEYS * L::CHUNKS; e += THREADS) {
            const int row = e / L::CHUNKS, chunk = e % L::CHUNKS;
            const int kpos = kt * TILE_KEYS + row;
            const long long base = qb[row >> 4];
            const bool valid = kpos >= first && kpos <= pos_hi && base >= 0;
            const long long off = valid ? base + (long long)(row & 15) * HD + chunk * 8 : 0;
            cp_async_16(ks + L::offset(row, chunk), p.k_cache + off, valid);
            cp_async_16(vs + L::offset(row, chunk), p.v_cache + off, valid);
        }
    };

    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float acc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

#pragma unroll
    for (int s = 0; s < PL::STAGES - 1; ++s) {
        if (s < ntiles) load_tile(tile_lo + s, s);
        cp_async_commit();
    }
    for (int it = 0; it < ntiles; ++it) {
        cp_async_wait<PL::STAGES - 2>();
        __syncthreads();
        {
            const int nxt = it + PL::STAGES - 1;
            if (nxt < ntiles && nxt % QUARTER_TILES == 0) {
                fill_quarters(tile_lo + nxt);
                __syncthreads();
            }
            if (nxt < ntiles) load_tile(tile_lo + nxt, nxt % PL::STAGES);
            cp_async_commit();
        }
        const unsigned char* ks = smem + (it % PL::STAGES) * PL::STAGE_BYTES;
        const unsigned char* vs = ks + PL::TILE_BYTES;
        const int key_base = (tile_lo + it) * TILE_KEYS;
        // this warp's rows see keys up to qp1 (or qp0): skip a key tile that lies wholly behind or before them
        const int warp_hi = pos_lo + min(count - 1, warp * 16 + 15), warp_lo = pos_lo + warp * 16;
        const int warp_first = (p.window > 0 && warp_lo - p.window + 1 > 0) ? warp_lo - p.window + 1 : 0;
        if (warp * 16 >= count || key_base > warp_hi || key_base + TILE_KEYS - 1 < warp_first) continue;

        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {                                    // 16 keys each
                uint32_t b[4];
                const int mi = lane >> 3, r = lane & 7;
                ldmatrix_x4(b, ks + L::offset(kb * 16 + (mi >> 1) * 8 + r, kk * 2 + (mi & 1)));
                mma_bf16_16816(s[2 * kb], qf[kk], b[0], b[1]);
                mma_bf16_16816(s[2 * kb + 1], qf[kk], b[2], b[3]);
            }
        }
        // Scores stay unscaled here; the scale goes into the exponent's multiply-add.  Only a tile that crosses the
        // diagonal, the window's far edge or the end of the portion needs the per-element limits.
        const bool limits = key_base + TILE_KEYS - 1 > warp_lo || warp * 16 + 15 >= count ||
                            (p.window > 0 && key_base <= warp_lo + 15 - p.window);
        if (limits) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int kpos = key_base + j * 8 + 2 * tig + (e & 1);
                    const int qp = e < 2 ? qp0 : qp1;
                    const bool ok = (e < 2 ? v0 : v1) && kpos <= qp && (p.window <= 0 || kpos > qp - p.window);
                    if (!ok) s[j][e] = -INFINITY;
                }
        }
        float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            tmax0 = fmaxf(tmax0, fmaxf(s[j][0], s[j][1]));
            tmax1 = fmaxf(tmax1, fmaxf(s[j][2], s[j][3]));
        }
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 1));
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 2));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 1));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 2));
        // m0, m1: running maxima in scaled (base-2) units
        const float mn0 = fmaxf(m0, tmax0 * scale_log2), mn1 = fmaxf(m1, tmax1 * scale_log2);
        // a row that sees nothing yet keeps m = -inf: use 0 as the reference so that exp(-inf - 0) = 0
        const float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
        const float c0 = exp2_approx(m0 - ref0), c1 = exp2_approx(m1 - ref1);
        m0 = mn0;
        m1 = mn1;
        uint32_t pf[4][4];
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
            const float e00 = exp2_approx(fmaf(s[2 * kb][0], scale_log2, -ref0)), e01 = exp2_approx(fmaf(s[2 * kb][1], scale_log2, -ref0));
            const float e02 = exp2_approx(fmaf(s[2 * kb][2], scale_log2, -ref1)), e03 = exp2_approx(fmaf(s[2 * kb][3], scale_log2, -ref1));
            const float e10 = exp2_approx(fmaf(s[2 * kb + 1][0], scale_log2, -ref0)), e11 = exp2_approx(fmaf(s[2 * kb + 1][1], scale_log2, -ref0));
            const float e12 = exp2_approx(fmaf(s[2 * kb + 1][2], scale_log2, -ref1)), e13 = exp2_approx(fmaf(s[2 * kb + 1][3], scale_log2, -ref1));
            ps0 += e00 + e01 + e10 + e11;
            ps1 += e02 + e03 + e12 + e13;
            pf[kb][0] = pack_bf16(e00, e01);
            pf[kb][1] = pack_bf16(e02, e03);
            pf[kb][2] = pack_bf16(e10, e11);
            pf[kb][3] = pack_bf16(e12, e13);
        }
        l0 = l0 * c0 + ps0;
        l1 = l1 * c1 + ps1;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            acc[i][0] *= c0;
            acc[i][1] *= c0;
            acc[i][2] *= c1;
            acc[i][3] *= c1;
        }
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
#pragma unroll
            for (int nt = 0; nt < HD / 8; nt += 2) {
                uint32_t b[4];
                const int mi = lane >> 3, r = lane & 7;
                ldmatrix_x4_trans(b, vs + L::offset(kb * 16 + (mi & 1) * 8 + r, nt + (mi >> 1)));
                mma_bf16_16816(acc[nt], pf[kb], b[0], b[1]);
                mma_bf16_16816(acc[nt + 1], pf[kb], b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = l0 > 0.f ? 1.0f / l0 : 0.f, i1 = l1 > 0.f ? 1.0f / l1 : 0.f;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        const int d = i * 8 + 2 * tig;
        if (v0) *reinterpret_cast<uint32_t*>(p.out + (size_t)(t0 + r0) * p.ldo + (size_t)h * HD + d) = pack_bf16(acc[i][0] * i0, acc[i][1] * i0);
        if (v1) *reinterpret_cast<uint32_t*>(p.out + (size_t)(t0 + r1) * p.ldo + (size_t)h * HD + d) = pack_bf16(acc[i][2] * i1, acc[i][3] * i1);
    }
}

template <int HD>
int launch_prefill(cudaStream_t stream, const PrefillParams& p, int num_tiles) {
    using PL = PrefillLayout<HD>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, PL::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(2 * num_tiles, p.num_heads);
    attention_prefill_kernel<HD><<<grid, THREADS, PL::SMEM, stream>>>(p);
    return eg_launch_status();
}

}  // namespace

// Head sizes 32, 64, 128, 256 and page sizes that are multiples of 16; anything else
// returns cudaErrorInvalidValue and the caller uses the generic kernel.
// partial_acc / partial_ml: scratch of tokens*heads*splits*(head_dim + 2) floats, and counters: one zeroed int
// per (token, KV head block) (left zero), needed when splits > 1.  seq_context (may be null): per block-table row, the
// number of keys that were in the cache before this step; those may be fetched before the kernel in front has finished.
// token_list (may be null): `tokens` indices of the tokens to work on (scratch and counters are indexed by token index,
// so they cover all tokens of the step either way).
EG_API int eg_attention_paged(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache,
                              const int* block_table, int table_stride, const int* token_seq, const int* positions,
                              const int* seq_context, void* out, int ldo, float* partial_acc, float* partial_ml, int tokens, int num_heads,
                              int num_kv_heads, int head_dim, int page_size, long long page_stride, long long head_stride,
                              int num_pages, int window, float scale, int splits, int* status, const void* prefetch,
                              long long prefetch_bytes, int* counters, int use_pdl, unsigned long long* trace, const int* token_list) {
    if (tokens <= 0) return 0;
    if (page_size % 16 || num_kv_heads <= 0 || num_heads % num_kv_heads || splits < 1 || tokens > 0x7fffffff ||
        splits > MAX_SPLITS || (splits > 1 && (!partial_acc || !partial_ml || !counters || ldo % 4 || (uintptr_t)out % 8)))
        return (int)cudaErrorInvalidValue;
    Params p{(const bf16*)q, ldq, (const bf16*)k_cache, (const bf16*)v_cache, page_stride, head_stride, block_table,
             table_stride, token_seq, positions, seq_context, (bf16*)out, ldo, partial_acc, partial_ml, num_heads, num_kv_heads,
             page_size, num_pages, window, splits, scale, status, prefetch_bytes >= 16 ? prefetch : nullptr, prefetch_bytes,
             counters, use_pdl, trace, token_list};
    switch (head_dim) {
        case 32: return launch<32>(stream, p, tokens);
        case 64: return launch<64>(stream, p, tokens);
        case 128: return launch<128>(stream, p, tokens);
        case 256: return launch<256>(stream, p, tokens);
        default: return (int)cudaErrorInvalidValue;
    }
}

// Prompt portions in tiles of 64 query tokens: tiles[num_tiles][3] = (block table row, first token, count <= 64);
// the tokens of a tile are consecutive positions of one request.  Head sizes 32, 64, 128; pages of a multiple of 16.
EG_API int eg_attention_prefill(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache,
                                const int* block_table, int table_stride, const int* positions, const int* tiles,
                                int num_tiles, void* out, int ldo, int num_heads, int num_kv_heads, int head_dim,
                                int page_size, long long page_stride, long long head_stride, int num_pages, int window,
                                float scale, int* status) {
    if (num_tiles <= 0) return 0;
    if (page_size % 16 || num_kv_heads <= 0 || num_heads % num_kv_heads || num_heads > 65535) return (int)cudaErrorInvalidValue;
    PrefillParams p{(const bf16*)q, ldq, (const bf16*)k_cache, (const bf16*)v_cache, page_stride, head_stride, block_table,
                    table_stride, positions, tiles, (bf16*)out, ldo, num_heads, num_kv_heads, page_size, num_pages, window,
                    scale, status};
    switch (head_dim) {
        case 32: return launch_prefill<32>(stream, p, num_tiles);
        case 64: return launch_prefill<64>(stream, p, num_tiles);
        case 128: return launch_prefill<128>(stream, p, num_tiles);
        default: return (int)cudaErrorInvalidValue;
    }
}
