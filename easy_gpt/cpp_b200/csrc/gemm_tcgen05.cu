// Prefill matrix product on the 5th-generation tensor cores:
//   C[M, N] = A[M, K] * W[N, K]^T (+ bias), bfloat16 in, float32 accumulation in TMEM.
//
// One CTA computes one 128 x 128 tile of C.  Its warps have fixed roles:
//   warp 0   one thread issues the TMA loads (cp.async.bulk.tensor) of the A and W tiles
//            [128 x 64] into a ring of shared-memory stages, 128-byte swizzled
//   warp 1   allocates 128 TMEM columns; one thread issues tcgen05.mma (M 128, N 128, K 16,
//            four per stage) straight from shared-memory descriptors and hands each stage
//            back with tcgen05.commit; the last commit announces the accumulator
//   warps 2-5  read the accumulator (tcgen05.ld, 32 lanes x 32 columns per warp at a time),
//            apply the epilogue and store bfloat16:
//              store    C = acc + bias
//              swiglu   columns interleaved (2i = gate_i, 2i+1 = up_i): out[m, i] = up * silu(gate)
// Stages are handed over with mbarriers (full: TMA bytes landed; empty: the MMAs that read the
// stage are done).  Two CTAs fit an SM (3 stages x 32 KB each, 2 x 128 TMEM columns), so one
// tile's epilogue overlaps the other's main loop.
//
// A second kernel (gemm_tcgen05_wide_kernel) takes the wide products (N % 256 == 0): tiles of 128 x 256
// (MMA N = 256, 87 flop per operand byte instead of 64), four stages, and one persistent CTA per SM that
// walks its tiles with TWO accumulators in TMEM (2 x 256 columns): while the epilogue warps drain one, the
// MMA thread already fills the other (acc_full / acc_empty mbarriers).  Tiles are numbered so that the
// CTAs running at the same time share W tiles through the L2.
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT polls the thread raises the CTA's
// abort flag and EG_STATUS_WAIT_TIMEOUT in the status word; all roles then leave their loops,
// meet at the final barrier, and the TMEM is freed as usual.  Nothing spins for ever.
//
// Takes N % 128 == 0, K % 64 == 0, 16-byte aligned rows; any M (rows beyond M are zero-filled by
// the TMA and not stored).  Anything else: cudaErrorInvalidValue, and the caller uses the library product.
#define EG_NEEDS_TENSOR_MAPS

#include "common.cuh"
#include "mbarrier.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int STAGES = 3;
constexpr int TILE_A_BYTES = BM * BK * 2, TILE_B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = TILE_A_BYTES + TILE_B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;          // + slack to align the ring to 1024 bytes
constexpr int THREADS = 192;                                     // 6 warps
constexpr int TMEM_COLS = 128;
constexpr unsigned WAIT_LIMIT = 1u << 24;

enum { EPI_STORE = 0, EPI_SWIGLU = 2 };


// Bounded wait: false if it gave up (or another role already did).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status) {
    return mbar_wait_bounded(bar, parity, abort_flag, status, WAIT_LIMIT);
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(smem_addr(smem_dst)), "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bfloat16), 128-byte swizzled:
// groups of 8 rows are 1024 bytes apart (stride byte offset); the leading byte offset is unused for this layout.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_address) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_address & 0x3FFFF) >> 4);              // start address, 16-byte units
    d |= (uint64_t)1 << 16;                                      // leading byte offset (ignored), 16-byte units
    d |= (uint64_t)(1024 >> 4) << 32;                            // stride byte offset
    d |= (uint64_t)1 << 46;                                      // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                                      // layout: 128-byte swizzle
    return d;
}

// The same descriptor from its two words: only the low one (start address) changes from tile to tile, and putting
// a descriptor together costs the issuing thread more than the MMA it feeds.
__device__ __forceinline__ uint64_t umma_desc_from(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}
template <bool ACCUMULATE>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "n"(ACCUMULATE ? 1 : 0) : "memory");
}

// silu(g) * u for an epilogue whose result is rounded to bfloat16: the hardware's base-2 exponent and reciprocal
// (relative error about 2^-22 each) instead of expf and a division, which cost the epilogue warps more than the
// main loop costs the tensor core.
__device__ __forceinline__ float swiglu_fast(float g, float u) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * g));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return u * (g * r);
}

// Instruction descriptor for kind::f16: D float32, A and B bfloat16, both K-major, M = 128, N = BN.
__device__ __forceinline__ uint32_t umma_idesc(int n = BN) {
    uint32_t d = 0;
    d |= 1u << 4;                                                // D format: F32
    d |= 1u << 7;                                                // A format: BF16
    d |= 1u << 10;                                               // B format: BF16
    d |= (uint32_t)(n >> 3) << 17;                               // N / 8
    d |= (uint32_t)(BM >> 4) << 24;                              // M / 16
    return d;
}

struct Params {
    bf16* out;
    long long ldo;
    const float* bias;
    int M, N, K;
    int epilogue;
    int* status;
    long long* trace;          // optional (profiling): clock stamps of the first pair's MMA thread, three per step of K
};

__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const Params p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
    const int k_blocks = p.K / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&acc_bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {                                             // TMEM: 128 columns of 128 lanes x 32 bits
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {                                         // ---- TMA producer
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % STAGES;
                if (kb >= STAGES && !mbar_wait(&empty_bar[s], ((kb / STAGES) - 1) & 1, &abort_flag, p.status)) break;
                mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                unsigned char* a = ring + s * STAGE_BYTES;
                tma_load_2d(a, &map_a, &full_bar[s], kb * BK, m0);
                tma_load_2d(a + TILE_A_BYTES, &map_w, &full_bar[s], kb * BK, n0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                         // ---- MMA issuer
            const uint32_t idesc = umma_idesc();
            const uint32_t desc_hi = (uint32_t)(umma_desc(0) >> 32), ring_lo = (uint32_t)umma_desc(smem_addr(ring));
            bool ok = true;
            for (int kb = 0; kb < k_blocks && ok; ++kb) {
                const int s = kb % STAGES;
                // descriptors first, then the wait: 16 elements of K = 32 bytes further inside the swizzled row
                const uint32_t a_lo = ring_lo + (uint32_t)((s * STAGE_BYTES) >> 4), b_lo = a_lo + (TILE_A_BYTES >> 4);
                uint64_t adesc[BK / 16], bdesc[BK / 16];
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    adesc[k] = umma_desc_from(a_lo + 2 * k, desc_hi);
                    bdesc[k] = umma_desc_from(b_lo + 2 * k, desc_hi);
                }
                ok = mbar_wait(&full_bar[s], (kb / STAGES) & 1, &abort_flag, p.status);
                if (!ok) break;
                if (kb) umma<true>(tmem_base, adesc[0], bdesc[0], idesc);
                else umma<false>(tmem_base, adesc[0], bdesc[0], idesc);
#pragma unroll
                for (int k = 1; k < BK / 16; ++k) umma<true>(tmem_base, adesc[k], bdesc[k], idesc);
                // hands the stage back once the MMAs above have read it
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_addr(&empty_bar[s])) : "memory");
            }
            if (ok) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_addr(&acc_bar)) : "memory");
        }
    } else {                                                     // ---- epilogue warps 2..5
        const bool ok = mbar_wait(&acc_bar, 0, &abort_flag, p.status);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        if (ok) {
            const int quad = warp & 3;                           // a warp may touch TMEM lanes 32*(warp % 4) ..
            const int row = m0 + quad * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0;
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                             "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                             "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                               "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                               "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                               "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                             : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (row < p.M) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        v[j] = __uint_as_float(r[j]);
                        if (p.bias) v[j] += p.bias[n0 + c0 + j];
                    }
                    if (p.epilogue == EPI_SWIGLU) {
                        uint32_t packed[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float g0 = v[4 * j], u0 = v[4 * j + 1], g1 = v[4 * j + 2], u1 = v[4 * j + 3];
                            const float y0 = swiglu_fast(g0, u0), y1 = swiglu_fast(g1, u1);
                            __nv_bfloat162 h = __floats2bfloat162_rn(y0, y1);
                            packed[j] = *reinterpret_cast<uint32_t*>(&h);
                        }
                        uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)row * p.ldo + (n0 + c0) / 2);
                        dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                    } else {
                        uint32_t packed[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                            packed[j] = *reinterpret_cast<uint32_t*>(&h);
                        }
                        uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)row * p.ldo + n0 + c0);
#pragma unroll
                        for (int j = 0; j < 4; ++j) dst[j] = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}


// ---------------------------------------------------------------------------
// wide products: 128 x 256 tiles, persistent CTAs, double-buffered accumulator
// ---------------------------------------------------------------------------
namespace wide {
constexpr int WTHREADS = 320;                                    // TMA warp, MMA warp, eight epilogue warps (two per 32 rows)
constexpr int WBN = 256;
constexpr int WSTAGES = 4;
constexpr int W_TILE_B_BYTES = WBN * BK * 2;
constexpr int W_STAGE_BYTES = TILE_A_BYTES + W_TILE_B_BYTES;
constexpr int W_SMEM_BYTES = WSTAGES * W_STAGE_BYTES + 1024;
constexpr int W_TMEM_COLS = 512;
}  // namespace wide

__global__ void __launch_bounds__(wide::WTHREADS)
gemm_tcgen05_wide_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const Params p) {
    using namespace wide;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[WSTAGES], empty_bar[WSTAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = p.K / BK;
    const int m_tiles = (p.M + BM - 1) / BM, n_tiles = p.N / WBN;
    const int total_tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < WSTAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8);                          // one arrival per epilogue warp
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(&tmem_base_slot)), "r"(W_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {                                         // ---- TMA producer
            int g = 0;                                           // k-blocks issued so far, over all tiles
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int n0 = (t / m_tiles) * WBN, m0 = (t % m_tiles) * BM;
                for (int kb = 0; kb < k_blocks; ++kb, ++g) {
                    const int s = g % WSTAGES;
                    if (g >= WSTAGES && !mbar_wait(&empty_bar[s], ((g / WSTAGES) - 1) & 1, &abort_flag, p.status)) { ok = false; break; }
                    mbar_expect_tx(&full_bar[s], W_STAGE_BYTES);
                    unsigned char* a = ring + s * W_STAGE_BYTES;
                    tma_load_2d(a, &map_a, &full_bar[s], kb * BK, m0);
                    // the W box is 128 rows: two boxes make the 256-row tile
                    tma_load_2d(a + TILE_A_BYTES, &map_w, &full_bar[s], kb * BK, n0);
                    tma_load_2d(a + TILE_A_BYTES + TILE_B_BYTES, &map_w, &full_bar[s], kb * BK, n0 + 128);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                         // ---- MMA issuer
            const uint32_t idesc = umma_idesc(WBN);
            const uint32_t desc_hi = (uint32_t)(umma_desc(0) >> 32), ring_lo = (uint32_t)umma_desc(smem_addr(ring));
            int g = 0, local = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
                const int buf = local & 1;
                if (local >= 2) ok = mbar_wait(&acc_empty[buf], ((local >> 1) - 1) & 1, &abort_flag, p.status);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * WBN);
                for (int kb = 0; kb < k_blocks; ++kb, ++g) {
                    const int s = g % WSTAGES;
                    const uint32_t a_lo = ring_lo + (uint32_t)((s * W_STAGE_BYTES) >> 4), b_lo = a_lo + (TILE_A_BYTES >> 4);
                    uint64_t adesc[BK / 16], bdesc[BK / 16];
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        adesc[k] = umma_desc_from(a_lo + 2 * k, desc_hi);
                        bdesc[k] = umma_desc_from(b_lo + 2 * k, desc_hi);
                    }
                    ok = mbar_wait(&full_bar[s], (g / WSTAGES) & 1, &abort_flag, p.status);
                    if (!ok) break;
                    if (kb) umma<true>(tmem_acc, adesc[0], bdesc[0], idesc);
                    else umma<false>(tmem_acc, adesc[0], bdesc[0], idesc);
#pragma unroll
                    for (int k = 1; k < BK / 16; ++k) umma<true>(tmem_acc, adesc[k], bdesc[k], idesc);
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_addr(&empty_bar[s])) : "memory");
                }
                if (ok) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_addr(&acc_full[buf])) : "memory");
            }
        }
    } else {                                                     // ---- epilogue warps 2..5
        const int quad = warp & 3;                               // a warp may touch TMEM lanes 32 * (warp % 4) ..
        const int col_lo = ((warp - 2) >> 2) * (WBN / 2);        // the two warps of a quad share its rows' columns
        int local = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
            const int buf = local & 1;
            const int n0 = (t / m_tiles) * WBN, m0 = (t % m_tiles) * BM;
            ok = mbar_wait(&acc_full[buf], (local >> 1) & 1, &abort_flag, p.status);
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if (!ok) break;
            const int row = m0 + quad * 32 + lane;
#pragma unroll 1
            for (int c0 = col_lo; c0 < col_lo + WBN / 2; c0 += 32) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * WBN + c0);
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                             "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                             "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                               "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                               "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                               "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                             : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (row < p.M) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        v[j] = __uint_as_float(r[j]);
                        if (p.bias) v[j] += p.bias[n0 + c0 + j];
                    }
                    if (p.epilogue == EPI_SWIGLU) {
                        uint32_t packed[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float g0 = v[4 * j], u0 = v[4 * j + 1], g1 = v[4 * j + 2], u1 = v[4 * j + 3];
                            const float y0 = swiglu_fast(g0, u0), y1 = swiglu_fast(g1, u1);
                            __nv_bfloat162 h = __floats2bfloat162_rn(y0, y1);
                            packed[j] = *reinterpret_cast<uint32_t*>(&h);
                        }
                        uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)row * p.ldo + (n0 + c0) / 2);
                        dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                    } else {
                        uint32_t packed[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                            packed[j] = *reinterpret_cast<uint32_t*>(&h);
                        }
                        uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)row * p.ldo + n0 + c0);
#pragma unroll
                        for (int j = 0; j < 4; ++j) dst[j] = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                    }
                }
            }
            // this warp has read its part of the accumulator: the MMA thread may overwrite it
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(&acc_empty[buf])) : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(W_TMEM_COLS) : "memory");
    }
}


// ---------------------------------------------------------------------------
// wide products on CTA pairs: 256 x 256 tiles, each CTA of a pair loads half of either operand
// ---------------------------------------------------------------------------
// Two CTAs of a cluster (two neighbouring SMs) compute one 256 x 256 tile: CTA r holds rows r * 128 .. of the A tile and
// rows r * 128 .. of the W tile in its shared memory, the leader (rank 0) issues tcgen05.mma.cta_group::2 (M 256, N 256),
// which reads both CTAs' shared memory, and each CTA's TMEM receives its 128 rows of the accumulator.  A 64-deep step
// of K costs a CTA 32 KB of operands for 4.2 MFLOP, where the single-CTA kernel above moves 48 KB.
//   warp 0   (both CTAs) TMA loads of the CTA's halves; the bytes are counted on the leader's full barrier
//   warp 1   allocates TMEM (both CTAs, cta_group::2); in the leader one thread issues the MMAs and commits to the
//            empty and accumulator barriers of both CTAs (multicast commit)
//   warps 2-9 (both CTAs) read the CTA's accumulator rows, apply the epilogue, and arrive on the leader's
//            accumulator-empty barrier (a remote arrive for the second CTA)
// Persistent: a pair walks the tiles pair, pair + pairs, ...; two accumulators of 256 columns alternate.
namespace pairk {
constexpr int PTHREADS = 320;
constexpr int PBK = 128;                                         // K per stage: two 64-wide boxes per operand, eight MMAs per barrier round
constexpr int EPI_BOX_BYTES = 32 * 128;                           // an epilogue warp's [32 rows x 64 bfloat16] box
// PBN: columns of the pair's tile, 256 or 128 (narrow products: more tiles, so that most pairs get one)
template <int PBN>
struct PairCfg {
    static constexpr int STAGES = PBN == 256 ? 3 : 4;
    static constexpr int A_SUB_BYTES = 128 * BK * 2;              // a [128 x 64] box of A
    static constexpr int W_SUB_BYTES = (PBN / 2) * BK * 2;        // a [PBN/2 x 64] box of W: this CTA's half of the tile's columns
    static constexpr int STAGE_BYTES = 2 * A_SUB_BYTES + 2 * W_SUB_BYTES;     // A low K, A high K, W low K, W high K
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 8 * EPI_BOX_BYTES + 1024;
    static constexpr int TMEM_COLS = 2 * PBN;
};
constexpr uint32_t PEER_BIT_MASK = 0xFEFFFFFFu;                  // clears the bit that tells the pair's CTAs apart in a shared::cluster address

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// The CTA's own load, counted on the barrier at the same place in the pair's leader.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(smem_addr(smem_dst)), "l"(map), "r"(smem_addr(bar) & PEER_BIT_MASK), "r"(x), "r"(y) : "memory");
}
template <bool ACCUMULATE>
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "n"(ACCUMULATE ? 1 : 0) : "memory");
}
// arrives on the barrier at this place in both CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
                 ::"r"(smem_addr(bar)), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void arrive_at_leader(uint64_t* bar) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(smem_addr(bar)), "r"(0));
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(remote) : "memory");
}

template <int PBN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PTHREADS)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                         const __grid_constant__ CUtensorMap map_out, const Params p) {
    using C = PairCfg<PBN>;
    constexpr int PSTAGES = C::STAGES, P_STAGE_BYTES = C::STAGE_BYTES, P_TMEM_COLS = C::TMEM_COLS;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[PSTAGES], empty_bar[PSTAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)cluster_rank();
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int k_blocks = (p.K + PBK - 1) / PBK;                  // a last half block reads zeros past K (the TMA fills them)
    const int m_tiles = (p.M + 2 * BM - 1) / (2 * BM), n_tiles = p.N / PBN;
    const int total_tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PSTAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 16);                         // one arrival per epilogue warp of either CTA
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(&tmem_base_slot)), "r"(P_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    cluster_sync();                                              // both CTAs' barriers exist before anyone arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {                                         // ---- TMA producer, in both CTAs
            int g = 0;
            bool ok = true;
            for (int t = pair; t < total_tiles && ok; t += pairs) {
                const int n0 = (t / m_tiles) * PBN + rank * (PBN / 2), m0 = (t % m_tiles) * 2 * BM + rank * BM;
                for (int kb = 0; kb < k_blocks; ++kb, ++g) {
                    const int s = g % PSTAGES;
                    if (g >= PSTAGES && !mbar_wait(&empty_bar[s], ((g / PSTAGES) - 1) & 1, &abort_flag, p.status)) { ok = false; break; }
                    if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * P_STAGE_BYTES);
                    unsigned char* a = ring + s * P_STAGE_BYTES;
                    tma_load_2d_pair(a, &map_a, &full_bar[s], kb * PBK, m0);
                    tma_load_2d_pair(a + C::A_SUB_BYTES, &map_a, &full_bar[s], kb * PBK + BK, m0);
                    tma_load_2d_pair(a + 2 * C::A_SUB_BYTES, &map_w, &full_bar[s], kb * PBK, n0);
                    tma_load_2d_pair(a + 2 * C::A_SUB_BYTES + C::W_SUB_BYTES, &map_w, &full_bar[s], kb * PBK + BK, n0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {                            // ---- MMA issuer, in the leader
            uint32_t idesc = 0;                                  // D float32, A and B bfloat16 K-major, M 256, N = PBN
            idesc |= 1u << 4;
            idesc |= 1u << 7;
            idesc |= 1u << 10;
            idesc |= (uint32_t)(PBN >> 3) << 17;
            idesc |= (uint32_t)((2 * BM) >> 4) << 24;
            const uint32_t desc_hi = (uint32_t)(umma_desc(0) >> 32), ring_lo = (uint32_t)umma_desc(smem_addr(ring));
            int g = 0, local = 0;
            bool ok = true;
            for (int t = pair; t < total_tiles && ok; t += pairs, ++local) {
                const int buf = local & 1;
                if (local >= 2) ok = mbar_wait(&acc_empty[buf], ((local >> 1) - 1) & 1, &abort_flag, p.status);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * PBN);
                for (int kb = 0; kb < k_blocks; ++kb, ++g) {
                    const int s = g % PSTAGES;
                    const uint32_t a_lo = ring_lo + (uint32_t)((s * P_STAGE_BYTES) >> 4), b_lo = a_lo + (2 * C::A_SUB_BYTES >> 4);
                    uint64_t adesc[PBK / 16], bdesc[PBK / 16];
#pragma unroll
                    for (int k = 0; k < PBK / 16; ++k) {             // 16 of K = 32 bytes in the row; 64 of K = the next box
                        adesc[k] = umma_desc_from(a_lo + (k / 4) * (C::A_SUB_BYTES >> 4) + 2 * (k % 4), desc_hi);
                        bdesc[k] = umma_desc_from(b_lo + (k / 4) * (C::W_SUB_BYTES >> 4) + 2 * (k % 4), desc_hi);
                    }
                    const bool tr = p.trace && blockIdx.x == 0 && g < 64;
                    if (tr) p.trace[g * 3] = clock64();
                    ok = mbar_wait(&full_bar[s], (g / PSTAGES) & 1, &abort_flag, p.status);
                    if (!ok) break;
                    if (tr) p.trace[g * 3 + 1] = clock64();
                    if (kb) umma_pair<true>(tmem_acc, adesc[0], bdesc[0], idesc);
                    else umma_pair<false>(tmem_acc, adesc[0], bdesc[0], idesc);
#pragma unroll
                    for (int k = 1; k < PBK / 16; ++k) umma_pair<true>(tmem_acc, adesc[k], bdesc[k], idesc);
                    commit_pair(&empty_bar[s]);
                    if (tr) p.trace[g * 3 + 2] = clock64();
                }
                if (ok) commit_pair(&acc_full[buf]);
            }
        }
    } else {                                                     // ---- epilogue warps 2..9, in both CTAs
        // A warp takes 32 rows x PBN / 2 accumulator columns.  Its results go through a [32 x 64] bfloat16 box in shared
        // memory (128-byte rows, swizzled like the TMA's tiles: a lane writes its own row without bank conflicts)
        // and leave with a TMA store: rows of a tile are 19 KB apart in the output, and 32 scattered 16-byte stores
        // per instruction kept the load/store path busy enough to hold up the MMA thread's barrier traffic.
        const int quad = warp & 3;                               // a warp may touch TMEM lanes 32 * (warp % 4) ..
        const int half = (warp - 2) >> 2;                        // the two warps of a quad share its rows' columns
        unsigned char* box = ring + PSTAGES * P_STAGE_BYTES + (warp - 2) * EPI_BOX_BYTES;
        const uint32_t box_row = smem_addr(box) + (uint32_t)lane * 128u;
        int local = 0;
        bool ok = true;
        for (int t = pair; t < total_tiles && ok; t += pairs, ++local) {
            const int buf = local & 1;
            const int n0 = (t / m_tiles) * PBN, m0 = (t % m_tiles) * 2 * BM + rank * BM;
            ok = mbar_wait(&acc_full[buf], (local >> 1) & 1, &abort_flag, p.status);
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if (!ok) break;
            const int row0 = m0 + quad * 32;
            // The warp has PBN / 2 accumulator columns.  Store: a box per 64 of them.  SwiGLU (PBN 256 only): its 128
            // columns give one box of 64 outputs.
            const int boxes = p.epilogue == EPI_SWIGLU ? 1 : PBN / 128;
#pragma unroll 1
            for (int bx = 0; bx < boxes; ++bx) {
                const int cols_per_box = p.epilogue == EPI_SWIGLU ? 128 : 64;
                const int c_first = half * (PBN / 2) + bx * 64;  // first accumulator column of this box
                // the box in shared memory must have left with the store before it is written again
                if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
                __syncwarp();
#pragma unroll 1
                for (int c0 = 0; c0 < cols_per_box; c0 += 32) {
                    uint32_t r[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * PBN + c_first + c0);
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                                 : "r"(taddr));
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        v[j] = __uint_as_float(r[j]);
                        if (p.bias) v[j] += p.bias[n0 + c_first + c0 + j];
                    }
                    if (p.epilogue == EPI_SWIGLU) {
                        // 32 accumulator columns = 16 outputs = two 16-byte pieces of the box row
                        uint32_t packed[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float y0 = swiglu_fast(v[4 * j], v[4 * j + 1]), y1 = swiglu_fast(v[4 * j + 2], v[4 * j + 3]);
                            __nv_bfloat162 h = __floats2bfloat162_rn(y0, y1);
                            packed[j] = *reinterpret_cast<uint32_t*>(&h);
                        }
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            const uint32_t dst = box_row + (uint32_t)((((c0 / 32) * 2 + q) ^ (lane & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(dst), "r"(packed[4 * q]), "r"(packed[4 * q + 1]),
                                         "r"(packed[4 * q + 2]), "r"(packed[4 * q + 3]) : "memory");
                        }
                    } else {
                        uint32_t packed[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                            packed[j] = *reinterpret_cast<uint32_t*>(&h);
                        }
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint32_t dst = box_row + (uint32_t)((((c0 / 32) * 4 + q) ^ (lane & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(dst), "r"(packed[4 * q]), "r"(packed[4 * q + 1]),
                                         "r"(packed[4 * q + 2]), "r"(packed[4 * q + 3]) : "memory");
                        }
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    const int x = p.epilogue == EPI_SWIGLU ? (n0 + c_first) / 2 : n0 + c_first;
                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];\n"
                                 ::"l"(&map_out), "r"(smem_addr(box)), "r"(x), "r"(row0) : "memory");
                    asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
                }
            }
            // this warp has read its part of the accumulator: the leader's MMA thread may overwrite it
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) arrive_at_leader(&acc_empty[buf]);
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");      // the last boxes have been written
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    cluster_sync();                                              // nobody leaves while its partner may still read its shared memory
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(P_TMEM_COLS) : "memory");
    }
}
}  // namespace pairk

// ---------------------------------------------------------------------------
// few rows (17 .. 128 tokens: the larger decode batches, short prompt portions): the weights stream once
// ---------------------------------------------------------------------------
// The tokens are the MMA's 128 rows (rows past M come zero-filled from the TMA and are not stored), a CTA takes BN
// output columns (32, 64 or 128: narrow tiles, so that most SMs get one) and one of gridDim.y slices of K.  With
// several slices every CTA writes its float32 partial tile to scratch memory and draws a ticket; the CTA that draws
// the last one of its column tile adds the slices in order and applies the epilogue.  Nobody waits for another CTA.
// The kernel is launched with programmatic dependent launch: W tiles are requested before the kernel in front has
// finished (weights do not depend on it), A tiles after.
namespace few {
constexpr int FSTAGES = 4;
enum { EPI_F32 = 1 };
template <int FBN>
struct Cfg {
    static constexpr int W_BYTES = FBN * BK * 2;
    static constexpr int STAGE = TILE_A_BYTES + W_BYTES;
    static constexpr int SMEM = FSTAGES * STAGE + 1024;
    static constexpr int TMEM = FBN < 32 ? 32 : FBN;
};
struct FewParams {
    void* out;                 // bfloat16 [M, N] (store), [M, N/2] (swiglu) or float32 [M, N]
    long long ldo;
    const float* bias;
    int M, N, K;
    int epilogue;
    float* partial;            // [column tiles][slices][128][BN] float32, when gridDim.y > 1
    int* tickets;              // [column tiles], zero before and after
    int* status;
};

__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void grid_dependents_launch() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }

// 32 columns of one token row: bias, then store / SwiGLU / float32
__device__ __forceinline__ void few_epilogue(const FewParams& p, int row, int col0, float (&v)[32]) {
    if (p.bias) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] += p.bias[col0 + j];
    }
    if (p.epilogue == EPI_SWIGLU) {
        uint32_t packed[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float g0 = v[4 * j], u0 = v[4 * j + 1], g1 = v[4 * j + 2], u1 = v[4 * j + 3];
            const float y0 = swiglu_fast(g0, u0), y1 = swiglu_fast(g1, u1);
            __nv_bfloat162 h = __floats2bfloat162_rn(y0, y1);
            packed[j] = *reinterpret_cast<uint32_t*>(&h);
        }
        uint4* dst = reinterpret_cast<uint4*>((bf16*)p.out + (size_t)row * p.ldo + col0 / 2);
        dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    } else if (p.epilogue == EPI_F32) {
        float4* dst = reinterpret_cast<float4*>((float*)p.out + (size_t)row * p.ldo + col0);
#pragma unroll
        for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
            packed[j] = *reinterpret_cast<uint32_t*>(&h);
        }
        uint4* dst = reinterpret_cast<uint4*>((bf16*)p.out + (size_t)row * p.ldo + col0);
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[j] = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
    }
}

template <int FBN>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_few_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const FewParams p) {
    using C = Cfg<FBN>;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[FSTAGES], empty_bar[FSTAGES], acc_bar, parts_written, ticket_drawn;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag, reduces_here;

    grid_dependents_launch();
    unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * FBN;
    const int slices = gridDim.y, slice = blockIdx.y;
    const int all_blocks = p.K / BK;
    const int kb0 = (int)((long long)all_blocks * slice / slices), kb1 = (int)((long long)all_blocks * (slice + 1) / slices);
    const int k_blocks = kb1 - kb0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < FSTAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&acc_bar, 1);
        mbar_init(&parts_written, 4);
        mbar_init(&ticket_drawn, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(&tmem_base_slot)), "r"(C::TMEM) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {                                         // ---- TMA producer
            // the W tiles of the first stages go out before the kernel in front is known to be done, the A tiles after
            const int early = k_blocks < FSTAGES ? k_blocks : FSTAGES;
            for (int kb = 0; kb < early; ++kb) {
                mbar_expect_tx(&full_bar[kb], C::STAGE);
                tma_load_2d(ring + kb * C::STAGE + TILE_A_BYTES, &map_w, &full_bar[kb], (kb0 + kb) * BK, n0);
            }
            grid_dependency_wait();
            for (int kb = 0; kb < early; ++kb) tma_load_2d(ring + kb * C::STAGE, &map_a, &full_bar[kb], (kb0 + kb) * BK, 0);
            for (int kb = early; kb < k_blocks; ++kb) {
                const int s = kb % FSTAGES;
                if (!mbar_wait(&empty_bar[s], ((kb / FSTAGES) - 1) & 1, &abort_flag, p.status)) break;
                mbar_expect_tx(&full_bar[s], C::STAGE);
                tma_load_2d(ring + s * C::STAGE + TILE_A_BYTES, &map_w, &full_bar[s], (kb0 + kb) * BK, n0);
                tma_load_2d(ring + s * C::STAGE, &map_a, &full_bar[s], (kb0 + kb) * BK, 0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                         // ---- MMA issuer
            const uint32_t idesc = umma_idesc(FBN);
            const uint32_t desc_hi = (uint32_t)(umma_desc(0) >> 32), ring_lo = (uint32_t)umma_desc(smem_addr(ring));
            bool ok = true;
            for (int kb = 0; kb < k_blocks && ok; ++kb) {
                const int s = kb % FSTAGES;
                const uint32_t a_lo = ring_lo + (uint32_t)((s * C::STAGE) >> 4), b_lo = a_lo + (TILE_A_BYTES >> 4);
                uint64_t adesc[BK / 16], bdesc[BK / 16];
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    adesc[k] = umma_desc_from(a_lo + 2 * k, desc_hi);
                    bdesc[k] = umma_desc_from(b_lo + 2 * k, desc_hi);
                }
                ok = mbar_wait(&full_bar[s], (kb / FSTAGES) & 1, &abort_flag, p.status);
                if (!ok) break;
                if (kb) umma<true>(tmem_base, adesc[0], bdesc[0], idesc);
                else umma<false>(tmem_base, adesc[0], bdesc[0], idesc);
#pragma unroll
                for (int k = 1; k < BK / 16; ++k) umma<true>(tmem_base, adesc[k], bdesc[k], idesc);
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_addr(&empty_bar[s])) : "memory");
            }
            if (ok) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_addr(&acc_bar)) : "memory");
        }
    } else {                                                     // ---- epilogue warps 2..5: one token row per thread
        bool ok = __all_sync(0xffffffffu, mbar_wait(&acc_bar, 0, &abort_flag, p.status));
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const int quad = warp & 3;                               // a warp may touch TMEM lanes 32 * (warp % 4) ..
        const int row = quad * 32 + lane;
        const bool valid = row < p.M;
        float* my_partial = p.partial + (((size_t)blockIdx.x * slices + slice) * BM + row) * FBN;
        if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < FBN; c0 += 32) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0;
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                             "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                             "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                               "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                               "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                               "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                             : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (!valid) continue;
                if (slices == 1) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    few_epilogue(p, row, n0 + c0, v);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) *reinterpret_cast<uint4*>(my_partial + c0 + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
                }
            }
        }
        if (slices > 1) {
            __threadfence();
            __syncwarp();
            if (lane == 0) mbar_arrive(&parts_written);
            if (warp == 2) {
                const bool all_in = __all_sync(0xffffffffu, mbar_wait(&parts_written, 0, &abort_flag, p.status)) && ok;
                if (lane == 0) {
                    int last = 0;
                    if (all_in) {
                        last = atomicAdd(p.tickets + blockIdx.x, 1) == slices - 1;
                        if (last) p.tickets[blockIdx.x] = 0;     // every slice has drawn: ready for the next launch
                    }
                    reduces_here = last;
                    mbar_arrive(&ticket_drawn);
                }
            }
            ok = __all_sync(0xffffffffu, mbar_wait(&ticket_drawn, 0, &abort_flag, p.status));
            if (ok && reduces_here && valid) {
                __threadfence();
                const float* base = p.partial + ((size_t)blockIdx.x * slices * BM + row) * FBN;
#pragma unroll 1
                for (int c0 = 0; c0 < FBN; c0 += 32) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0.f;
                    for (int i = 0; i < slices; ++i) {           // in order: the sum does not depend on who came last
                        const float4* src = reinterpret_cast<const float4*>(base + (size_t)i * BM * FBN + c0);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float4 t = __ldcg(src + j);
                            v[4 * j] += t.x;
                            v[4 * j + 1] += t.y;
                            v[4 * j + 2] += t.z;
                            v[4 * j + 3] += t.w;
                        }
                    }
                    few_epilogue(p, row, n0 + c0, v);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(C::TMEM) : "memory");
    }
}
}  // namespace few

// A [rows, cols] bfloat16 matrix with row stride ld (elements), cut into boxes of [box_rows x 64], 128-byte swizzled.
int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    const eg_encode_tiled_fn encode = eg_encode_tiled();
    if (!encode) return (int)cudaErrorNotSupported;
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

}  // namespace

// epilogue: 0 store (out [M, N]), 2 swiglu on interleaved columns (out [M, N/2]).
EG_API int eg_gemm_tcgen05(cudaStream_t stream, int epilogue, const void* A, long long lda, const void* W, long long ldw,
                           const float* bias, void* out, long long ldo, int M, int N, int K, int* status) {
    if (M <= 0 || N <= 0) return 0;
    if (N % BN || K % BK || K <= 0 || lda % 8 || ldw % 8 || ldo % 8 || (uintptr_t)A % 16 || (uintptr_t)W % 16 ||
        (uintptr_t)out % 16 || (epilogue != EPI_STORE && epilogue != EPI_SWIGLU) || !status)
        return (int)cudaErrorInvalidValue;
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 148;
    }
    CUtensorMap map_a, map_w;
    if (make_map(&map_a, A, M, K, lda, BM) || make_map(&map_w, W, N, K, ldw, BN)) return (int)cudaErrorInvalidValue;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    Params p{(bf16*)out, ldo, bias, M, N, K, epilogue, status};
    const int m_tiles = (M + BM - 1) / BM;
    if (N % wide::WBN == 0 && m_tiles * (N / wide::WBN) >= sm_count) {
        // wide product: persistent CTAs over 128 x 256 tiles
        static bool wide_configured = false;
        if (!wide_configured) {
            cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, wide::W_SMEM_BYTES);
            if (e != cudaSuccess) return (int)e;
            wide_configured = true;
        }
        const int tiles = m_tiles * (N / wide::WBN);
        gemm_tcgen05_wide_kernel<<<tiles < sm_count ? tiles : sm_count, wide::WTHREADS, wide::W_SMEM_BYTES, stream>>>(map_a, map_w, p);
        return eg_launch_status();
    }
    dim3 grid(N / BN, (M + BM - 1) / BM);
    gemm_tcgen05_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(map_a, map_w, p);
    return eg_launch_status();
}

namespace {
template <int FBN>
int launch_few(cudaStream_t stream, const CUtensorMap& map_a, const CUtensorMap& map_w, const few::FewParams& p, int slices, int use_pdl) {
    using C = few::Cfg<FBN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(few::gemm_tcgen05_few_kernel<FBN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.N / FBN, slices);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = C::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, few::gemm_tcgen05_few_kernel<FBN>, map_a, map_w, p);
}
}  // namespace

// Products of at most 128 rows.  epilogue: 0 store bfloat16 [M, N], 1 float32 [M, N], 2 swiglu on interleaved columns
// (bfloat16 [M, N/2]).  tile_n: 32, 64 or 128 columns per CTA (N % tile_n == 0); slices of K (<= K / 64); with more
// than one slice, partial takes (N / tile_n) * slices * 128 * tile_n floats and tickets N / tile_n zeroed ints (left zero).
EG_API int eg_gemm_tcgen05_few(cudaStream_t stream, int epilogue, int use_pdl, const void* A, long long lda, const void* W, long long ldw,
                               const float* bias, void* out, long long ldo, int M, int N, int K, int tile_n, int slices,
                               float* partial, int* tickets, int* status) {
    if (M <= 0 || N <= 0) return 0;
    if (M > BM || (tile_n != 32 && tile_n != 64 && tile_n != 128) || N % tile_n || K % BK || K <= 0 || slices < 1 || slices > K / BK ||
        lda % 8 || ldw % 8 || (uintptr_t)A % 16 || (uintptr_t)W % 16 || (uintptr_t)out % 16 || !status ||
        (epilogue != EPI_STORE && epilogue != EPI_SWIGLU && epilogue != few::EPI_F32) || (slices > 1 && (!partial || !tickets)) ||
        (epilogue == few::EPI_F32 ? ldo % 4 : ldo % 8))
        return (int)cudaErrorInvalidValue;
    CUtensorMap map_a, map_w;
    if (make_map(&map_a, A, M, K, lda, BM) || make_map(&map_w, W, N, K, ldw, tile_n)) return (int)cudaErrorInvalidValue;
    few::FewParams p{out, ldo, bias, M, N, K, epilogue, partial, tickets, status};
    switch (tile_n) {
        case 32: return launch_few<32>(stream, map_a, map_w, p, slices, use_pdl);
        case 64: return launch_few<64>(stream, map_a, map_w, p, slices, use_pdl);
        default: return launch_few<128>(stream, map_a, map_w, p, slices, use_pdl);
    }
}

namespace {
template <int PBN>
int launch_pair(cudaStream_t stream, const CUtensorMap& map_a, const CUtensorMap& map_w, const CUtensorMap& map_out, const Params& p, int sm_count) {
    using C = pairk::PairCfg<PBN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(pairk::gemm_tcgen05_pair_kernel<PBN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * (p.N / PBN);
    const int pairs = tiles < sm_count / 2 ? tiles : sm_count / 2;
    pairk::gemm_tcgen05_pair_kernel<PBN><<<2 * pairs, pairk::PTHREADS, C::SMEM_BYTES, stream>>>(map_a, map_w, map_out, p);
    return eg_launch_status();
}
}  // namespace

// The same product on CTA pairs (tcgen05.mma.cta_group::2): tiles of 256 x tile_n, tile_n 256 or 128 (N % tile_n == 0),
// K % 64 == 0; epilogues as eg_gemm_tcgen05 (SwiGLU with tile_n 256 only).
EG_API int eg_gemm_tcgen05_pair(cudaStream_t stream, int epilogue, const void* A, long long lda, const void* W, long long ldw,
                                const float* bias, void* out, long long ldo, int M, int N, int K, int tile_n, int* status,
                                long long* trace) {
    if (M <= 0 || N <= 0) return 0;
    if ((tile_n != 128 && tile_n != 256) || N % tile_n || K % BK || K <= 0 || lda % 8 || ldw % 8 || ldo % 8 || (uintptr_t)A % 16 ||
        (uintptr_t)W % 16 || (uintptr_t)out % 16 || (epilogue != EPI_STORE && epilogue != EPI_SWIGLU) ||
        (epilogue == EPI_SWIGLU && tile_n != 256) || !status)
        return (int)cudaErrorInvalidValue;
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 148;
    }
    CUtensorMap map_a, map_w, map_out;
    if (make_map(&map_a, A, M, K, lda, BM) || make_map(&map_w, W, N, K, ldw, tile_n / 2) ||
        make_map(&map_out, out, M, epilogue == EPI_SWIGLU ? N / 2 : N, ldo, 32))
        return (int)cudaErrorInvalidValue;
    Params p{(bf16*)out, ldo, bias, M, N, K, epilogue, status, trace};
    return tile_n == 256 ? launch_pair<256>(stream, map_a, map_w, map_out, p, sm_count) : launch_pair<128>(stream, map_a, map_w, map_out, p, sm_count);
}
