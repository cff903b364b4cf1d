// Matrix products for decode steps (1..64 tokens): y[m, n] = sum_k x[m, k] W[n, k].
//
// With so few tokens the product is a stream of the weights from HBM, so the
// kernel is built around that stream.  The roles of the MMA are swapped: 16 weight
// rows are the M side of mma.m16n8k16 and 8 tokens are its N side, so no tensor
// core work is wasted on padding tokens up to a tile.  Every thread fetches its
// piece of the weight fragment with one 32-byte load straight from global memory
// (16 consecutive k of one row, so that a warp's load covers whole 128-byte lines;
// the k order inside a 64-wide chunk is permuted the same way for both operands,
// which a sum does not notice), several chunks ahead, and nothing of W passes
// through shared memory.  A CTA's warps are arranged as RB row blocks x KS slices
// of K, and K may be cut further across gridDim.y CTAs.  Slices are summed in a
// fixed order: inside a CTA through shared memory, across CTAs through scratch
// memory by the CTA that arrives last (a ticket counter; nobody waits for anybody).
//
// Prologues (what x is):
//   plain      x is a bfloat16 matrix in global memory
//   norm       x = gain * rmsnorm(residual_in + delta), computed by every CTA in one
//              pass: v = residual_in + delta, the row's sum of squares in float32
//              (src/models/norm.cpp:46-60) and bfloat16(gain * v) into shared memory;
//              the row's factor 1/sqrt(mean + eps) multiplies the product's result
//              instead of every x (the product is linear in x).  CTA 0 also writes v to
//              residual_out (another buffer, so that no CTA reads what CTA 0 has
//              already updated).  Meant for a few tokens: every CTA repeats it.  The input
//              rows come into shared memory by bulk copies (one trip to the L2).
//   prenormed  the kernel in front (epilogue resid_norm) has already added its result to the
//              residual and left bfloat16(gain * v) and, per CTA of its own, the partial sums
//              of squares of v: the rows come in by bulk copy and every CTA only adds up the
//              partial sums, in their order, for the rows' factors.
// Epilogues (what happens to y):
//   store      + bias -> bfloat16 [M, N]
//   f32        + bias -> float32 [M, N] (logits)
//   swiglu     rows of W interleaved (2i = gate_i, 2i+1 = up_i): up * silu(gate) -> bfloat16 [M, N/2]
//   qkv_rope   one CTA per head (RB*16 == head_dim): + bias, q and k rotated
//              (src/ops.cpp:404-421), q -> bfloat16 [M, NH*HD], k and v -> paged cache
//   resid_norm the result (rounded to bfloat16, as a stored delta would be) is added to the
//              float32 residual in place, v = residual + y; bfloat16(gain * v) goes to xn_out
//              and this CTA's sum of v^2 per token to ss_out[CTA][tokens]: the input of the
//              next kernel's prenormed prologue, so that the add and the norm that follow a
//              product are computed once, by the product's own CTAs, and not by every CTA
//              of the next one.
//
// Every kernel starts streaming its weights before it waits for the kernel in front
// of it (programmatic dependent launch), so the pipeline of small kernels overlaps.
// A kernel can also be told which weights a later kernel will stream; when its own
// stream has been issued it asks the L2 (126 MB) to fetch them.
#include <cstdlib>

#include "mma_utils.cuh"

namespace {

constexpr int MAX_THREADS = 512;
constexpr int UNROLL = 4;            // 64-wide k chunks in flight per warp (256 bytes per thread)
constexpr int CHUNK = 64;

enum { EPI_STORE = 0, EPI_F32 = 1, EPI_SWIGLU = 2, EPI_QKV_ROPE = 3, EPI_RESID_NORM = 4 };

struct Params {
    const bf16* W;
    long long ldw;
    const float* bias;
    int M, N, K;
    const bf16* x;
    long long ldx;
    const float* resid_in;
    float* resid_out;
    const bf16* delta;
    const float* gain;
    float eps;
    bf16* out;
    long long ldo;
    float* out_f32;
    int num_heads, num_kv_heads, head_dim;
    const int* positions;
    const int* slot_map;
    bf16* k_cache;
    bf16* v_cache;
    const float* inv_freq;
    int page_size;
    long long page_stride, head_stride, pool_slots;
    int* status;
    int RB, KS;
    int use_pdl;
    int stage_norm;              // the norm prologue's input comes through one bulk copy into shared memory
    int norm_mode;               // 1: add + norm here; 2: prenormed rows (delta = xn) and partial sums (ss_in)
    const float* ss_in;          // [ss_parts][padded tokens] partial sums of squares, prenormed prologue
    int ss_parts;
    float* resid_inout;          // resid_norm epilogue: the residual, updated in place
    const float* gain_out;       //   the following norm's gain
    bf16* xn_out;                //   bfloat16(gain_out * v) [M, N]
    float* ss_out;               //   [gridDim.x][padded tokens]
    const void* prefetch;        // weights of a kernel that runs soon: pulled into L2 meanwhile
    long long prefetch_bytes;
    float* scratch;              // [gridDim.y][gridDim.x][RB*16][tokens] partial sums when K is cut across CTAs
    int* counters;               // [gridDim.x] tickets, zero before and after every launch
    unsigned long long* trace;   // optional: [2] earliest start / latest end of this launch's CTAs (%globaltimer, ns)
    int parts_offset;            // where in shared memory the cluster's parts arrive (bytes)
    int cluster_reduce;          // the gridDim.y CTAs of a row group are one cluster and sum their parts through the first one's shared memory
};

struct W32 {                      // 16 consecutive bfloat16 of one weight row
    uint32_t r[8];
};

__device__ __forceinline__ W32 ldg256(const void* p) {
    W32 v;
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(v.r[0]), "=r"(v.r[1]), "=r"(v.r[2]), "=r"(v.r[3]), "=r"(v.r[4]), "=r"(v.r[5]), "=r"(v.r[6]), "=r"(v.r[7])
                 : "l"(p));
    return v;
}

// Asks the L2 to fetch [ptr, ptr + bytes) (16-byte aligned, a multiple of 16 bytes); nothing waits for it.
__device__ __forceinline__ void prefetch_l2(const void* ptr, unsigned bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(ptr), "r"(bytes) : "memory");
}

// Every CTA asks for its share of a later kernel's weights, in pieces of 4 KB.
__device__ __forceinline__ void prefetch_next_weights(const void* base, long long bytes) {
    constexpr long long PIECE = 4096;
    const long long pieces = (bytes + PIECE - 1) / PIECE;
    const long long cta = (long long)blockIdx.y * gridDim.x + blockIdx.x;
    const long long ctas = (long long)gridDim.x * gridDim.y;
    for (long long i = cta * blockDim.x + threadIdx.x; i < pieces; i += ctas * blockDim.x) {
        const long long off = i * PIECE;
        const long long n = bytes - off < PIECE ? bytes - off : PIECE;
        prefetch_l2(static_cast<const char*>(base) + off, (unsigned)(n & ~15LL));
    }
}

// ---- one bulk copy of the norm prologue's input, completion counted on an mbarrier; the wait is bounded
constexpr unsigned WAIT_LIMIT = 1u << 22;
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bulk_copy_to_smem(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}

__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void grid_dependents_launch() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }

template <int NT, int EPI, int NORM>
__global__ void __launch_bounds__(MAX_THREADS) skinny_kernel(const Params p) {
    extern __shared__ __align__(32) unsigned char smem[];
    __shared__ int is_last;
    __shared__ __align__(8) uint64_t staged_bar;
    TraceScope trace_scope(p.trace);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if ((NORM == 2 || (NORM == 1 && p.stage_norm)) && threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(&staged_bar)), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    const int gid = lane >> 2, tig = lane & 3;
    const int rb = warp % p.RB, ks = warp / p.RB;
    const int rows_per_cta = p.RB * 16;
    const int n0 = blockIdx.x * rows_per_cta;
    const int row_a = n0 + rb * 16 + gid, row_b = row_a + 8;
    const bool ok_a = row_a < p.N, ok_b = row_b < p.N;
    const bf16* wa = p.W + (size_t)(ok_a ? row_a : 0) * p.ldw;
    const bf16* wb = p.W + (size_t)(ok_b ? row_b : 0) * p.ldw;
    const int chunks = (p.K + CHUNK - 1) / CHUNK;
    const int slices = p.KS * gridDim.y;
    const int per = (chunks + slices - 1) / slices;
    const int c_lo = (blockIdx.y * p.KS + ks) * per, c_hi = min(chunks, c_lo + per);
    constexpr int MT = NT * 8;

    // The next kernel may start at once: what it does before its own wait (weights, cached keys) does not
    // depend on this kernel, and its wait still covers this kernel's completion.
    if (p.use_pdl == 1) grid_dependents_launch();

    // ---- start the weight stream: UNROLL chunks per row in registers
    W32 wra[UNROLL], wrb[UNROLL];
    auto fetch = [&](int c, W32& ra, W32& rb_) {
        const int k = c * CHUNK + tig * 16;
        const bool in = c < c_hi && k < p.K;                      // K is a multiple of 16
        if (in && ok_a) ra = ldg256(wa + k);
        else
#pragma unroll
            for (int i = 0; i < 8; ++i) ra.r[i] = 0u;
        if (in && ok_b) rb_ = ldg256(wb + k);
        else
#pragma unroll
            for (int i = 0; i < 8; ++i) rb_.r[i] = 0u;
    };
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) fetch(c_lo + u, wra[u], wrb[u]);
    if (p.prefetch) prefetch_next_weights(p.prefetch, p.prefetch_bytes);
    // The norm's gain is a weight too: it goes to shared memory (behind x and the row factors)
    // before the wait, so that its trip from HBM is off the critical path.
    const int xs_stride = ((p.K * 2 + 127) / 128) * 128 + 64;     // bytes; rows 16 banks apart
    float* gain_s = reinterpret_cast<float*>(smem + (size_t)MT * xs_stride + MT * sizeof(float));
    if (NORM == 1) {
        const float4* g = reinterpret_cast<const float4*>(p.gain);
        for (int i = threadIdx.x; i < p.K / 4; i += blockDim.x) reinterpret_cast<float4*>(gain_s)[i] = g[i];
    }

    // qkv_rope epilogue: positions, cache slots, frequencies and biases were there before the step began, so the
    // rotation of this thread's first output pair is prepared here, off the critical path
    float rope_cos = 1.f, rope_sin = 0.f, first_bias0 = 0.f, first_bias1 = 0.f;
    long long first_slot = -1;
    if (EPI == EPI_QKV_ROPE) {
        const int half = p.head_dim / 2, e = threadIdx.x;
        const bool rotated = (int)blockIdx.x < p.num_heads + p.num_kv_heads;
        if (rotated && e < half * p.M) {
            const float a = (float)p.positions[e / half] * p.inv_freq[e % half];
            rope_cos = cosf(a);
            rope_sin = sinf(a);
            if (p.bias) {
                first_bias0 = p.bias[n0 + e % half];
                first_bias1 = p.bias[n0 + e % half + half];
            }
            if ((int)blockIdx.x >= p.num_heads) first_slot = p.slot_map[e / half];
        } else if (!rotated && e < p.head_dim * p.M) {
            if (p.bias) first_bias0 = p.bias[n0 + e % p.head_dim];
            first_slot = p.slot_map[e / p.head_dim];
        }
    }

    trace_scope.mark(0);
    if (p.use_pdl) grid_dependency_wait();                        // from here on the previous kernel's results are read
    // (Measured on B200, decode at batch 8: letting the next kernel start here takes 0.855 ms a step; once this kernel's
    // input rows are there 0.854, once its product is done 0.876, once its slices are summed 0.917.)
    if (p.use_pdl == 2) grid_dependents_launch();
    trace_scope.mark(1);

    // ---- x: staged into shared memory by the norm prologue, or read from global memory
    unsigned char* xs = smem;
    float* row_factor = reinterpret_cast<float*>(smem + (size_t)MT * xs_stride);      // [MT]
    const int nwarps = blockDim.x >> 5;
    if (NORM) {
        const int quads = p.K / 4;
        float* ss_part = gain_s + p.K;                            // [rows][parts] partial sums of squares
        // With more warps than rows, several warps share a row (a stretch each), so that every lane's
        // loads go out in one batch; with fewer, a warp takes several rows one after the other.
        const int parts = p.M > 0 && nwarps >= p.M ? min(nwarps / p.M, 8) : 1;
        const int per_part = (quads + parts - 1) / parts;
        // The residual (and the delta, straight into its row of xs, where the normalised value replaces it) come
        // in one batch of bulk copies: one trip to the L2 for the whole input, instead of one per pass of the loop.
        const float* staged_resid = reinterpret_cast<const float*>(ss_part + MT * 8);
        __syncthreads();                                          // gain_s is complete, and everyone sees the barrier's init
        if (NORM == 2) {
            // rows bfloat16(gain * v) straight into xs, the partial sums of squares where the residual would be staged
            float* ss_s = const_cast<float*>(staged_resid);       // [ss_parts][MT]
            // (Plain 16-byte loads by every thread instead of the bulk copies were measured slower: 0.853 against 0.821 ms a
            // decode step at batch 8.)
            {
            if (warp == 0) {
                if (lane == 0) {
                    const unsigned bytes = (unsigned)p.M * (unsigned)p.K * 2u + (unsigned)p.ss_parts * MT * 4u;
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(&staged_bar)), "r"(bytes) : "memory");
                    bulk_copy_to_smem(ss_s, p.ss_in, (unsigned)p.ss_parts * MT * 4u, &staged_bar);
                }
                __syncwarp();
                for (int m = lane; m < p.M; m += 32)
                    bulk_copy_to_smem(xs + (size_t)m * xs_stride, p.delta + (size_t)m * p.K, (unsigned)p.K * 2u, &staged_bar);
            }
            for (int e = threadIdx.x; e < (MT - p.M) * quads; e += blockDim.x)      // rows that only pad the token tile
                reinterpret_cast<uint2*>(xs + (size_t)(p.M + e / quads) * xs_stride)[e % quads] = make_uint2(0u, 0u);
            bool landed = false;
            for (unsigned i = 0; i < WAIT_LIMIT && !landed; ++i) landed = mbar_try_wait(&staged_bar, 0);
            if (!landed && p.status) atomicOr(p.status, EG_STATUS_WAIT_TIMEOUT);
            }
            if (threadIdx.x < MT) {
                float f = 0.f;
                if ((int)threadIdx.x < p.M) {
                    float ss = 0.f;
                    for (int q = 0; q < p.ss_parts; ++q) ss += ss_s[q * MT + threadIdx.x];      // fixed order
                    f = 1.0f / sqrtf(ss / (float)p.K + p.eps);
                }
                row_factor[threadIdx.x] = f;
            }
            __syncthreads();
        } else {
        if (p.stage_norm) {
            if (warp == 0) {
                if (lane == 0) {
                    const unsigned bytes = (unsigned)p.M * (unsigned)p.K * (p.delta ? 6u : 4u);
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(&staged_bar)), "r"(bytes) : "memory");
                    bulk_copy_to_smem(const_cast<float*>(staged_resid), p.resid_in, (unsigned)p.M * (unsigned)p.K * 4u, &staged_bar);
                }
                __syncwarp();
                if (p.delta)
                    for (int m = lane; m < p.M; m += 32)
                        bulk_copy_to_smem(xs + (size_t)m * xs_stride, p.delta + (size_t)m * p.K, (unsigned)p.K * 2u, &staged_bar);
            }
            bool landed = false;
            for (unsigned i = 0; i < WAIT_LIMIT && !landed; ++i) landed = mbar_try_wait(&staged_bar, 0);
            if (!landed && p.status) atomicOr(p.status, EG_STATUS_WAIT_TIMEOUT);
        }
        for (int task = warp; task < p.M * parts; task += nwarps) {
            const int m = task / parts, part = task % parts;
            const int q_lo = part * per_part, q_hi = min(quads, q_lo + per_part);
            uint2* dst = reinterpret_cast<uint2*>(xs + (size_t)m * xs_stride);
            const float4* r = reinterpret_cast<const float4*>((p.stage_norm ? staged_resid : p.resid_in) + (size_t)m * p.K);
            const uint2* d = !p.delta ? nullptr
                             : p.stage_norm ? reinterpret_cast<const uint2*>(xs + (size_t)m * xs_stride)
                                            : reinterpret_cast<const uint2*>(p.delta + (size_t)m * p.K);
            const float4* g = reinterpret_cast<const float4*>(gain_s);
            float4* ro = (blockIdx.x == 0 && blockIdx.y == 0 && p.resid_out)
                             ? reinterpret_cast<float4*>(p.resid_out + (size_t)m * p.K) : nullptr;
            float ss = 0.f;
            // four quads per lane at a time: all loads of a batch are issued before anything is
            // stored, so that they overlap (a store to the residual could alias them otherwise)
            constexpr int BATCH = 4;
            for (int i0 = q_lo + lane; i0 < q_hi; i0 += 32 * BATCH) {
                float4 rv[BATCH], gv[BATCH];
                uint2 dv[BATCH];
#pragma unroll
                for (int b = 0; b < BATCH; ++b) {
                    const int i = i0 + 32 * b;
                    if (i < q_hi) {
                        rv[b] = r[i];
                        gv[b] = g[i];
                        dv[b] = d ? d[i] : make_uint2(0u, 0u);
                    }
                }
#pragma unroll
                for (int b = 0; b < BATCH; ++b) {
                    const int i = i0 + 32 * b;
                    if (i < q_hi) {
                        float4 v = rv[b];
                        const __nv_bfloat162 d01 = *reinterpret_cast<const __nv_bfloat162*>(&dv[b].x);
                        const __nv_bfloat162 d23 = *reinterpret_cast<const __nv_bfloat162*>(&dv[b].y);
                        v.x += __low2float(d01); v.y += __high2float(d01); v.z += __low2float(d23); v.w += __high2float(d23);
                        if (ro) ro[i] = v;
                        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                        dst[i] = make_uint2(pack_bf16(gv[b].x * v.x, gv[b].y * v.y), pack_bf16(gv[b].z * v.z, gv[b].w * v.w));
                    }
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) ss_part[m * parts + part] = ss;
        }
        // rows that only pad the token tile are zero
        for (int e = threadIdx.x; e < (MT - p.M) * quads; e += blockDim.x)
            reinterpret_cast<uint2*>(xs + (size_t)(p.M + e / quads) * xs_stride)[e % quads] = make_uint2(0u, 0u);
        __syncthreads();
        if (threadIdx.x < MT) {
            float f = 0.f;
            if ((int)threadIdx.x < p.M) {
                float ss = 0.f;
                for (int q = 0; q < parts; ++q) ss += ss_part[threadIdx.x * parts + q];      // fixed order
                f = 1.0f / sqrtf(ss / (float)p.K + p.eps);
            }
            row_factor[threadIdx.x] = f;
        }
        __syncthreads();
        }
    }

    trace_scope.mark(2);
    // resid_norm epilogue: this thread's first output (token, column) is known now; its residual element and gain
    // are asked for here, so that their trip from the L2 runs beside the product
    float resid_first = 0.f, gain_first = 0.f;
    if (EPI == EPI_RESID_NORM) {
        const int e = threadIdx.x;
        if (e < rows_per_cta * p.M) {
            const int m = e / rows_per_cta, n = n0 + e % rows_per_cta;
            if (n < p.N) {
                resid_first = p.resid_inout[(size_t)m * p.N + n];
                gain_first = p.gain_out[n];
            }
        }
    }
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    for (int c = c_lo; c < c_hi; c += UNROLL) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = (c + u) * CHUNK + tig * 16;
            if (c + u < c_hi) {                                   // the same for the whole warp
                // Lanes whose k lies beyond K feed zeros but still take part: mma.sync is
                // a warp-wide instruction and must not be skipped by some lanes.
                const bool k_in = k < p.K;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int m = nt * 8 + gid;
                    uint4 x0 = make_uint4(0, 0, 0, 0), x1 = make_uint4(0, 0, 0, 0);
                    if (NORM) {
                        if (k_in) {
                            const uint4* src = reinterpret_cast<const uint4*>(xs + (size_t)m * xs_stride + (size_t)k * 2);
                            x0 = src[0];
                            x1 = src[1];
                        }
                    } else if (k_in && m < p.M) {
                        const uint4* src = reinterpret_cast<const uint4*>(p.x + (size_t)m * p.ldx + k);
                        x0 = src[0];
                        x1 = src[1];
                    }
                    // four k-steps of 16: step s takes this thread's elements 4s .. 4s+3 of both operands
                    const uint32_t xr[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
                        const uint32_t a[4] = {wra[u].r[2 * s], wrb[u].r[2 * s], wra[u].r[2 * s + 1], wrb[u].r[2 * s + 1]};
                        mma_bf16_16816(acc[nt], a, xr[2 * s], xr[2 * s + 1]);
                    }
                }
            }
            fetch(c + UNROLL + u, wra[u], wrb[u]);                // this register set's next chunk, UNROLL chunks ahead
        }
    }
    trace_scope.mark(3, true);

    // ---- sum the K slices of this CTA: red[warp][row][token] -> tile[row in CTA][token]
    float my_factor = 1.f;
    if (NORM && threadIdx.x < MT) my_factor = row_factor[threadIdx.x];
    __syncthreads();                                              // xs is dead; reuse the memory
    float* red = reinterpret_cast<float*>(smem);                  // [nwarps][16][MT]
    float* tile = red + (size_t)nwarps * 16 * MT;                 // [rows_per_cta][MT]
    float* factor = tile + (size_t)rows_per_cta * MT;             // [MT]
    if (threadIdx.x < MT) factor[threadIdx.x] = my_factor;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        float* base = red + (size_t)warp * 16 * MT + nt * 8 + 2 * tig;
        base[(size_t)gid * MT] = acc[nt][0];
        base[(size_t)gid * MT + 1] = acc[nt][1];
        base[(size_t)(gid + 8) * MT] = acc[nt][2];
        base[(size_t)(gid + 8) * MT + 1] = acc[nt][3];
    }
    __syncthreads();
    const int tile_elems = rows_per_cta * MT;
    for (int e = threadIdx.x; e < tile_elems; e += blockDim.x) {
        const int r = e / MT, m = e % MT;
        float v = 0.f;
        for (int s = 0; s < p.KS; ++s) v += red[((size_t)(s * p.RB + r / 16) * 16 + (r % 16)) * MT + m];
        tile[e] = v;
    }
    __syncthreads();

    trace_scope.mark(4);
    // ---- K cut across CTAs that form a cluster: every CTA puts its part into the first one's shared memory (two
    // trips to the L2 fewer than the ticket below), the first one sums them, in order
    if (gridDim.y > 1 && p.cluster_reduce) {
        float* parts = reinterpret_cast<float*>(smem + p.parts_offset);   // [gridDim.y][tile_elems], used in the cluster's first CTA only; behind the input rows
        unsigned rank;
        asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(smem_addr(parts + (size_t)rank * tile_elems)), "r"(0));
        for (int e = threadIdx.x; e < tile_elems; e += blockDim.x)
            asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(remote + (uint32_t)e * 4u), "f"(tile[e]) : "memory");
        asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
        if (rank != 0) return;
        for (int e = threadIdx.x; e < tile_elems; e += blockDim.x) {
            float v = 0.f;
            for (int y = 0; y < (int)gridDim.y; ++y) v += parts[(size_t)y * tile_elems + e];
            tile[e] = v;
        }
        __syncthreads();
    } else
    // ---- K cut across CTAs: the last CTA of this row group to arrive sums all parts, in order
    if (gridDim.y > 1) {
        float* mine = p.scratch + ((size_t)blockIdx.y * gridDim.x + blockIdx.x) * tile_elems;
        for (int e = threadIdx.x; e < tile_elems; e += blockDim.x) mine[e] = tile[e];
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const int ticket = atomicAdd(&p.counters[blockIdx.x], 1);
            is_last = ticket == (int)gridDim.y - 1;
            if (is_last) p.counters[blockIdx.x] = 0;              // everyone has arrived: ready for the next launch
        }
        __syncthreads();
        if (!is_last) return;
        __threadfence();
        for (int e = threadIdx.x; e < tile_elems; e += blockDim.x) {
            float v = 0.f;
            for (int y = 0; y < (int)gridDim.y; ++y)
                v += __ldcg(p.scratch + ((size_t)y * gridDim.x + blockIdx.x) * tile_elems + e);
            tile[e] = v;
        }
        __syncthreads();
    }

    trace_scope.mark(5);
    auto product = [&](int r, int m) -> float {                   // r: row inside the CTA; without the bias
        float v = tile[r * MT + m];
        if (NORM) v *= factor[m];
        return v;
    };
    auto value = [&](int r, int m) -> float {
        float v = product(r, m);
        const int n = n0 + r;
        if (p.bias && n < p.N) v += p.bias[n];
        return v;
    };

    if (EPI == EPI_STORE || EPI == EPI_F32) {
        for (int e = threadIdx.x; e < rows_per_cta * p.M; e += blockDim.x) {
            const int m = e / rows_per_cta, r = e % rows_per_cta;
            const int n = n0 + r;
            if (n >= p.N) continue;
            const float v = value(r, m);
            if (EPI == EPI_F32) p.out_f32[(size_t)m * p.ldo + n] = v;
            else p.out[(size_t)m * p.ldo + n] = __float2bfloat16_rn(v);
        }
    } else if (EPI == EPI_SWIGLU) {
        const int half = rows_per_cta / 2;
        for (int e = threadIdx.x; e < half * p.M; e += blockDim.x) {
            const int m = e / half, i = e % half;
            const int n = n0 + 2 * i;
            if (n + 1 >= p.N) continue;
            const float g = value(2 * i, m), u = value(2 * i + 1, m);
            const float sig = 1.0f / (1.0f + expf(-g));
            p.out[(size_t)m * p.ldo + (n >> 1)] = __float2bfloat16_rn(u * (g * sig));
        }
    } else if (EPI == EPI_RESID_NORM) {
        float* sq = red;                                              // [rows_per_cta][MT] squares (the slices' memory is free)
        for (int e = threadIdx.x; e < rows_per_cta * MT; e += blockDim.x) sq[e] = 0.f;
        __syncthreads();
        for (int e = threadIdx.x; e < rows_per_cta * p.M; e += blockDim.x) {
            const int m = e / rows_per_cta, r = e % rows_per_cta;
            const int n = n0 + r;
            if (n >= p.N) continue;
            const bool first = e == (int)threadIdx.x;
            const float y = __bfloat162float(__float2bfloat16_rn(value(r, m)));      // what a stored delta would hold
            const float v = (first ? resid_first : p.resid_inout[(size_t)m * p.N + n]) + y;
            const float g = first ? gain_first : p.gain_out[n];
            p.resid_inout[(size_t)m * p.N + n] = v;
            p.xn_out[(size_t)m * p.N + n] = __float2bfloat16_rn(g * v);
            sq[r * MT + m] = v * v;
        }
        __syncthreads();
        if (threadIdx.x < MT) {
            float ss = 0.f;
            for (int r = 0; r < rows_per_cta; ++r) ss += sq[r * MT + threadIdx.x];   // fixed order
            p.ss_out[(size_t)blockIdx.x * MT + threadIdx.x] = ss;
        }
    } else {   // EPI_QKV_ROPE: this CTA holds one whole head
        const int HD = p.head_dim, half = HD / 2;
        const int head = blockIdx.x;
        const bool is_q = head < p.num_heads, is_k = !is_q && head < p.num_heads + p.num_kv_heads;
        if (is_q || is_k) {
            for (int e = threadIdx.x; e < half * p.M; e += blockDim.x) {
                const int m = e / half, j = e % half;
                const bool first = e == (int)threadIdx.x;               // what was fetched before the wait
                const float x0 = first ? product(j, m) + first_bias0 : value(j, m);
                const float x1 = first ? product(j + half, m) + first_bias1 : value(j + half, m);
                float cs = rope_cos, sn = rope_sin;
                if (!first) {
                    const float a = (float)p.positions[m] * p.inv_freq[j];
                    cs = cosf(a);
                    sn = sinf(a);
                }
                const float y0 = x0 * cs - x1 * sn, y1 = x0 * sn + x1 * cs;
                if (is_q) {
                    bf16* o = p.out + (size_t)m * p.ldo + (size_t)head * HD;
                    o[j] = __float2bfloat16_rn(y0);
                    o[j + half] = __float2bfloat16_rn(y1);
                } else {
                    const long long slot = first ? first_slot : p.slot_map[m];
                    if (slot < 0 || slot >= p.pool_slots) {
                        if (slot >= p.pool_slots) atomicOr(p.status, EG_STATUS_BAD_SLOT);
                        continue;
                    }
                    bf16* o = p.k_cache + (slot / p.page_size) * p.page_stride + (long long)(head - p.num_heads) * p.head_stride +
                              (slot % p.page_size) * HD;
                    o[j] = __float2bfloat16_rn(y0);
                    o[j + half] = __float2bfloat16_rn(y1);
                }
            }
        } else {
            for (int e = threadIdx.x; e < HD * p.M; e += blockDim.x) {
                const int m = e / HD, j = e % HD;
                const bool first = e == (int)threadIdx.x;
                const long long slot = first ? first_slot : p.slot_map[m];
                if (slot < 0 || slot >= p.pool_slots) {
                    if (slot >= p.pool_slots) atomicOr(p.status, EG_STATUS_BAD_SLOT);
                    continue;
                }
                bf16* o = p.v_cache + (slot / p.page_size) * p.page_stride +
                          (long long)(head - p.num_heads - p.num_kv_heads) * p.head_stride + (slot % p.page_size) * HD;
                o[j] = __float2bfloat16_rn(first ? product(j, m) + first_bias0 : value(j, m));
            }
        }
    }
}

template <int NT, int EPI, int NORM>
int launch_one(cudaStream_t stream, const Params& p_in, int ctas, int k_split) {
    constexpr int MT = NT * 8;
    Params p = p_in;
    const int nwarps = p.RB * p.KS;
    const size_t red_bytes = ((size_t)nwarps * 16 * MT + (size_t)p.RB * 16 * MT + MT) * sizeof(float);
    // The CTAs that share a row group's K range as a cluster (up to 8, the portable size): their parts arrive in the
    // first CTA's shared memory behind everything else, since that CTA may still be multiplying from its input rows.
    static const bool cluster_allowed = !(getenv("EASY_GPT_CLUSTER_REDUCE") && atoi(getenv("EASY_GPT_CLUSTER_REDUCE")) == 0);
    const size_t parts_bytes_cluster = (size_t)k_split * p.RB * 16 * MT * sizeof(float);
    p.cluster_reduce = cluster_allowed && k_split > 1 && k_split <= 8 && parts_bytes_cluster <= 32 * 1024;
    size_t xs_bytes = NORM ? (size_t)MT * (((p.K * 2 + 127) / 128) * 128 + 64) + MT * sizeof(float) + (size_t)p.K * sizeof(float) + (size_t)MT * 8 * sizeof(float) : 0;
    // the residual rows staged in shared memory, where they fit and the copies' alignment rule (16 bytes) holds
    const size_t staged_bytes = (size_t)p.M * p.K * sizeof(float);
    if (NORM == 2) {
        const size_t parts_bytes = (size_t)p.ss_parts * MT * sizeof(float);
        if ((uintptr_t)p.delta % 16 || (uintptr_t)p.ss_in % 16 || (size_t)p.M * p.K * 2 + parts_bytes >= (1u << 20))
            return (int)cudaErrorInvalidValue;
        xs_bytes += parts_bytes;
    }
    p.stage_norm = NORM == 1 && xs_bytes + staged_bytes + (p.cluster_reduce ? parts_bytes_cluster + 16 : 0) <= 200 * 1024 && (uintptr_t)p.resid_in % 16 == 0 && (uintptr_t)p.delta % 16 == 0 &&
                   (size_t)p.M * p.K * 6 < (1u << 20);
    if (p.stage_norm) xs_bytes += staged_bytes;
    size_t smem_bytes = red_bytes > xs_bytes ? red_bytes : xs_bytes;
    if (p.cluster_reduce) {
        p.parts_offset = (int)((smem_bytes + 15) / 16 * 16);
        smem_bytes = (size_t)p.parts_offset + parts_bytes_cluster;
    }
    if (smem_bytes > 200 * 1024) return (int)cudaErrorInvalidValue;
    auto kernel = skinny_kernel<NT, EPI, NORM>;
    static size_t configured = 0;
    if (smem_bytes > 48 * 1024 && smem_bytes > configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
        if (e != cudaSuccess) return (int)e;
        configured = smem_bytes;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas, k_split);
    cfg.blockDim = dim3(nwarps * 32);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int nattr = 0;
    if (p.use_pdl) {
        attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[nattr].val.programmaticStreamSerializationAllowed = 1;
        ++nattr;
    }
    if (p.cluster_reduce) {
        attr[nattr].id = cudaLaunchAttributeClusterDimension;
        attr[nattr].val.clusterDim.x = 1;
        attr[nattr].val.clusterDim.y = (unsigned)k_split;
        attr[nattr].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = nattr + 1;
        // All clusters have to find room on the GPU together, or the last ones run as a second wave, after the first
        // (1.5B sizes, down product, 96 clusters of 3: their last CTAs started 9 us after the kernel in front had ended).
        // Then the parts go through scratch memory and a ticket, which asks nothing of where the CTAs run.
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) == cudaSuccess && clusters >= ctas) {
            ++nattr;
        } else {
            (void)cudaGetLastError();
            if (!p.scratch || !p.counters) return (int)cudaErrorInvalidValue;
            p.cluster_reduce = 0;
        }
    }
    cfg.attrs = attr;
    cfg.numAttrs = nattr;
    return (int)cudaLaunchKernelEx(&cfg, kernel, p);
}

template <int EPI, int NORM>
int launch_nt(cudaStream_t stream, const Params& p, int ctas, int k_split) {
    if (p.M <= 8) return launch_one<1, EPI, NORM>(stream, p, ctas, k_split);
    if (p.M <= 16) return launch_one<2, EPI, NORM>(stream, p, ctas, k_split);
    if (p.M <= 32) return launch_one<4, EPI, NORM>(stream, p, ctas, k_split);
    if (p.M <= 64) return launch_one<8, EPI, NORM>(stream, p, ctas, k_split);
    return (int)cudaErrorInvalidValue;
}

}  // namespace

// epilogue: 0 store bf16, 1 store f32, 2 swiglu (interleaved rows), 3 qkv + rope + cache (one CTA per head).
// epilogue 4 (resid_norm): resid_inout is the residual [M, N], updated in place; gain_out [N], xn_out bfloat16 [M, N],
// ss_out float32 [ceil(N / (row_blocks*16))][padded tokens] receive what the next kernel's norm == 2 prologue reads.
// norm == 1: x = gain * rmsnorm(resid_in + delta) (delta may be null), resid_out (may be null) receives the sum.
// norm == 2: delta holds bfloat16(gain * v) [M, K] and ss_in [ss_parts][padded tokens] the partial sums of v^2.
// row_blocks x k_slices warps per CTA (their product 1..16); k_split CTAs share the K range of a row group and
// then need `scratch` (k_split * ceil(N / (row_blocks*16)) * row_blocks*16 * padded tokens floats) and `counters`
// (one zeroed int per row group; left zero).  Takes M <= 64, K % 16 == 0, 32-byte aligned rows of W, 16-byte
// aligned rows of x.  Anything else: cudaErrorInvalidValue.
EG_API int eg_gemm_skinny(cudaStream_t stream, int epilogue, int norm, int use_pdl, const void* W, long long ldw,
                          const float* bias, int M, int N, int K, const void* x, long long ldx, const float* resid_in,
                          float* resid_out, const void* delta, const float* gain, float eps, void* out, long long ldo,
                          int row_blocks, int k_slices, int k_split, float* scratch, int* counters, int num_heads,
                          int num_kv_heads, int head_dim, const int* positions, const int* slot_map, void* k_cache,
                          void* v_cache, const float* inv_freq, int page_size, long long page_stride,
                          long long head_stride, long long pool_slots, int* status, const void* prefetch,
                          long long prefetch_bytes, unsigned long long* trace, const float* ss_in, int ss_parts,
                          float* resid_inout, const float* gain_out, void* xn_out, float* ss_out) {
    if (M <= 0 || N <= 0) return 0;
    if (norm < 0 || norm > 2 || (norm == 2 && (!delta || !ss_in || ss_parts < 1)) ||
        (epilogue == EPI_RESID_NORM && (!resid_inout || !gain_out || !xn_out || !ss_out)))
        return (int)cudaErrorInvalidValue;
    if (M > 64 || K % 16 || ldw % 16 || (!norm && ldx % 8) || row_blocks < 1 || k_slices < 1 ||
        row_blocks * k_slices > MAX_THREADS / 32 || k_split < 1 || k_split > 64 || (k_split > 1 && (!scratch || !counters)))
        return (int)cudaErrorInvalidValue;
    if (epilogue == EPI_QKV_ROPE && (row_blocks * 16 != head_dim || N != (num_heads + 2 * num_kv_heads) * head_dim))
        return (int)cudaErrorInvalidValue;
    if (epilogue == EPI_SWIGLU && (N % 2)) return (int)cudaErrorInvalidValue;
    Params p{};
    p.W = (const bf16*)W; p.ldw = ldw; p.bias = bias; p.M = M; p.N = N; p.K = K;
    p.x = (const bf16*)x; p.ldx = ldx; p.resid_in = resid_in; p.resid_out = resid_out; p.delta = (const bf16*)delta;
    p.gain = gain; p.eps = eps; p.out = (bf16*)out; p.ldo = ldo; p.out_f32 = (float*)out;
    p.num_heads = num_heads; p.num_kv_heads = num_kv_heads; p.head_dim = head_dim; p.positions = positions;
    p.slot_map = slot_map; p.k_cache = (bf16*)k_cache; p.v_cache = (bf16*)v_cache; p.inv_freq = inv_freq;
    p.page_size = page_size; p.page_stride = page_stride; p.head_stride = head_stride; p.pool_slots = pool_slots;
    p.status = status; p.RB = row_blocks; p.KS = k_slices; p.use_pdl = use_pdl;
    p.prefetch = prefetch_bytes >= 16 ? prefetch : nullptr; p.prefetch_bytes = prefetch_bytes;
    p.scratch = scratch; p.counters = counters; p.trace = trace;
    p.norm_mode = norm; p.ss_in = ss_in; p.ss_parts = ss_parts;
    p.resid_inout = resid_inout; p.gain_out = gain_out; p.xn_out = (bf16*)xn_out; p.ss_out = ss_out;
    const int ctas = (N + row_blocks * 16 - 1) / (row_blocks * 16);
#define EG_SKINNY(E)                                                                             \
    case E: return norm == 2 ? launch_nt<E, 2>(stream, p, ctas, k_split)                          \
                   : norm ? launch_nt<E, 1>(stream, p, ctas, k_split) : launch_nt<E, 0>(stream, p, ctas, k_split);
    switch (epilogue) {
        EG_SKINNY(EPI_STORE)
        EG_SKINNY(EPI_F32)
        EG_SKINNY(EPI_SWIGLU)
        EG_SKINNY(EPI_QKV_ROPE)
        EG_SKINNY(EPI_RESID_NORM)
        default: return (int)cudaErrorInvalidValue;
    }
#undef EG_SKINNY
}
