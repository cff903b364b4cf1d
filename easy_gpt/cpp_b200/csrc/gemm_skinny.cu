// Matrix products for decode steps (1..64 tokens): y[m, n] = sum_k x[m, k] W[n, k].
//
// With so few tokens the product is a stream of the weights from HBM, so the
// kernel is built around that stream.  The roles of the MMA are swapped: 16 weight
// rows are the M side of mma.m16n8k16 and 8 tokens are its N side, so no tensor
// core work is wasted on padding tokens up to a tile.  Every thread fetches its
// piece of the weight fragment with one 16-byte load straight from global memory
// (8 consecutive k of one row; the k order inside a 32-wide chunk is permuted the
// same way for both operands, which a sum does not notice), several chunks ahead,
// and nothing of W passes through shared memory.  A CTA has 8 warps arranged as
// RB row blocks x KS slices of K; the slices are summed through shared memory in a
// fixed order.
//
// Prologues (what x is):
//   plain      x is a bfloat16 matrix in global memory
//   norm       x = gain * rmsnorm(residual_in + delta) computed by every CTA into
//              shared memory (float32 sums, src/models/norm.cpp:46-60); CTA 0 also
//              writes residual_in + delta to residual_out (another buffer, so that
//              no CTA reads what CTA 0 has already updated)
// Epilogues (what happens to y):
//   store      + bias -> bfloat16 [M, N]
//   f32        + bias -> float32 [M, N] (logits)
//   swiglu     rows of W interleaved (2i = gate_i, 2i+1 = up_i): up * silu(gate) -> bfloat16 [M, N/2]
//   qkv_rope   one CTA per head (RB*16 == head_dim): + bias, q and k rotated
//              (src/ops.cpp:404-421), q -> bfloat16 [M, NH*HD], k and v -> paged cache
//
// Every kernel starts streaming its weights before it waits for the kernel in front
// of it (programmatic dependent launch), so the pipeline of small kernels overlaps.
#include "mma_utils.cuh"

namespace {

constexpr int THREADS = 256;
constexpr int UNROLL = 4;            // 32-wide k chunks in flight per warp

enum { EPI_STORE = 0, EPI_F32 = 1, EPI_SWIGLU = 2, EPI_QKV_ROPE = 3 };

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
};

__device__ __forceinline__ uint4 ldg128(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void grid_dependents_launch() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }

template <int NT, int EPI, bool NORM>
__global__ void __launch_bounds__(THREADS) skinny_kernel(const Params p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int rb = warp % p.RB, ks = warp / p.RB;
    const int rows_per_cta = p.RB * 16;
    const int n0 = blockIdx.x * rows_per_cta;
    const int row_a = n0 + rb * 16 + gid, row_b = row_a + 8;
    const bool ok_a = row_a < p.N, ok_b = row_b < p.N;
    const bf16* wa = p.W + (size_t)(ok_a ? row_a : 0) * p.ldw;
    const bf16* wb = p.W + (size_t)(ok_b ? row_b : 0) * p.ldw;
    const int chunks = (p.K + 31) / 32;
    const int per = (chunks + p.KS - 1) / p.KS;
    const int c_lo = ks * per, c_hi = min(chunks, c_lo + per);

    // ---- start the weight stream: UNROLL chunks per row in registers
    uint4 wra[UNROLL], wrb[UNROLL];
    auto fetch = [&](int c, uint4& ra, uint4& rb_) {
        const int k = c * 32 + tig * 8;
        const bool in = c < c_hi && k < p.K;                      // K is a multiple of 8
        ra = (in && ok_a) ? ldg128(wa + k) : make_uint4(0, 0, 0, 0);
        rb_ = (in && ok_b) ? ldg128(wb + k) : make_uint4(0, 0, 0, 0);
    };
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) fetch(c_lo + u, wra[u], wrb[u]);

    if (p.use_pdl) grid_dependency_wait();                        // from here on the previous kernel's results are read

    // ---- x: normalised into shared memory, or read from global memory
    const int xs_stride = ((p.K * 2 + 127) / 128) * 128 + 64;     // bytes; rows 16 banks apart
    unsigned char* xs = smem;
    if (NORM) {
        for (int m = warp; m < NT * 8; m += THREADS / 32) {
            bf16* dst = reinterpret_cast<bf16*>(xs + (size_t)m * xs_stride);
            if (m >= p.M) {
                for (int k = lane; k < p.K; k += 32) dst[k] = __float2bfloat16_rn(0.f);
                continue;
            }
            const float* r = p.resid_in + (size_t)m * p.K;
            const bf16* d = p.delta ? p.delta + (size_t)m * p.K : nullptr;
            float* ro = (blockIdx.x == 0 && p.resid_out) ? p.resid_out + (size_t)m * p.K : nullptr;
            float ss = 0.f;
            for (int k = lane; k < p.K; k += 32) {
                float v = r[k];
                if (d) v += __bfloat162float(d[k]);
                if (ro) ro[k] = v;
                ss += v * v;
            }
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)p.K + p.eps);
            for (int k = lane; k < p.K; k += 32) {
                float v = r[k];
                if (d) v += __bfloat162float(d[k]);
                dst[k] = __float2bfloat16_rn(p.gain[k] * (v * inv));
            }
        }
        __syncthreads();
    }

    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    for (int c = c_lo; c < c_hi; c += UNROLL) {
        uint4 ca[UNROLL], cb[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            ca[u] = wra[u];
            cb[u] = wrb[u];
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) fetch(c + UNROLL + u, wra[u], wrb[u]);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = (c + u) * 32 + tig * 8;
            if (c + u >= c_hi) continue;                          // the same for the whole warp
            // Lanes whose k lies beyond K feed zeros but still take part: mma.sync is
            // a warp-wide instruction and must not be skipped by some lanes.
            const bool k_in = k < p.K;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int m = nt * 8 + gid;
                uint4 xv = make_uint4(0, 0, 0, 0);
                if (NORM) {
                    if (k_in) xv = *reinterpret_cast<const uint4*>(xs + (size_t)m * xs_stride + (size_t)k * 2);
                } else {
                    if (k_in && m < p.M) xv = *reinterpret_cast<const uint4*>(p.x + (size_t)m * p.ldx + k);
                }
                const uint32_t a0[4] = {ca[u].x, cb[u].x, ca[u].y, cb[u].y};
                const uint32_t a1[4] = {ca[u].z, cb[u].z, ca[u].w, cb[u].w};
                mma_bf16_16816(acc[nt], a0, xv.x, xv.y);
                mma_bf16_16816(acc[nt], a1, xv.z, xv.w);
            }
        }
    }
    if (p.use_pdl) grid_dependents_launch();                      // the next kernel may start its own weight stream

    // ---- sum the K slices: red[ks][row in CTA][token]
    __syncthreads();                                              // xs is dead; reuse the memory
    float* red = reinterpret_cast<float*>(smem);
    const int MT = NT * 8;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        float* base = red + ((size_t)ks * rows_per_cta + rb * 16) * MT + nt * 8 + 2 * tig;
        base[(size_t)gid * MT] = acc[nt][0];
        base[(size_t)gid * MT + 1] = acc[nt][1];
        base[(size_t)(gid + 8) * MT] = acc[nt][2];
        base[(size_t)(gid + 8) * MT + 1] = acc[nt][3];
    }
    __syncthreads();
    auto value = [&](int r, int m) -> float {                     // r: row inside the CTA
        float v = 0.f;
        for (int s = 0; s < p.KS; ++s) v += red[((size_t)s * rows_per_cta + r) * MT + m];
        const int n = n0 + r;
        if (p.bias && n < p.N) v += p.bias[n];
        return v;
    };

    if (EPI == EPI_STORE || EPI == EPI_F32) {
        for (int e = threadIdx.x; e < rows_per_cta * p.M; e += THREADS) {
            const int m = e / rows_per_cta, r = e % rows_per_cta;
            const int n = n0 + r;
            if (n >= p.N) continue;
            const float v = value(r, m);
            if (EPI == EPI_F32) p.out_f32[(size_t)m * p.ldo + n] = v;
            else p.out[(size_t)m * p.ldo + n] = __float2bfloat16_rn(v);
        }
    } else if (EPI == EPI_SWIGLU) {
        const int half = rows_per_cta / 2;
        for (int e = threadIdx.x; e < half * p.M; e += THREADS) {
            const int m = e / half, i = e % half;
            const int n = n0 + 2 * i;
            if (n + 1 >= p.N) continue;
            const float g = value(2 * i, m), u = value(2 * i + 1, m);
            const float sig = 1.0f / (1.0f + expf(-g));
            p.out[(size_t)m * p.ldo + (n >> 1)] = __float2bfloat16_rn(u * (g * sig));
        }
    } else {   // EPI_QKV_ROPE: this CTA holds one whole head
        const int HD = p.head_dim, half = HD / 2;
        const int head = blockIdx.x;
        const bool is_q = head < p.num_heads, is_k = !is_q && head < p.num_heads + p.num_kv_heads;
        if (is_q || is_k) {
            for (int e = threadIdx.x; e < half * p.M; e += THREADS) {
                const int m = e / half, j = e % half;
                const float x0 = value(j, m), x1 = value(j + half, m);
                const float a = (float)p.positions[m] * p.inv_freq[j];
                const float cs = cosf(a), sn = sinf(a);
                const float y0 = x0 * cs - x1 * sn, y1 = x0 * sn + x1 * cs;
                if (is_q) {
                    bf16* o = p.out + (size_t)m * p.ldo + (size_t)head * HD;
                    o[j] = __float2bfloat16_rn(y0);
                    o[j + half] = __float2bfloat16_rn(y1);
                } else {
                    const long long slot = p.slot_map[m];
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
            for (int e = threadIdx.x; e < HD * p.M; e += THREADS) {
                const int m = e / HD, j = e % HD;
                const long long slot = p.slot_map[m];
                if (slot < 0 || slot >= p.pool_slots) {
                    if (slot >= p.pool_slots) atomicOr(p.status, EG_STATUS_BAD_SLOT);
                    continue;
                }
                bf16* o = p.v_cache + (slot / p.page_size) * p.page_stride +
                          (long long)(head - p.num_heads - p.num_kv_heads) * p.head_stride + (slot % p.page_size) * HD;
                o[j] = __float2bfloat16_rn(value(j, m));
            }
        }
    }
}

template <int NT, int EPI, bool NORM>
int launch_one(cudaStream_t stream, const Params& p, int ctas) {
    const int MT = NT * 8;
    const size_t red_bytes = (size_t)8 * 16 * MT * sizeof(float);                 // RB*KS = 8 warps x 16 rows
    const size_t xs_bytes = NORM ? (size_t)MT * (((p.K * 2 + 127) / 128) * 128 + 64) : 0;
    const size_t smem_bytes = red_bytes > xs_bytes ? red_bytes : xs_bytes;
    if (smem_bytes > 200 * 1024) return (int)cudaErrorInvalidValue;
    auto kernel = skinny_kernel<NT, EPI, NORM>;
    static size_t configured = 0;
    if (smem_bytes > 48 * 1024 && smem_bytes > configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
        if (e != cudaSuccess) return (int)e;
        configured = smem_bytes;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.use_pdl ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, p);
}

template <int EPI, bool NORM>
int launch_nt(cudaStream_t stream, const Params& p, int ctas) {
    if (p.M <= 8) return launch_one<1, EPI, NORM>(stream, p, ctas);
    if (p.M <= 16) return launch_one<2, EPI, NORM>(stream, p, ctas);
    if (p.M <= 32) return launch_one<4, EPI, NORM>(stream, p, ctas);
    if (p.M <= 64) return launch_one<8, EPI, NORM>(stream, p, ctas);
    return (int)cudaErrorInvalidValue;
}

}  // namespace

// epilogue: 0 store bf16, 1 store f32, 2 swiglu (interleaved rows), 3 qkv + rope + cache (one CTA per head).
// norm != 0: x = gain * rmsnorm(resid_in + delta) (delta may be null), resid_out (may be null) receives the sum.
// row_blocks: 16-row blocks per CTA (1, 2, 4 or 8); the 8 warps of a CTA cover row_blocks x (8 / row_blocks) K slices.
// Takes M <= 64, K % 8 == 0, 16-byte aligned rows of W and x.  Anything else: cudaErrorInvalidValue.
EG_API int eg_gemm_skinny(cudaStream_t stream, int epilogue, int norm, int use_pdl, const void* W, long long ldw,
                          const float* bias, int M, int N, int K, const void* x, long long ldx, const float* resid_in,
                          float* resid_out, const void* delta, const float* gain, float eps, void* out, long long ldo,
                          int row_blocks, int num_heads, int num_kv_heads, int head_dim, const int* positions,
                          const int* slot_map, void* k_cache, void* v_cache, const float* inv_freq, int page_size,
                          long long page_stride, long long head_stride, long long pool_slots, int* status) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K % 8 || ldw % 8 || (!norm && ldx % 8) || (row_blocks != 1 && row_blocks != 2 && row_blocks != 4 && row_blocks != 8))
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
    p.status = status; p.RB = row_blocks; p.KS = 8 / row_blocks; p.use_pdl = use_pdl;
    const int ctas = (N + row_blocks * 16 - 1) / (row_blocks * 16);
#define EG_SKINNY(E)                                                                             \
    case E: return norm ? launch_nt<E, true>(stream, p, ctas) : launch_nt<E, false>(stream, p, ctas);
    switch (epilogue) {
        EG_SKINNY(EPI_STORE)
        EG_SKINNY(EPI_F32)
        EG_SKINNY(EPI_SWIGLU)
        EG_SKINNY(EPI_QKV_ROPE)
        default: return (int)cudaErrorInvalidValue;
    }
#undef EG_SKINNY
}
