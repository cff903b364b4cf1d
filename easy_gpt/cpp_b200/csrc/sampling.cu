// Sampling on float32 logits, one block per row.
//
// Greedy: the lowest index among the maxima (std::max_element over the
// probabilities in the reference, src/sampler.cpp:13-20; the softmax is
// monotonic, so the logits give the same token).
#include "common.cuh"

namespace {
constexpr int SAMPLE_THREADS = 1024;
constexpr int ARGMAX_THREADS = 256;      // a thread keeps four 16-byte loads in flight
}

struct ArgMax {
    float v;
    int i;
};

__device__ __forceinline__ ArgMax argmax_better(ArgMax a, ArgMax b) {
    // larger value wins; on a tie the lower index
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ __forceinline__ ArgMax block_argmax(ArgMax a, ArgMax* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b;
        b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
        a = argmax_better(a, b);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = a;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    ArgMax r;
    r.v = -INFINITY;
    r.i = 0x7fffffff;
    if (lane < nwarps) r = scratch[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b;
        b.v = __shfl_xor_sync(0xffffffffu, r.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, r.i, o);
        r = argmax_better(r, b);
    }
    return r;
}

// Several blocks share a row (one block cannot pull 600 KB of logits fast enough to
// matter beside a decode step); each writes its best (value, index) to scratch and the
// block that finishes last (a ticket counter; nobody waits) picks the row's winner.
__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_kernel(const float* __restrict__ logits, long long ld, int vocab, int* __restrict__ out,
              float* __restrict__ part_val, int* __restrict__ part_idx, int* __restrict__ counters) {
    __shared__ ArgMax scratch[32];
    __shared__ int is_last;
    const int r = blockIdx.x, nb = gridDim.y;
    const float* row = logits + (size_t)r * ld;
    const int per = (((vocab + nb - 1) / nb) + 3) & ~3;              // a multiple of 4, so that every block's stretch starts on 16 bytes
    const int lo = min(vocab, blockIdx.y * per), hi = min(vocab, lo + per);
    ArgMax best;
    best.v = -INFINITY;
    best.i = 0x7fffffff;
    auto take = [&](float v, int i) {
        ArgMax c;
        c.v = v;
        c.i = i;
        // NaN never wins; a row of NaNs yields index 0 below
        if (v == v) best = argmax_better(best, c);
    };
    int i0 = lo;
    if ((ld & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
        // (measured on B200, 64 rows of 151,936: 35.7 us with 4-byte loads, one in flight a thread)
        const float4* row4 = reinterpret_cast<const float4*>(row + lo);
        const int n4 = (hi - lo) / 4;
        constexpr int UNROLL = 4;
        for (int q0 = threadIdx.x; q0 < n4; q0 += blockDim.x * UNROLL) {
            float4 v[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int q = q0 + u * blockDim.x;
                if (q < n4) v[u] = row4[q];
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int q = q0 + u * blockDim.x;
                if (q < n4) {
                    const int i = lo + 4 * q;
                    take(v[u].x, i);
                    take(v[u].y, i + 1);
                    take(v[u].z, i + 2);
                    take(v[u].w, i + 3);
                }
            }
        }
        i0 = lo + 4 * n4;
    }
    for (int i = i0 + threadIdx.x; i < hi; i += blockDim.x) take(row[i], i);
    best = block_argmax(best, scratch);
    if (nb == 1) {
        if (threadIdx.x == 0) out[r] = best.i == 0x7fffffff ? 0 : best.i;
        return;
    }
    if (threadIdx.x == 0) {
        part_val[(size_t)r * nb + blockIdx.y] = best.v;
        part_idx[(size_t)r * nb + blockIdx.y] = best.i;
        __threadfence();
        const int ticket = atomicAdd(&counters[r], 1);
        is_last = ticket == nb - 1;
        if (is_last) counters[r] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    ArgMax a;
    a.v = -INFINITY;
    a.i = 0x7fffffff;
    if ((int)threadIdx.x < nb) {
        a.v = __ldcg(part_val + (size_t)r * nb + threadIdx.x);
        a.i = __ldcg(part_idx + (size_t)r * nb + threadIdx.x);
        if (a.i == 0x7fffffff) a.v = -INFINITY;
    }
    a = block_argmax(a, scratch);
    if (threadIdx.x == 0) out[r] = a.i == 0x7fffffff ? 0 : a.i;
}

// blocks_per_row > 1 needs part_val / part_idx (rows * blocks_per_row each) and counters (rows, zeroed; left zero).
EG_API int eg_argmax(cudaStream_t stream, const float* logits, long long ld, int rows, int vocab, int* out,
                     int blocks_per_row, float* part_val, int* part_idx, int* counters) {
    if (rows <= 0) return 0;
    if (blocks_per_row < 1 || blocks_per_row > ARGMAX_THREADS || (blocks_per_row > 1 && (!part_val || !part_idx || !counters)))
        return (int)cudaErrorInvalidValue;
    argmax_kernel<<<dim3(rows, blocks_per_row), ARGMAX_THREADS, 0, stream>>>(logits, ld, vocab, out, part_val, part_idx, counters);
    return eg_launch_status();
}

// ---------------------------------------------------------------------------
// Temperature / top-k / top-p sampling
// ---------------------------------------------------------------------------
// The rule is the reference's (src/sampler.cpp:39-106), restated on logits:
//   p_i  ∝ exp((x_i - max) / T)                      (p^(1/T) of the softmax, :50-58)
//   keep the top_k most probable if 0 < top_k < V     (:60-64), ties to the lower index
//   keep the shortest prefix of the descending order whose mass reaches top_p
//   of what is kept, at least one token, if 0 < top_p < 1   (:73-94)
//   draw by inverse CDF with one uniform number            (:96-105)
// Two things differ on purpose.  The uniform number comes from the host, keyed by
// (seed, request, token index), not from one generator shared by the batch; and the
// CDF is walked in index order over the kept tokens (the distribution is the same;
// no sort of the vocabulary is needed).  T <= 0 means greedy.
//
// Nothing here depends on the order in which threads run: the thresholds are found
// by bitwise search with block-wide sums of fixed shape, no floating-point atomics.
// One block per row; cost is a few dozen passes over the row from L2 when top-k or
// top-p is on, three passes when only the temperature is.

__device__ __forceinline__ unsigned int order_key(float x) {
    if (!(x == x)) return 0u;                                    // NaN sorts lowest
    const unsigned int b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float key_value(unsigned int k) {
    const unsigned int b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(b);
}

__device__ __forceinline__ int block_sum_int(int v, int* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    int r = (lane < (int)((blockDim.x + 31) >> 5)) ? scratch[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
}

__device__ __forceinline__ float block_max_float(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < (int)((blockDim.x + 31) >> 5)) ? scratch[lane] : -INFINITY;
    return warp_max(r);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long ld, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
              int* __restrict__ out) {
    __shared__ ArgMax arg_scratch[32];
    __shared__ float f_scratch[32];
    __shared__ int i_scratch[32];
    __shared__ float seg_mass[SAMPLE_THREADS];
    __shared__ int seg_eq[SAMPLE_THREADS];
    __shared__ int chosen;

    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    const float T = temperature[r];
    const int tid = threadIdx.x;

    if (!(T > 0.0f)) {                                           // greedy
        ArgMax best;
        best.v = -INFINITY;
        best.i = 0x7fffffff;
        for (int i = tid; i < vocab; i += blockDim.x) {
            ArgMax c;
            c.v = row[i];
            c.i = i;
            if (c.v == c.v) best = argmax_better(best, c);
        }
        best = block_argmax(best, arg_scratch);
        if (tid == 0) out[r] = best.i == 0x7fffffff ? 0 : best.i;
        return;
    }

    const float inv_t = 1.0f / fmaxf(T, 1e-6f);
    float mx = -INFINITY;
    for (int i = tid; i < vocab; i += blockDim.x) {
        const float x = row[i];
        if (x == x) mx = fmaxf(mx, x);
    }
    mx = block_max_float(mx, f_scratch);

    // ---- top-k: tk = key of the k-th largest logit; need_k of the tokens equal to it are kept
    const int k = top_k[r];
    unsigned int tk = 0u;
    int need_k = 0x7fffffff;
    if (k > 0 && k < vocab) {
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned int cand = tk | (1u << bit);
            int c = 0;
            for (int i = tid; i < vocab; i += blockDim.x) c += order_key(row[i]) >= cand;
            if (block_sum_int(c, i_scratch) >= k) tk = cand;
        }
        int gt = 0;
        for (int i = tid; i < vocab; i += blockDim.x) gt += order_key(row[i]) > tk;
        need_k = k - block_sum_int(gt, i_scratch);
    }
    // Key 0 is what NaN sorts as, below every real logit: it is never kept.  tk is 0 with top-k off,
    // and with top-k on when the row has fewer than k logits that are numbers.
    if (tk == 0u) {
        need_k = 0;
    } else {
        int eq_tk = 0;
        for (int i = tid; i < vocab; i += blockDim.x) eq_tk += order_key(row[i]) == tk;
        eq_tk = block_sum_int(eq_tk, i_scratch);
        need_k = min(need_k, eq_tk);
    }
    const float p_tk = need_k > 0 ? expf((key_value(tk) - mx) * inv_t) : 0.0f;

    // mass of the kept tokens whose key is >= t (t >= tk is what matters)
    auto mass_from = [&](unsigned int t) -> float {
        float s = 0.0f;
        for (int i = tid; i < vocab; i += blockDim.x) {
            const unsigned int key = order_key(row[i]);
            if (key >= t && key > tk) s += expf((row[i] - mx) * inv_t);
        }
        s = block_sum(s, f_scratch);
        if (t <= tk && need_k > 0) s += (float)need_k * p_tk;
        return s;
    };

    // ---- top-p: thr = lowest key kept, n_eq = how many of the tokens equal to it are kept
    unsigned int thr = tk;
    int n_eq = need_k;
    const float pp = top_p[r];
    if (pp > 0.0f && pp < 1.0f) {
        const float target = pp * mass_from(tk);
        unsigned int t = 0u;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned int cand = t | (1u << bit);
            if (mass_from(cand) >= target) t = cand;
        }
        if (t < tk) t = tk;
        int avail;
        if (t == tk) {
            avail = need_k;
        } else {
            int c = 0;
            for (int i = tid; i < vocab; i += blockDim.x) c += order_key(row[i]) == t;
            avail = block_sum_int(c, i_scratch);
        }
        const float above = (t == 0xffffffffu) ? 0.0f : mass_from(t + 1u);
        const float p_eq = expf((key_value(t) - mx) * inv_t);
        int n = (p_eq > 0.0f) ? (int)ceilf((target - above) / p_eq) : avail;
        n = max(1, min(n, avail));
        thr = t;
        n_eq = n;
    }

    // ---- draw: inverse CDF in index order over {key > thr} and the first n_eq of {key == thr}
    const int seg = (vocab + blockDim.x - 1) / blockDim.x;
    const int lo = min(vocab, tid * seg), hi = min(vocab, lo + seg);
    int eq_here = 0;
    for (int i = lo; i < hi; ++i) eq_here += order_key(row[i]) == thr;
    seg_eq[tid] = eq_here;
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int j = 0; j < (int)blockDim.x; ++j) {
            const int c = seg_eq[j];
            seg_eq[j] = run;
            run += c;
        }
    }
    __syncthreads();
    int eq_rank = seg_eq[tid];
    float mass_here = 0.0f;
    for (int i = lo; i < hi; ++i) {
        const unsigned int key = order_key(row[i]);
        if (key > thr || (key == thr && eq_rank < n_eq)) mass_here += expf((row[i] - mx) * inv_t);
        eq_rank += key == thr;
    }
    seg_mass[tid] = mass_here;
    if (tid == 0) chosen = -1;
    __syncthreads();
    if (tid == 0) {
        float run = 0.0f;
        for (int j = 0; j < (int)blockDim.x; ++j) {
            const float c = seg_mass[j];
            seg_mass[j] = run;
            run += c;
        }
        f_scratch[0] = run;                                      // total mass of the kept set
    }
    __syncthreads();
    const float total = f_scratch[0];
    const float target = uniform[r] * total;
    const float before = seg_mass[tid];
    const float after = (tid + 1 < (int)blockDim.x) ? seg_mass[tid + 1] : total;
    int last_kept = -1;
    {
        float run = before;
        int rank = seg_eq[tid];
        const bool mine = target >= before && target < after;
        for (int i = lo; i < hi; ++i) {
            const unsigned int key = order_key(row[i]);
            const bool kept = key > thr || (key == thr && rank < n_eq);
            rank += key == thr;
            if (!kept) continue;
            last_kept = i;
            run += expf((row[i] - mx) * inv_t);
            if (mine && target < run) {
                chosen = i;                                      // only one thread has `mine`
                break;
            }
        }
        if (mine && chosen < 0 && last_kept >= 0) chosen = last_kept;   // rounding at the segment's end
    }
    // rounding at the very end of the CDF: the last kept token of the row
    __syncthreads();
    if (chosen < 0) {
        int best = last_kept;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
        if ((tid & 31) == 0) i_scratch[tid >> 5] = best;
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < (int)((blockDim.x + 31) >> 5); ++w) best = max(best, i_scratch[w]);
            out[r] = max(0, best);
        }
    } else if (tid == 0) {
        out[r] = chosen;
    }
}

EG_API int eg_sample(cudaStream_t stream, const float* logits, long long ld, int rows, int vocab, const float* temperature,
                     const int* top_k, const float* top_p, const float* uniform, int* out) {
    if (rows <= 0) return 0;
    sample_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, ld, vocab, temperature, top_k, top_p, uniform, out);
    return eg_launch_status();
}
