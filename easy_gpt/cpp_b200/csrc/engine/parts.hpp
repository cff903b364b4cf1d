// The parts the engine ships: grouped-query attention over the paged cache, the SwiGLU feed-forward, RMSNorm,
// the rotary position encoding, the token embedding and the output head, and the linear product they share.
// Formulas and their order are the reference's (cited at each part); sizes and constants are parameters.
#pragma once
#include <cmath>
#include <cstring>

#include "parts_base.hpp"

namespace easygpt::engine {

// ---- host-side assembly of weights ---------------------------------------------------------------------------
inline std::vector<float> host_floats(const StoredTensor& t) {
    std::vector<float> out((size_t)t.numel());
    t.to_float(out.data());
    return out;
}
inline const StoredTensor& need_tensor(const HostTensors& file, const std::string& name) {
    const StoredTensor* t = file.find(name);
    if (!t) throw WeightError("Missing required model weights: " + name);
    return *t;
}
// float32 values -> device memory in `dtype` (bfloat16: round to nearest even)
inline DeviceBuffer upload(const float* values, size_t n, DType dtype) {
    DeviceBuffer buf(n * dtype_size(dtype));
    if (dtype == DType::F32) {
        EG_CUDA(cudaMemcpy(buf.get(), values, n * 4, cudaMemcpyHostToDevice));
    } else {
        std::vector<uint16_t> low(n);
        for (size_t i = 0; i < n; ++i) low[i] = float_to_bf16(values[i]);
        EG_CUDA(cudaMemcpy(buf.get(), low.data(), n * 2, cudaMemcpyHostToDevice));
    }
    return buf;
}
// a stored tensor as it is, where its stored precision is the wanted one (no round trip through float32)
inline DeviceBuffer upload(const StoredTensor& t, DType dtype) {
    if ((t.dtype == Stored::BF16 && dtype == DType::BF16) || (t.dtype == Stored::F32 && dtype == DType::F32)) {
        DeviceBuffer buf(t.bytes);
        EG_CUDA(cudaMemcpy(buf.get(), t.data, t.bytes, cudaMemcpyHostToDevice));
        return buf;
    }
    const std::vector<float> f = host_floats(t);
    return upload(f.data(), f.size(), dtype);
}

// ---- y = x W^T + b with W stored [out, in] (src/models/linear.cpp:42-44) ------------------------------------------
// In bfloat16, steps of up to 16 tokens go to the engine's own weight-streaming kernel (gemm_skinny.cu); larger ones
// to the library product (cuBLAS), where the reference's engine calls cublasGemmEx too (src/cuda/ops/matmul.cu:194-204).
// In float32 it is always the engine's own FFMA kernel: true 32-bit arithmetic whose sums do not depend on the batch.
struct SkinnyRope {
    int num_heads, num_kv_heads, head_dim;
    const int *positions, *slot_map;
    void *k_cache, *v_cache;
    const float* inv_freq;
    int page_size;
    long long page_stride, head_stride, pool_slots;
};

class Linear {
public:
    Linear() = default;
    Linear(const float* w, int out_features, int in_features, const float* bias, DType dtype)
        : out_features(out_features), in_features(in_features), dtype(dtype) {
        store_ = upload(w, (size_t)out_features * in_features, dtype);
        weight = store_.get();
        set_bias(bias);
    }
    Linear(const StoredTensor& w, const float* bias, DType dtype)
        : out_features((int)w.shape[0]), in_features((int)w.shape[1]), dtype(dtype) {
        store_ = upload(w, dtype);
        weight = store_.get();
        set_bias(bias);
    }
    // a bias-free product with a weight that another part owns (a tied head multiplies by the embedding table itself)
    static Linear sharing(const void* weight, int out_features, int in_features, DType dtype) {
        Linear l;
        l.weight = weight;
        l.out_features = out_features;
        l.in_features = in_features;
        l.dtype = dtype;
        return l;
    }
    size_t weight_bytes() const { return (size_t)out_features * in_features * dtype_size(dtype); }

    static bool aligned(const Rows& x) { return x.ld % 8 == 0 && (uintptr_t)x.p % 16 == 0; }

    // the decode product with every prologue and epilogue it has; see csrc/gemm_skinny.cu
    void skinny(const StepContext& ctx, int epilogue, int M, const Rows* x, const NormInFront* norm, void* out, long long ldo,
                const SkinnyRope* rope, float* follow_residual, const float* follow_gain, void* xn_out, float* ss_out,
                const plans::SkinnyPlan* plan_override = nullptr) const {
        const int N = out_features, K = in_features;
        const plans::SkinnyPlan plan = plan_override ? *plan_override : plans::skinny_plan(N, K, rope ? rope->head_dim : 0);
        int norm_mode = 0;
        const void* delta = nullptr;
        const float *resid_in = nullptr, *gain = nullptr, *ss_in = nullptr;
        float* resid_out = nullptr;
        float eps = 0.f;
        int ss_parts = 0;
        if (norm) {
            eps = norm->eps;
            if (norm->prepared_rows) {
                norm_mode = 2;
                delta = norm->prepared_rows;
                ss_in = norm->prepared_sums;
                ss_parts = norm->prepared_parts;
            } else {
                norm_mode = 1;
                resid_in = norm->residual;
                resid_out = norm->residual_out;
                delta = norm->delta;
                gain = norm->gain;
            }
        }
        float* partials = nullptr;
        int* counters = nullptr;
        if (plan.k_split > 1) {
            const size_t groups = (size_t)(N + plan.row_blocks * 16 - 1) / (plan.row_blocks * 16);
            const size_t floats = (size_t)plan.k_split * groups * plan.row_blocks * 16 * plans::skinny_padded_tokens(M);
            if (floats > KernelScratch::SKINNY_FLOATS || groups > KernelScratch::SKINNY_COUNTERS)
                throw DeviceError("a decode product's split needs more scratch memory than the engine holds");
            partials = ctx.scratch->skinny_partials.as<float>();
            counters = ctx.scratch->skinny_counters.as<int>();
        }
        SkinnyRope none{};
        const SkinnyRope& r = rope ? *rope : none;
        launch_check(eg_gemm_skinny(ctx.stream, epilogue, norm_mode, plans::use_pdl(), weight, in_features, bias_f32(), M, N, K,
                                    x ? x->p : nullptr, x ? x->ld : 0, resid_in, resid_out, delta, gain, eps, out, ldo, plan.row_blocks,
                                    plan.k_slices, plan.k_split, partials, counters, r.num_heads, r.num_kv_heads, r.head_dim, r.positions,
                                    r.slot_map, r.k_cache, r.v_cache, r.inv_freq, r.page_size, r.page_stride, r.head_stride, r.pool_slots,
                                    ctx.status, nullptr, 0, nullptr, ss_in, ss_parts, follow_residual, follow_gain, xn_out, ss_out),
                     "gemm_skinny");
    }

    // whether with_following_norm can run for this input (the decode kernel takes it)
    bool takes_following_norm(const Rows& x) const {
        return dtype == DType::BF16 && plans::gemm_skinny_takes(dtype, x.rows, in_features) && x.rows <= plans::FUSED_NORM_MAX_TOKENS && aligned(x);
    }
    // The product, the add to the residual and the preparation of the norm that follows, in one kernel:
    // follow.residual() += x W^T + b (in place); returns a PreNormed for follow.norm.
    PreNormed with_following_norm(const StepContext& ctx, const Rows& x, const FollowingNorm& follow) const {
        const plans::SkinnyPlan plan = plans::skinny_plan(out_features, in_features);
        const int parts = (out_features + plan.row_blocks * 16 - 1) / (plan.row_blocks * 16);
        void* xn = ctx.take_rows(x.rows, out_features, DType::BF16);
        float* ss = ctx.take<float>((size_t)parts * plans::skinny_padded_tokens(x.rows));
        skinny(ctx, plans::EPI_RESID_NORM, x.rows, &x, nullptr, nullptr, 0, nullptr, follow.residual(), follow.gain, xn, ss, &plan);
        return PreNormed{follow.norm, xn, ss, parts};
    }

    // out [M, out_features] from the arena, in the compute dtype or (out_f32) in float32
    Rows operator()(const StepContext& ctx, const Rows& x, bool out_f32 = false) const {
        const int M = x.rows;
        Rows out{nullptr, (out_f32 || dtype == DType::F32) ? DType::F32 : DType::BF16, M, out_features, out_features};
        out.p = ctx.take_rows(M, out_features, out.dtype);
        if (dtype == DType::F32) {
            launch_check(eg_gemm_f32_nt(ctx.stream, (const float*)x.p, (int)x.ld, (const float*)weight, in_features, bias_f32(), (float*)out.p,
                                        out_features, M, out_features, in_features), "gemm_f32_nt");
            return out;
        }
        if (plans::gemm_skinny_takes(dtype, M, in_features) && aligned(x)) {
            skinny(ctx, out_f32 ? plans::EPI_F32 : plans::EPI_STORE, M, &x, nullptr, out.p, out_features, nullptr, nullptr, nullptr, nullptr, nullptr);
            return out;
        }
        if (out_f32 && has_bias()) throw DeviceError("a library product into float32 takes no bias");
        ctx.blas->gemm_bf16(ctx.stream, x.p, x.ld, weight, in_features, has_bias() ? bias_lp_.get() : nullptr, out.p, out_features, M, out_features,
                            in_features, out_f32);
        return out;
    }

    const float* bias_f32() const { return bias_f32_.get() ? bias_f32_.as<float>() : nullptr; }
    bool has_bias() const { return bias_f32_.get() != nullptr; }

    const void* weight = nullptr;
    int out_features = 0, in_features = 0;
    DType dtype = DType::BF16;

private:
    void set_bias(const float* bias) {
        if (!bias) return;
        // the bias is added in float32 by our kernels; the library product wants it in its own dtype
        bias_f32_ = upload(bias, (size_t)out_features, DType::F32);
        if (dtype == DType::BF16) bias_lp_ = upload(bias, (size_t)out_features, DType::BF16);
    }
    DeviceBuffer store_, bias_f32_, bias_lp_;
};

// ---- RMSNorm: y = w * (x / sqrt(mean(x^2) + eps)) (src/models/norm.cpp:46-60), eps a parameter (the reference fixes
// 1e-6, src/models/norm.cpp:41), fused with the float32 residual add ---------------------------------------------------
class RMSNorm : public Norm {
public:
    RMSNorm(const Params& p, const std::string& prefix) : Norm(p, prefix), size_((int)p.integer("size")), eps_((float)p.real("eps")) {}
    std::vector<TensorRequest> tensor_requests() const override { return {TensorRequest::vector(prefix + ".weight", size_)}; }
    void load(const HostTensors& file, DType) override {
        const std::vector<float> g = host_floats(need_tensor(file, prefix + ".weight"));       // gains are used in float32 whatever they were stored in
        gain_ = upload(g.data(), g.size(), DType::F32);
    }
    size_t weight_bytes() const override { return (size_t)size_ * 4; }
    bool capturable() const override { return true; }
    bool rms_parameters(const float** gain, float* eps) const override {
        *gain = gain_.as<float>();
        *eps = eps_;
        return true;
    }
    void forward(const StepContext& ctx, float* residual, const void* delta, DType delta_dtype, void* out, DType out_dtype, int num_rows,
                 const int* rows) const override {
        launch_check(eg_add_rmsnorm(ctx.stream, (int)(delta ? delta_dtype : out_dtype), (int)out_dtype, residual, delta, rows, gain_.as<float>(), out,
                                    num_rows, size_, eps_), "add_rmsnorm");
    }
    int size() const override { return size_; }

private:
    int size_;
    float eps_;
    DeviceBuffer gain_;
};

// ---- rotary position encoding, half rotation over rotary_dim dimensions of each head (src/ops.cpp:404-421).  The table
// inv_freq[k] = theta^(-2k/rotary_dim) (src/ops.cpp:172-177) is built once on the host, in double, rounded to float32 -----
class RotaryEncoding : public PositionEncoding {
public:
    RotaryEncoding(const Params& p, const std::string& prefix)
        : PositionEncoding(p, prefix), head_dim_((int)p.integer("head_dim")), rotary_dim_((int)p.integer("rotary_dim", p.integer("head_dim"))),
          theta_(p.real("theta")) {
        if (rotary_dim_ % 2 || rotary_dim_ <= 0 || rotary_dim_ > head_dim_)
            throw std::invalid_argument("rotary_dim " + std::to_string(rotary_dim_) + " must be even and within head_dim " + std::to_string(head_dim_));
        if (theta_ <= 0) throw std::invalid_argument("rope theta must be > 0");
    }
    void load(const HostTensors&, DType) override {
        std::vector<float> inv(rotary_dim_ / 2);
        for (int k = 0; k < rotary_dim_ / 2; ++k) inv[k] = (float)(1.0 / std::pow(theta_, 2.0 * k / rotary_dim_));
        inv_freq_ = upload(inv.data(), inv.size(), DType::F32);
    }
    bool capturable() const override { return true; }
    bool half_rotation(HalfRotation* out) const override {
        out->inv_freq = inv_freq_.as<float>();
        out->rotary_dim = rotary_dim_;
        out->key = "rope:" + std::to_string(theta_) + ":" + std::to_string(rotary_dim_);
        return true;
    }

private:
    int head_dim_, rotary_dim_;
    double theta_;
    DeviceBuffer inv_freq_;
};

// ---- grouped-query attention over the paged cache -----------------------------------------------------------------
// Per token: q, k, v = x Wq^T + bq, ... (src/models/self_attn.cpp:225-227) as ONE product with the three weights
// stacked; q and k are changed by the layer's position encoding (a half rotation is applied by the kernel that also
// stores k, v in the cache; another encoding changes q and k itself; none is fine too); every query head h attends
// the keys of KV head h / (NH/NKV) of its own request up to its own position (optionally only the last `window` of
// them); the heads are concatenated head-major and projected by Wo (src/models/self_attn.cpp:255-258).  Scale
// 1/sqrt(head_dim) (:253).  Parameters: hidden_size, num_heads, num_kv_heads, head_dim, qkv_bias, out_bias, window.
class Attention : public Mixer {
public:
    Attention(const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> position)
        : Mixer(p, prefix, std::move(position)), hidden_((int)p.integer("hidden_size")), heads_((int)p.integer("num_heads")),
          kv_heads_((int)p.integer("num_kv_heads")), head_dim_((int)p.integer("head_dim")), qkv_bias_(p.flag("qkv_bias", false)),
          out_bias_(p.flag("out_bias", false)), window_(p.has("window") ? p.integer("window") : -1) {
        if (heads_ % kv_heads_) throw std::invalid_argument("num_heads must be a multiple of num_kv_heads");
        if (p.has("window") && window_ <= 0) throw std::invalid_argument("window must be positive");
        if (head_dim_ <= 0 || head_dim_ > plans::MAX_HEAD_DIM)
            throw std::invalid_argument("head_dim " + std::to_string(head_dim_) + " is outside what the attention kernels take (1.." +
                                        std::to_string(plans::MAX_HEAD_DIM) + ")");
        scale_ = (float)(1.0 / std::sqrt((double)head_dim_));
    }
    std::vector<TensorRequest> tensor_requests() const override {
        const long long q_out = (long long)heads_ * head_dim_, kv_out = (long long)kv_heads_ * head_dim_;
        std::vector<TensorRequest> r = {TensorRequest::matrix(prefix + ".q_proj.weight", q_out, hidden_), TensorRequest::matrix(prefix + ".k_proj.weight", kv_out, hidden_),
                                        TensorRequest::matrix(prefix + ".v_proj.weight", kv_out, hidden_), TensorRequest::matrix(prefix + ".o_proj.weight", hidden_, q_out)};
        if (qkv_bias_) {
            r.push_back(TensorRequest::vector(prefix + ".q_proj.bias", q_out));
            r.push_back(TensorRequest::vector(prefix + ".k_proj.bias", kv_out));
            r.push_back(TensorRequest::vector(prefix + ".v_proj.bias", kv_out));
        }
        if (out_bias_) r.push_back(TensorRequest::vector(prefix + ".o_proj.bias", hidden_));
        return r;
    }
    void load(const HostTensors& file, DType dtype) override {
        std::vector<float> w, b;
        for (const char* n : {"q", "k", "v"}) {
            const std::vector<float> part = host_floats(need_tensor(file, prefix + "." + n + "_proj.weight"));
            w.insert(w.end(), part.begin(), part.end());
            if (qkv_bias_) {
                const std::vector<float> bias = host_floats(need_tensor(file, prefix + "." + n + "_proj.bias"));
                b.insert(b.end(), bias.begin(), bias.end());
            }
        }
        const int rows = (heads_ + 2 * kv_heads_) * head_dim_;
        qkv_ = Linear(w.data(), rows, hidden_, qkv_bias_ ? b.data() : nullptr, dtype);
        std::vector<float> ob;
        if (out_bias_) ob = host_floats(need_tensor(file, prefix + ".o_proj.bias"));
        out_ = Linear(need_tensor(file, prefix + ".o_proj.weight"), out_bias_ ? ob.data() : nullptr, dtype);
        if (position) position->load(file, dtype);
    }
    size_t weight_bytes() const override { return qkv_.weight_bytes() + out_.weight_bytes(); }
    bool capturable() const override { return true; }
    CacheNeed cache_need() const override { return CacheNeed::paged(kv_heads_, head_dim_, window_); }
    bool accepts_pending_norm() const override { return true; }
    bool fuses_following_norm() const override { return true; }

    // norm + QKV (+ bias, rotation, cache write); attention over the cache; output projection into the residual
    bool emit_fused(FusedBuilder& b, const float* gain, float eps, const CacheView& cache) const override {
        const StepContext& ctx = *b.ctx;
        HalfRotation rot;
        const bool rotates = position && position->half_rotation(&rot);
        const int G = heads_ / kv_heads_;
        if (ctx.dtype != DType::BF16 || head_dim_ != 64 || G > 16 || cache.group < 0 || !cache.writes || cache.page_size % 16 || hidden_ != b.hidden) return false;
        if (position && (!rotates || rot.rotary_dim != head_dim_)) return false;
        const GroupTables& tables = ctx.groups.at(cache.group);
        const int q_width = heads_ * head_dim_, T = b.tokens;
        void* q = b.arena->take((size_t)T * q_width * 2);
        void* attn = b.arena->take((size_t)T * q_width * 2);
        EgFusedTemplate t = FusedBuilder::blank();
        t.input = EGF_IN_NORM;
        t.output = EGF_OUT_QKV_ROPE;
        t.N = (heads_ + 2 * kv_heads_) * head_dim_;
        t.K = hidden_;
        t.tiles_per_unit = 2;
        t.group_rows = head_dim_;
        t.units_per_group = head_dim_ / 16;
        t.pair_offset = head_dim_ / 2;
        t.eps = eps;
        t.out = q;
        t.ldo = q_width;
        t.num_heads = heads_;
        t.num_kv_heads = kv_heads_;
        t.head_dim = head_dim_;
        t.page_size = cache.page_size;
        t.num_pages = cache.num_pages;
        t.positions = ctx.positions;
        t.slot_map = tables.slot_map;
        t.inv_freq = rotates ? rot.inv_freq : nullptr;
        t.page_stride = cache.page_stride;
        t.head_stride = cache.head_stride;
        t.pool_slots = (long long)cache.num_pages * cache.page_size;
        if (!b.linear(t, qkv_.weight, hidden_, qkv_.bias_f32(), gain, cache.k, cache.v)) return false;

        // as many CTAs per (token, KV head) as the grid has for them, a key tile each at least
        const long long longest = window_ < 0 ? ctx.max_context_len : std::min<long long>(ctx.max_context_len, window_ + 255);
        const int tiles = (int)std::max<long long>(1, (longest + 63) / 64);
        // (at most 16, and four tiles each where there are that many: the merge of the splits is one CTA's work)
        const int splits = std::max(1, std::min({std::max(1, tiles / 4), 16, b.grid / std::max(1, T * kv_heads_)}));
        EgFusedTemplate a = FusedBuilder::blank();
        a.num_heads = heads_;
        a.num_kv_heads = kv_heads_;
        a.head_dim = head_dim_;
        a.page_size = cache.page_size;
        a.num_pages = cache.num_pages;
        a.window = window_ < 0 ? 0 : (int)window_;
        a.positions = ctx.positions;
        a.page_stride = cache.page_stride;
        a.head_stride = cache.head_stride;
        a.q = q;
        a.ldq = q_width;
        a.block_table = tables.block_table;
        a.table_stride = tables.table_width;
        a.seq_context = ctx.seq_context;
        a.scale = scale_;
        a.splits = splits;
        if (splits > 1) {
            if ((size_t)T * kv_heads_ > KernelScratch::ATTENTION_COUNTERS) return false;
            a.partial_acc = b.arena->take_n<float>((size_t)T * heads_ * splits * head_dim_);
            a.partial_ml = b.arena->take_n<float>((size_t)T * heads_ * splits * 2);
            a.tickets = ctx.scratch->attention_counters.as<int>();
        }
        a.attn_out = attn;
        a.ld_attn = q_width;
        b.attention(a, cache.k, cache.v);

        EgFusedTemplate o = FusedBuilder::blank();
        o.input = EGF_IN_ROWS;
        o.output = EGF_OUT_RESIDUAL;
        o.N = hidden_;
        o.K = q_width;
        o.tiles_per_unit = 1;
        o.group_rows = 8;
        o.units_per_group = 1;
        o.x = attn;
        o.ldx = q_width;
        return b.linear(o, out_.weight, q_width, out_.bias_f32(), nullptr);
    }

    Delta forward(const StepContext& ctx, PartInput in, const CacheView& cache, const FollowingNorm* follow) override {
        const int T = ctx.num_tokens;
        const GroupTables& tables = ctx.groups.at(cache.group);
        const DType dtype = ctx.dtype;
        const int q_width = heads_ * head_dim_, kv_width = kv_heads_ * head_dim_;
        const long long pool_slots = (long long)cache.num_pages * cache.page_size;
        HalfRotation rot;
        const bool rotates = position && position->half_rotation(&rot);
        Rows qkv;
        if (in.pending && in.pending->fusable && cache.writes && rotates && rot.rotary_dim == head_dim_ &&
            (head_dim_ == 16 || head_dim_ == 32 || head_dim_ == 64 || head_dim_ == 128)) {
            // decode: add + norm + QKV product + bias + rotation + cache write in one kernel
            qkv = Rows{ctx.take_rows(T, q_width, dtype), dtype, T, q_width, q_width};
            const NormInFront norm = in.pending->fused();
            const SkinnyRope rope{heads_, kv_heads_, head_dim_, ctx.positions, tables.slot_map, cache.k, cache.v, rot.inv_freq, cache.page_size,
                                  cache.page_stride, cache.head_stride, pool_slots};
            qkv_.skinny(ctx, plans::EPI_QKV_ROPE, T, nullptr, &norm, qkv.p, q_width, &rope, nullptr, nullptr, nullptr, nullptr);
        } else {
            const Rows x = in.pending ? in.pending->materialize() : in.rows;
            qkv = qkv_(ctx, x);
            const int* slot_map = cache.writes ? tables.slot_map : nullptr;
            void* kc = cache.writes ? cache.k : nullptr;
            void* vc = cache.writes ? cache.v : nullptr;
            if (rotates && rot.rotary_dim == head_dim_ && head_dim_ % (dtype == DType::BF16 ? 16 : 8) == 0) {      // halves of a head in 16-byte pieces
                launch_check(eg_rope_cache_vec(ctx.stream, (int)dtype, qkv.p, (int)qkv.ld, rotation_table(ctx, rot), slot_map, kc, vc, T, heads_, kv_heads_,
                                               head_dim_, cache.page_size, cache.page_stride, cache.head_stride, slot_map ? pool_slots : 0, ctx.status),
                             "rope_cache_table");
            } else {
                if (!rotates && position) {
                    char* base = (char*)qkv.p;
                    position->apply_to_query_key(base, base + (size_t)q_width * dtype_size(dtype), qkv.ld, heads_, kv_heads_, head_dim_, ctx);
                }
                launch_check(eg_rope_cache(ctx.stream, (int)dtype, qkv.p, (int)qkv.ld, nullptr, ctx.positions, slot_map, kc, vc,
                                           rotates ? rot.inv_freq : nullptr, T, heads_, kv_heads_, head_dim_, rotates ? rot.rotary_dim : 0,
                                           cache.page_size, cache.page_stride, cache.head_stride, slot_map ? pool_slots : 0, ctx.status),
                             "rope_cache");
            }
        }
        (void)kv_width;
        Rows attn{ctx.take_rows(T, q_width, dtype), dtype, T, q_width, q_width};
        const long long longest = window_ < 0 ? ctx.max_context_len : std::min<long long>(ctx.max_context_len, window_ + 255);
        const int window = window_ < 0 ? 0 : (int)window_;
        if (ctx.query_tiles && plans::attention_prefill_takes(dtype, head_dim_, cache.page_size)) {
            // prompt portions: tiles of query tokens against the cache, on the tcgen05 tensor cores when the portions are
            // long enough to fill their 128-row tiles
            if (ctx.max_query_len >= plans::TCGEN05_ATTENTION_MIN_QUERY && plans::attention_prefill_tcgen05_takes(dtype, head_dim_, cache.page_size)) {
                int parts, part_tiles;
                plans::attention_prefill_parts(ctx.num_tiles, heads_, head_dim_, longest, &parts, &part_tiles);
                const size_t slots = (size_t)ctx.num_tiles * heads_;
                while (parts > 1 && slots * parts * 128 * (head_dim_ + 2) * 4 > plans::PREFILL_PARTS_SCRATCH_BYTES) --parts;
                float *partial_o = nullptr, *partial_ml = nullptr;
                if (parts > 1) {
                    partial_o = ctx.take<float>(slots * parts * 128 * head_dim_);
                    partial_ml = ctx.take<float>(slots * parts * 128 * 2);
                }
                launch_check(eg_attention_prefill_tcgen05(ctx.stream, qkv.p, qkv.ld, T, cache.k, cache.v, tables.block_table, tables.table_width,
                                                          ctx.positions, ctx.query_tiles, ctx.num_tiles, attn.p, attn.ld, heads_, kv_heads_, head_dim_,
                                                          cache.page_size, cache.page_stride, cache.head_stride, cache.num_pages, window, scale_,
                                                          ctx.status, nullptr, parts, part_tiles, partial_o, partial_ml,
                                                          ctx.scratch->prefill_queue.as<int>()), "attention_prefill_tcgen05");
            } else {
                launch_check(eg_attention_prefill(ctx.stream, qkv.p, (int)qkv.ld, cache.k, cache.v, tables.block_table, tables.table_width, ctx.positions,
                                                  ctx.query_tiles, ctx.num_tiles, attn.p, (int)attn.ld, heads_, kv_heads_, head_dim_, cache.page_size,
                                                  cache.page_stride, cache.head_stride, cache.num_pages, window, scale_, ctx.status), "attention_prefill");
            }
            if (ctx.small_tokens)      // the decoded tokens beside them: token by token, split over their keys
                paged(ctx, qkv, cache, tables, attn, ctx.num_small, plans::attention_paged_splits(ctx.num_small, heads_, kv_heads_, longest, head_dim_), window,
                      nullptr, ctx.small_tokens);
        } else if (plans::attention_paged_takes(dtype, head_dim_, cache.page_size)) {
            paged(ctx, qkv, cache, tables, attn, T, plans::attention_paged_splits(T, heads_, kv_heads_, longest, head_dim_), window, ctx.seq_context, nullptr);
        } else {
            launch_check(eg_attention_generic(ctx.stream, (int)dtype, qkv.p, (int)qkv.ld, cache.k, cache.v, tables.block_table, tables.table_width,
                                              ctx.token_seq, ctx.positions, attn.p, (int)attn.ld, T, heads_, kv_heads_, head_dim_, cache.page_size,
                                              cache.page_stride, cache.head_stride, cache.num_pages, window, scale_, ctx.status), "attention_generic");
        }
        Delta d;
        if (follow && out_.takes_following_norm(attn)) {
            d.pre = out_.with_following_norm(ctx, attn, *follow);
            return d;
        }
        const Rows o = out_(ctx, attn);
        d.p = o.p;
        d.dtype = o.dtype;
        return d;
    }

private:
    // cos/sin [T, rotary_dim/2, 2] of this step's positions: computed by the first layer that asks and shared by every
    // layer whose rotation has the same key
    static const float* rotation_table(const StepContext& ctx, const HalfRotation& rot) {
        auto& shared = const_cast<StepContext&>(ctx).shared;
        const std::string key = "rotation table " + rot.key;
        auto it = shared.find(key);
        if (it != shared.end()) return (const float*)it->second;
        float* table = ctx.take_for_step<float>((size_t)ctx.num_tokens * rot.rotary_dim);
        launch_check(eg_rope_table(ctx.stream, ctx.positions, rot.inv_freq, table, ctx.num_tokens, rot.rotary_dim / 2), "rope_table");
        shared[key] = table;
        return table;
    }
    void paged(const StepContext& ctx, const Rows& qkv, const CacheView& cache, const GroupTables& tables, const Rows& attn, int tokens, int splits,
               int window, const int* seq_context, const int* token_list) const {
        float *acc = nullptr, *ml = nullptr;
        int* counters = nullptr;
        if (splits > 1) {
            const size_t T = (size_t)ctx.num_tokens;
            acc = ctx.take<float>(T * heads_ * splits * head_dim_);
            ml = ctx.take<float>(T * heads_ * splits * 2);
            if ((size_t)tokens * kv_heads_ * ((heads_ / kv_heads_ + 15) / 16) > KernelScratch::ATTENTION_COUNTERS)
                throw DeviceError("a step has more (token, KV head) pairs than the attention's ticket counters");
            counters = ctx.scratch->attention_counters.as<int>();
        }
        launch_check(eg_attention_paged(ctx.stream, qkv.p, (int)qkv.ld, cache.k, cache.v, tables.block_table, tables.table_width, ctx.token_seq,
                                        ctx.positions, seq_context, attn.p, (int)attn.ld, acc, ml, tokens, heads_, kv_heads_, head_dim_, cache.page_size,
                                        cache.page_stride, cache.head_stride, cache.num_pages, window, scale_, splits, ctx.status, nullptr, 0, counters,
                                        plans::use_pdl(), nullptr, token_list), "attention_paged");
    }

    int hidden_, heads_, kv_heads_, head_dim_;
    bool qkv_bias_, out_bias_;
    long long window_;
    float scale_;
    Linear qkv_, out_;
};

// ---- SwiGLU feed-forward: down( up(x) * silu(gate(x)) ) (src/models/mlp.cpp:41-49).  gate and up become one product whose
// weight rows are interleaved (gate_0, up_0, gate_1, up_1, ...), so that every tile of the product holds both halves of the
// outputs it covers and the activation can run in the product's epilogue.  Parameters: hidden_size, intermediate_size, bias ---
class SwiGLU : public FeedForward {
public:
    SwiGLU(const Params& p, const std::string& prefix)
        : FeedForward(p, prefix), hidden_((int)p.integer("hidden_size")), inter_((int)p.integer("intermediate_size")), bias_(p.flag("bias", false)) {}
    std::vector<TensorRequest> tensor_requests() const override {
        std::vector<TensorRequest> r = {TensorRequest::matrix(prefix + ".gate_proj.weight", inter_, hidden_), TensorRequest::matrix(prefix + ".up_proj.weight", inter_, hidden_),
                                        TensorRequest::matrix(prefix + ".down_proj.weight", hidden_, inter_)};
        if (bias_) {
            r.push_back(TensorRequest::vector(prefix + ".gate_proj.bias", inter_));
            r.push_back(TensorRequest::vector(prefix + ".up_proj.bias", inter_));
            r.push_back(TensorRequest::vector(prefix + ".down_proj.bias", hidden_));
        }
        return r;
    }
    void load(const HostTensors& file, DType dtype) override {
        const std::vector<float> gate = host_floats(need_tensor(file, prefix + ".gate_proj.weight")), up = host_floats(need_tensor(file, prefix + ".up_proj.weight"));
        std::vector<float> w((size_t)2 * inter_ * hidden_), b;
        for (int i = 0; i < inter_; ++i) {
            std::memcpy(&w[(size_t)(2 * i) * hidden_], &gate[(size_t)i * hidden_], (size_t)hidden_ * 4);
            std::memcpy(&w[(size_t)(2 * i + 1) * hidden_], &up[(size_t)i * hidden_], (size_t)hidden_ * 4);
        }
        std::vector<float> db;
        if (bias_) {
            const std::vector<float> gb = host_floats(need_tensor(file, prefix + ".gate_proj.bias")), ub = host_floats(need_tensor(file, prefix + ".up_proj.bias"));
            b.resize((size_t)2 * inter_);
            for (int i = 0; i < inter_; ++i) { b[2 * i] = gb[i]; b[2 * i + 1] = ub[i]; }
            db = host_floats(need_tensor(file, prefix + ".down_proj.bias"));
        }
        gate_up_ = Linear(w.data(), 2 * inter_, hidden_, bias_ ? b.data() : nullptr, dtype);
        down_ = Linear(need_tensor(file, prefix + ".down_proj.weight"), bias_ ? db.data() : nullptr, dtype);
    }
    size_t weight_bytes() const override { return gate_up_.weight_bytes() + down_.weight_bytes(); }
    bool capturable() const override { return true; }
    bool accepts_pending_norm() const override { return true; }
    bool fuses_following_norm() const override { return true; }

    // norm + gate/up + SwiGLU; down projection into the residual
    bool emit_fused(FusedBuilder& b, const float* gain, float eps) const override {
        if (b.ctx->dtype != DType::BF16 || hidden_ != b.hidden || inter_ % 8) return false;
        void* act = b.arena->take((size_t)b.tokens * inter_ * 2);
        EgFusedTemplate t = FusedBuilder::blank();
        t.input = EGF_IN_NORM;
        t.output = EGF_OUT_SWIGLU;
        t.N = 2 * inter_;
        t.K = hidden_;
        t.tiles_per_unit = 1;
        t.group_rows = 8;
        t.units_per_group = 1;
        t.warp_units = hidden_ <= EGF_STAGE_COLS;
        t.eps = eps;
        t.out = act;
        t.ldo = inter_;
        if (!b.linear(t, gate_up_.weight, hidden_, gate_up_.bias_f32(), gain)) return false;
        EgFusedTemplate d = FusedBuilder::blank();
        d.input = EGF_IN_ROWS;
        d.output = EGF_OUT_RESIDUAL;
        d.N = hidden_;
        d.K = inter_;
        d.tiles_per_unit = 1;
        d.group_rows = 8;
        d.units_per_group = 1;
        d.x = act;
        d.ldx = inter_;
        return b.linear(d, down_.weight, inter_, down_.bias_f32(), nullptr);
    }

    Delta forward(const StepContext& ctx, PartInput in, const FollowingNorm* follow) override {
        const int T = ctx.num_tokens;
        const DType dtype = ctx.dtype;
        Rows act{ctx.take_rows(T, inter_, dtype), dtype, T, inter_, inter_};
        if (in.pending && in.pending->fusable) {
            // decode: add + norm + gate/up product + SwiGLU in one kernel
            const NormInFront norm = in.pending->fused();
            gate_up_.skinny(ctx, plans::EPI_SWIGLU, T, nullptr, &norm, act.p, inter_, nullptr, nullptr, nullptr, nullptr, nullptr);
        } else {
            const Rows x = in.pending ? in.pending->materialize() : in.rows;
            if (plans::gemm_skinny_takes(dtype, T, hidden_) && Linear::aligned(x)) {
                gate_up_.skinny(ctx, plans::EPI_SWIGLU, T, &x, nullptr, act.p, inter_, nullptr, nullptr, nullptr, nullptr, nullptr);
            } else if (plans::gemm_tcgen05_wide_takes(dtype, T, 2 * inter_, hidden_) && Linear::aligned(x)) {
                // prompts: the product on the tcgen05 tensor cores (CTA pairs, 256 x 256 tiles) with SwiGLU in its epilogue
                launch_check(eg_gemm_tcgen05_pair(ctx.stream, plans::EPI_SWIGLU, x.p, x.ld, gate_up_.weight, hidden_, gate_up_.bias_f32(), act.p, inter_, T,
                                                  2 * inter_, hidden_, 256, ctx.status, nullptr), "gemm_tcgen05_pair");
            } else {
                const Rows gu = gate_up_(ctx, x);
                launch_check(eg_swiglu(ctx.stream, (int)dtype, gu.p, (int)gu.ld, act.p, inter_, T, inter_), "swiglu");
            }
        }
        Delta d;
        if (follow && down_.takes_following_norm(act)) {
            d.pre = down_.with_following_norm(ctx, act, *follow);
            return d;
        }
        const Rows o = down_(ctx, act);
        d.p = o.p;
        d.dtype = o.dtype;
        return d;
    }

private:
    int hidden_, inter_;
    bool bias_;
    Linear gate_up_, down_;
};

// ---- token embedding: residual[t] = E[id[t]] (src/models/embedding.cpp:54-76) ---------------------------------------
class TokenEmbedding : public Embedding {
public:
    TokenEmbedding(const Params& p, const std::string& prefix) : Embedding(p, prefix), vocab_((int)p.integer("vocab_size")), hidden_((int)p.integer("hidden_size")) {}
    std::vector<TensorRequest> tensor_requests() const override { return {TensorRequest::matrix(prefix + ".weight", vocab_, hidden_)}; }
    void load(const HostTensors& file, DType dtype) override {
        table_ = upload(need_tensor(file, prefix + ".weight"), dtype);
        dtype_ = dtype;
    }
    bool capturable() const override { return true; }
    void forward(const StepContext& ctx, float* residual) override {
        launch_check(eg_embedding_gather(ctx.stream, (int)dtype_, ctx.token_ids, table_.get(), residual, ctx.num_tokens, hidden_, vocab_, ctx.status),
                     "embedding_gather");
    }
    const void* table() const override { return table_.get(); }
    bool fused_gather(const void** table, int* vocab) const override {
        if (dtype_ != DType::BF16 || hidden_ % 4) return false;
        *table = table_.get();
        *vocab = vocab_;
        return true;
    }

private:
    int vocab_, hidden_;
    DType dtype_ = DType::BF16;
    DeviceBuffer table_;
};

// ---- output head: logits = x E^T when tied (the reference always is, src/models/gpt_model.cpp:324-328,
// src/models/embedding.cpp:78-81) or x W_head^T with lm_head.weight when not.  Logits are float32 in both precisions.
// Parameters: vocab_size, hidden_size, tied_to (prefix of the embedding, or absent) -------------------------------------
class LMHead : public Head {
public:
    LMHead(const Params& p, const std::string& prefix) : Head(p, prefix), vocab_((int)p.integer("vocab_size")), hidden_((int)p.integer("hidden_size")), tied_(p.has("tied_to")) {}
    std::vector<TensorRequest> tensor_requests() const override {
        if (tied_) return {};
        return {TensorRequest::matrix(prefix + ".weight", vocab_, hidden_)};
    }
    void load_head(const HostTensors& file, DType dtype, const void* tied_table) override {
        if (tied_) linear_ = Linear::sharing(tied_table, vocab_, hidden_, dtype);
        else linear_ = Linear(need_tensor(file, prefix + ".weight"), nullptr, dtype);
    }
    size_t weight_bytes() const override { return linear_.weight_bytes(); }
    bool capturable() const override { return true; }
    int vocab() const override { return vocab_; }
    bool emit_fused(FusedBuilder& b, const float* gain, float eps) const override {
        if (b.ctx->dtype != DType::BF16 || hidden_ != b.hidden || linear_.has_bias()) return false;
        b.logits = b.arena->take_n<float>((size_t)b.tokens * vocab_);
        EgFusedTemplate t = FusedBuilder::blank();
        t.input = EGF_IN_NORM;
        t.output = EGF_OUT_F32;
        t.N = vocab_;
        t.K = hidden_;
        t.tiles_per_unit = 1;
        t.group_rows = 8;
        t.units_per_group = 1;
        t.warp_units = hidden_ <= EGF_STAGE_COLS;
        t.eps = eps;
        t.out = b.logits;
        t.ldo = vocab_;
        return b.linear(t, linear_.weight, hidden_, nullptr, gain);
    }
    float* forward(const StepContext& ctx, PartInput in, int rows) override {
        // Thousands of CTAs share the head's rows, and each would repeat the add + norm of the few tokens in front of its
        // product: the norm runs once, in a kernel of its own.
        Rows x = in.pending ? in.pending->materialize() : in.rows;
        x.rows = rows;
        return (float*)linear_(ctx, x, /*out_f32=*/true).p;
    }

private:
    int vocab_, hidden_;
    bool tied_;
    Linear linear_;
};

inline void register_builtin_parts() {
    PartRegistry& r = PartRegistry::instance();
    if (r.mixers.count("attention")) return;
    r.mixers["attention"] = [](const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> pos) {
        return std::make_shared<Attention>(p, prefix, std::move(pos));
    };
    r.feed_forwards["swiglu"] = [](const Params& p, const std::string& prefix) { return std::make_shared<SwiGLU>(p, prefix); };
    r.norms["rmsnorm"] = [](const Params& p, const std::string& prefix) { return std::make_shared<RMSNorm>(p, prefix); };
    r.positions["rope"] = [](const Params& p, const std::string& prefix) { return std::make_shared<RotaryEncoding>(p, prefix); };
    r.embeddings["embedding"] = [](const Params& p, const std::string& prefix) { return std::make_shared<TokenEmbedding>(p, prefix); };
    r.heads["lm_head"] = [](const Params& p, const std::string& prefix) { return std::make_shared<LMHead>(p, prefix); };
}

}  // namespace easygpt::engine
