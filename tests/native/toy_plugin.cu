// A plugin of the native engine, defined by the tests: a mixer with state of its own, a routed feed-forward, another
// position encoding, and an architecture that puts them beside the engine's own attention and SwiGLU.  It shows that
// parts and a whole architecture are added without a change to the engine's files.  Toy parts only: they are no
// model of anyone's.
#include "common.cuh"
#include "plugin.hpp"

using namespace easygpt::engine;

namespace {

// s <- decay * s + W x per token, out = s; the state s [hidden] lives in the request's state slot.  One block per entry
// of the batch walks that entry's tokens in order; thread j owns element j of the state.
template <typename T>
__global__ void decaying_sum_kernel(const T* __restrict__ x, T* __restrict__ out, const float* __restrict__ w, float* __restrict__ state,
                                    const int* __restrict__ seq_starts, const int* __restrict__ seq_slots, int hidden, float decay) {
    const int entry = blockIdx.x;
    float* s = state + (size_t)seq_slots[entry] * hidden;
    for (int t = seq_starts[entry]; t < seq_starts[entry + 1]; ++t) {
        for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
            float y = 0.f;
            for (int k = 0; k < hidden; ++k) y += w[(size_t)j * hidden + k] * to_f32<T>(x[(size_t)t * hidden + k]);
            const float v = decay * s[j] + y;
            s[j] = v;
            out[(size_t)t * hidden + j] = from_f32<T>(v);
        }
    }
}

class DecayingSum : public Mixer {
public:
    DecayingSum(const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> position)
        : Mixer(p, prefix, std::move(position)), hidden_((int)p.integer("hidden_size")), decay_((float)p.real("decay")) {}
    std::vector<TensorRequest> tensor_requests() const override { return {TensorRequest::matrix(prefix + ".w", hidden_, hidden_)}; }
    void load(const HostTensors& file, DType) override {
        const std::vector<float> w = host_floats(need_tensor(file, prefix + ".w"));
        w_ = upload(w.data(), w.size(), DType::F32);
    }
    CacheNeed cache_need() const override { return CacheNeed::state({hidden_}); }
    bool capturable() const override { return true; }       // the kernel reads the batch's shape from device arrays
    Delta forward(const StepContext& ctx, PartInput in, const CacheView& cache, const FollowingNorm*) override {
        Delta d;
        d.dtype = ctx.dtype;
        d.p = ctx.take_rows(ctx.num_tokens, hidden_, ctx.dtype);
        const int threads = std::min(256, hidden_);
        if (ctx.dtype == DType::F32)
            decaying_sum_kernel<float><<<ctx.num_seqs, threads, 0, ctx.stream>>>((const float*)in.rows.p, (float*)d.p, w_.as<float>(), (float*)cache.state,
                                                                                ctx.seq_starts, ctx.seq_slots, hidden_, decay_);
        else
            decaying_sum_kernel<bf16><<<ctx.num_seqs, threads, 0, ctx.stream>>>((const bf16*)in.rows.p, (bf16*)d.p, w_.as<float>(), (float*)cache.state,
                                                                               ctx.seq_starts, ctx.seq_slots, hidden_, decay_);
        return d;
    }

private:
    int hidden_;
    float decay_;
    DeviceBuffer w_;
};

// Each token goes to the expert with the largest router logit (float32) and gets relu(W_e x) scaled by the softmax
// weight of that expert.  One block per token.
template <typename T>
__global__ void top_one_experts_kernel(const T* __restrict__ x, T* __restrict__ out, const float* __restrict__ router, const float* __restrict__ experts,
                                       int hidden, int num_experts) {
    __shared__ int choice;
    __shared__ float prob;
    const int t = blockIdx.x;
    const T* row = x + (size_t)t * hidden;
    if (threadIdx.x == 0) {
        float best = -INFINITY, sum = 0.f, logits[16];
        int arg = 0;
        for (int e = 0; e < num_experts; ++e) {
            float l = 0.f;
            for (int k = 0; k < hidden; ++k) l += router[(size_t)e * hidden + k] * to_f32<T>(row[k]);
            logits[e] = l;
            if (l > best) { best = l; arg = e; }
        }
        for (int e = 0; e < num_experts; ++e) sum += expf(logits[e] - best);
        choice = arg;
        prob = 1.0f / sum;
    }
    __syncthreads();
    const float* w = experts + (size_t)choice * hidden * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float y = 0.f;
        for (int k = 0; k < hidden; ++k) y += w[(size_t)j * hidden + k] * to_f32<T>(row[k]);
        out[(size_t)t * hidden + j] = from_f32<T>(fmaxf(y, 0.f) * prob);
    }
}

class TopOneExperts : public FeedForward {
public:
    TopOneExperts(const Params& p, const std::string& prefix) : FeedForward(p, prefix), hidden_((int)p.integer("hidden_size")), experts_((int)p.integer("experts")) {
        if (experts_ > 16) throw std::invalid_argument("the toy routed feed-forward takes at most 16 experts");
    }
    std::vector<TensorRequest> tensor_requests() const override {
        std::vector<TensorRequest> r = {TensorRequest::matrix(prefix + ".router", experts_, hidden_)};
        for (int e = 0; e < experts_; ++e) r.push_back(TensorRequest::matrix(prefix + ".expert" + std::to_string(e), hidden_, hidden_));
        return r;
    }
    void load(const HostTensors& file, DType) override {
        const std::vector<float> router = host_floats(need_tensor(file, prefix + ".router"));
        router_ = upload(router.data(), router.size(), DType::F32);
        std::vector<float> all;
        for (int e = 0; e < experts_; ++e) {
            const std::vector<float> w = host_floats(need_tensor(file, prefix + ".expert" + std::to_string(e)));
            all.insert(all.end(), w.begin(), w.end());
        }
        weights_ = upload(all.data(), all.size(), DType::F32);
    }
    bool capturable() const override { return true; }
    Delta forward(const StepContext& ctx, PartInput in, const FollowingNorm*) override {
        Delta d;
        d.dtype = ctx.dtype;
        d.p = ctx.take_rows(ctx.num_tokens, hidden_, ctx.dtype);
        if (ctx.dtype == DType::F32)
            top_one_experts_kernel<float><<<ctx.num_tokens, 64, 0, ctx.stream>>>((const float*)in.rows.p, (float*)d.p, router_.as<float>(), weights_.as<float>(), hidden_, experts_);
        else
            top_one_experts_kernel<bf16><<<ctx.num_tokens, 64, 0, ctx.stream>>>((const bf16*)in.rows.p, (bf16*)d.p, router_.as<float>(), weights_.as<float>(), hidden_, experts_);
        return d;
    }

private:
    int hidden_, experts_;
    DeviceBuffer router_, weights_;
};

// a learned vector per position, added to the residual stream right after the embedding
__global__ void add_positions_kernel(float* __restrict__ residual, const float* __restrict__ table, const int* __restrict__ positions, int hidden, int max_positions) {
    const int t = blockIdx.x;
    const int pos = min(positions[t], max_positions - 1);
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) residual[(size_t)t * hidden + j] += table[(size_t)pos * hidden + j];
}

class LearnedOffsets : public PositionEncoding {
public:
    LearnedOffsets(const Params& p, const std::string& prefix) : PositionEncoding(p, prefix), hidden_((int)p.integer("hidden_size")), max_positions_((int)p.integer("max_positions")) {}
    std::vector<TensorRequest> tensor_requests() const override { return {TensorRequest::matrix(prefix + ".table", max_positions_, hidden_)}; }
    void load(const HostTensors& file, DType) override {
        const std::vector<float> t = host_floats(need_tensor(file, prefix + ".table"));
        table_ = upload(t.data(), t.size(), DType::F32);
    }
    bool capturable() const override { return true; }
    void add_to_embedding(float* residual, const StepContext& ctx) const override {
        add_positions_kernel<<<ctx.num_tokens, 64, 0, ctx.stream>>>(residual, table_.as<float>(), ctx.positions, hidden_, max_positions_);
    }

private:
    int hidden_, max_positions_;
    DeviceBuffer table_;
};

// The architecture: learned positions at the embedding; layer 0 (pre-norm) the toy mixer and the routed experts; layer 1
// (post-norm, by the spec alone) the engine's own attention with rotary encoding and its SwiGLU.
ModelSpec toy_spec(const easygpt::json::Value& config) {
    auto integer = [&](const char* key) {
        const easygpt::json::Value* v = config.find(key);
        if (!v || !v->is_integer) throw ConfigError(std::string("config.json lacks: ") + key);
        return v->integer;
    };
    const long long hidden = integer("width"), vocab = integer("vocabulary"), experts = integer("experts"), positions = integer("positions");
    const double eps = config.find("eps")->number, decay = config.find("decay")->number;
    auto norm = [&](const std::string& prefix) { return PartSpec{"rmsnorm", Params{{"size", hidden}, {"eps", eps}}, prefix, true}; };
    ModelSpec spec;
    spec.architecture = "toy_native";
    spec.vocab_size = vocab;
    spec.hidden_size = hidden;
    spec.max_positions = positions;
    spec.layers.push_back(LayerSpec::pre_norm(PartSpec{"toy_decaying_sum", Params{{"hidden_size", hidden}, {"decay", decay}}, "l0.mix", true},
                                              PartSpec{"toy_top_one_experts", Params{{"hidden_size", hidden}, {"experts", experts}}, "l0.ff", true},
                                              norm("l0.n1"), norm("l0.n2"), PartSpec::none()));
    LayerSpec post;
    post.sublayers.push_back({"mixer", PartSpec{"attention", Params{{"hidden_size", hidden}, {"num_heads", 2}, {"num_kv_heads", 1}, {"head_dim", 16}}, "l1.att", true},
                              norm("l1.n1"), "post", PartSpec::none()});
    post.sublayers.push_back({"feed_forward", PartSpec{"swiglu", Params{{"hidden_size", hidden}, {"intermediate_size", 48}}, "l1.mlp", true}, norm("l1.n2"), "post",
                              PartSpec::none()});
    post.position = PartSpec{"rope", Params{{"head_dim", 16}, {"rotary_dim", 16}, {"theta", 10000.0}}, "", true};
    spec.layers.push_back(post);
    spec.run_order = {RunEntry{0, 0, true}, RunEntry{1, 1, true}};
    spec.embedding = PartSpec{"embedding", Params{{"vocab_size", vocab}, {"hidden_size", hidden}}, "emb", true};
    spec.embedding_position = PartSpec{"toy_learned_offsets", Params{{"hidden_size", hidden}, {"max_positions", positions}}, "pos", true};
    spec.final_norm = norm("norm");
    spec.lm_head = PartSpec{"lm_head", Params{{"vocab_size", vocab}, {"hidden_size", hidden}, {"tied_to", "emb"}}, "head", true};
    return spec;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) void easygpt_register(PartRegistry* parts, ArchitectureRegistry* architectures) {
    parts->mixers["toy_decaying_sum"] = [](const Params& p, const std::string& prefix, std::shared_ptr<PositionEncoding> pos) {
        return std::make_shared<DecayingSum>(p, prefix, std::move(pos));
    };
    parts->feed_forwards["toy_top_one_experts"] = [](const Params& p, const std::string& prefix) { return std::make_shared<TopOneExperts>(p, prefix); };
    parts->positions["toy_learned_offsets"] = [](const Params& p, const std::string& prefix) { return std::make_shared<LearnedOffsets>(p, prefix); };
    architectures->add("toy_native", toy_spec);
}
