// A model put together from a ModelSpec: parts built by kind from the registries, weights loaded by name with one
// error for everything that is wrong, and a forward over one step's batch that follows the spec's run order.
// (The reference's counterpart is GptModel::forward_logits, src/models/gpt_model.cpp:310-333.)
#pragma once
#include <fstream>
#include <sstream>

#include "architectures.hpp"
#include "parts.hpp"

namespace easygpt::engine {

// One built sub-layer of a block: the part, the norm in front of it or behind it, and an optional norm on its output.
struct SubLayer {
    std::string role, placement;
    std::shared_ptr<Norm> norm, output_norm;
    std::shared_ptr<Mixer> mixer;
    std::shared_ptr<FeedForward> feed_forward;
    bool plain_pre_norm = false;        // x = x + part(norm(x)) with nothing behind the part: the shape whose add and norm the parts may fuse
    Part* part() const { return mixer ? static_cast<Part*>(mixer.get()) : static_cast<Part*>(feed_forward.get()); }
    std::vector<Part*> parts() const {
        std::vector<Part*> out;
        if (norm) out.push_back(norm.get());
        out.push_back(part());
        if (output_norm) out.push_back(output_norm.get());
        return out;
    }
};

// A layer: its residual sub-layers in order.  For the pre-norm shape x += mixer(norm1(x)); x += feed_forward(norm2(x))
// (src/models/block.cpp:23-29) every addition is folded into the norm that follows it, or into the kernels around it
// where the parts offer that.  Other shapes (a norm behind the part, a norm on the part's output, no norm, no
// feed-forward) run the same parts with the additions and norms as kernels of their own.
class Block {
public:
    explicit Block(const LayerSpec& spec) {
        PartRegistry& reg = PartRegistry::instance();
        if (spec.position.present) position = PartRegistry::find(reg.positions, "position", spec.position.kind)(spec.position.params, spec.position.prefix);
        auto make_norm = [&](const PartSpec& p) -> std::shared_ptr<Norm> {
            return p.present ? PartRegistry::find(reg.norms, "norm", p.kind)(p.params, p.prefix) : nullptr;
        };
        for (const SubLayerSpec& s : spec.sublayers) {
            SubLayer sub;
            sub.role = s.role;
            sub.placement = s.norm_placement;
            sub.norm = make_norm(s.norm);
            sub.output_norm = make_norm(s.output_norm);
            if (s.role == "mixer") {
                sub.mixer = PartRegistry::find(reg.mixers, "mixer", s.part.kind)(s.part.params, s.part.prefix, position);
                mixer = sub.mixer.get();
            } else {
                sub.feed_forward = PartRegistry::find(reg.feed_forwards, "feed_forward", s.part.kind)(s.part.params, s.part.prefix);
            }
            sub.plain_pre_norm = sub.norm && sub.placement == "pre" && !sub.output_norm;
            sublayers.push_back(std::move(sub));
        }
    }
    std::vector<Part*> parts() const {
        std::vector<Part*> out;
        for (auto& s : sublayers)
            for (Part* p : s.parts()) out.push_back(p);
        return out;
    }
    // the norm that a fused add + norm in front of this layer would have to be (nullptr: nothing in front may prepare it)
    const Norm* first_norm() const { return sublayers.front().plain_pre_norm ? sublayers.front().norm.get() : nullptr; }

    struct Stream {
        float *residual, *spare;
        Delta delta;
    };

    // Returns the buffer that now holds the residual stream, the other one, and what the last sub-layer left still to be
    // added (its output, or the PreNormed it prepared for next_norm, the norm that runs after this block).
    Stream forward(StepContext& ctx, StepArenas& arenas, int* turn, Stream s, const CacheView& cache, void* work, const Norm* next_norm) const {
        const int T = ctx.num_tokens;
        for (size_t i = 0; i < sublayers.size(); ++i) {
            const SubLayer& sub = sublayers[i];
            // this sub-layer's arena: what the sub-layer before the last one left there is dead by now
            ctx.arena = &arenas.sub[(*turn)++ & 1];
            ctx.arena->reset();
            const Norm* following = (i + 1 < sublayers.size()) ? (sublayers[i + 1].plain_pre_norm ? sublayers[i + 1].norm.get() : nullptr) : next_norm;
            const int hidden = sub.norm ? sub.norm->size() : width_;
            if (sub.plain_pre_norm) {
                const int fused_rows = plans::fused_norm_max_tokens(sub.norm->size());
                PendingNorm pending(ctx, sub.norm.get(), s.residual, s.delta, s.spare, work, T, nullptr, 0, fused_rows);
                FollowingNorm follow;
                const FollowingNorm* offer = nullptr;
                const bool fuses = sub.mixer ? sub.mixer->fuses_following_norm() : sub.feed_forward->fuses_following_norm();
                if (fuses && following && following->rms_parameters(&follow.gain, &follow.eps) && ctx.dtype == DType::BF16 && T > 0 && T <= fused_rows) {
                    follow.norm = following;
                    follow.pending = &pending;
                    offer = &follow;
                }
                const bool accepts = sub.mixer ? sub.mixer->accepts_pending_norm() : sub.feed_forward->accepts_pending_norm();
                PartInput in;
                if (accepts) in.pending = &pending;
                else in.rows = pending.materialize();
                s.delta = sub.mixer ? sub.mixer->forward(ctx, in, cache, offer) : sub.feed_forward->forward(ctx, in, offer);
                if (!pending.consumed) throw DeviceError("a part that accepts a pending norm must use it");
                s.residual = pending.residual_after;
                s.spare = pending.spare_after;
                continue;
            }
            // the general shapes: the stream is settled first, every norm is a kernel of its own
            const long long n = (long long)T * hidden;
            if (s.delta.has_pre()) throw DeviceError("prepared rows reached a sub-layer that has no plain norm in front");
            if (s.delta.has_delta()) launch_check(eg_add_into_f32(ctx.stream, s.residual, s.delta.p, (int)s.delta.dtype, n), "add");
            s.delta = Delta();
            PartInput in;
            in.rows = Rows{work, ctx.dtype, T, hidden, hidden};
            if (sub.norm && sub.placement == "pre") sub.norm->forward(ctx, s.residual, nullptr, ctx.dtype, work, ctx.dtype, T, nullptr);
            else launch_check(eg_convert_rows(ctx.stream, s.residual, (int)DType::F32, work, (int)ctx.dtype, n), "convert");
            Delta d = sub.mixer ? sub.mixer->forward(ctx, in, cache, nullptr) : sub.feed_forward->forward(ctx, in, nullptr);
            if (d.has_pre()) throw DeviceError("a part returned prepared rows without having been offered the norm that follows");
            if (sub.output_norm) {
                // norm(delta) in the compute dtype: through the float32 spare buffer
                launch_check(eg_convert_rows(ctx.stream, d.p, (int)d.dtype, s.spare, (int)DType::F32, n), "convert");
                void* out = ctx.take_rows(T, hidden, ctx.dtype);
                sub.output_norm->forward(ctx, s.spare, nullptr, ctx.dtype, out, ctx.dtype, T, nullptr);
                d.p = out;
                d.dtype = ctx.dtype;
            }
            if (sub.norm && sub.placement == "post") {
                // x = norm(x + part(x)): the normalised sum is the new residual stream
                sub.norm->forward(ctx, s.residual, d.p, d.dtype, s.spare, DType::F32, T, nullptr);
                std::swap(s.residual, s.spare);
                d = Delta();
            }
            s.delta = d;
        }
        return s;
    }

    std::vector<SubLayer> sublayers;
    std::shared_ptr<PositionEncoding> position;
    Mixer* mixer = nullptr;
    int width_ = 0;                     // the model's width (for sub-layers without a norm of their own)
};

inline std::string read_text_file(const std::string& path) {
    std::ifstream in(path, std::ios::binary);
    if (!in) throw std::runtime_error("cannot open " + path);
    std::ostringstream ss;
    ss << in.rdbuf();
    return ss.str();
}

class Model {
public:
    Model(ModelSpec spec_, DType dtype) : spec(std::move(spec_)), dtype(dtype) {
        register_builtin_parts();
        spec.validate();
        PartRegistry& reg = PartRegistry::instance();
        embedding = PartRegistry::find(reg.embeddings, "embedding", spec.embedding.kind)(spec.embedding.params, spec.embedding.prefix);
        if (spec.embedding_position.present)
            embedding_position = PartRegistry::find(reg.positions, "position", spec.embedding_position.kind)(spec.embedding_position.params,
                                                                                                         spec.embedding_position.prefix);
        for (auto& l : spec.layers) {
            blocks.emplace_back(new Block(l));
            blocks.back()->width_ = (int)spec.hidden_size;
        }
        final_norm = PartRegistry::find(reg.norms, "norm", spec.final_norm.kind)(spec.final_norm.params, spec.final_norm.prefix);
        lm_head = PartRegistry::find(reg.heads, "head", spec.lm_head.kind)(spec.lm_head.params, spec.lm_head.prefix);
    }

    // the model class is chosen by config.json, as everywhere in the framework
    static std::unique_ptr<Model> from_dir(const std::string& dir, DType dtype) {
        register_builtin_architectures();
        const std::string cfg_path = dir + "/config.json";
        std::ifstream probe(cfg_path);
        if (!probe) throw std::runtime_error("no config.json in " + dir);
        probe.close();
        const json::Value config = json::parse(read_text_file(cfg_path));
        std::unique_ptr<Model> model(new Model(ArchitectureRegistry::instance().build(config), dtype));
        model->load_weights(dir + "/model.safetensors");
        return model;
    }

    std::vector<Part*> all_parts() const {
        std::vector<Part*> out{embedding.get()};
        if (embedding_position) out.push_back(embedding_position.get());
        for (auto& b : blocks)
            for (Part* p : b->parts()) out.push_back(p);
        out.push_back(final_norm.get());
        out.push_back(lm_head.get());
        return out;
    }
    // whether decode steps of this model may be captured in a CUDA graph: every part says so
    bool capturable() const {
        for (Part* p : all_parts())
            if (!p->capturable()) return false;
        for (auto& b : blocks)
            if (b->position && !b->position->capturable()) return false;
        return true;
    }
    std::vector<TensorRequest> tensor_requests() const {
        std::vector<TensorRequest> out;
        for (Part* p : all_parts())
            for (auto& r : p->tensor_requests()) out.push_back(r);
        for (auto& b : blocks)                                   // a layer's position encoding may have tensors of its own
            if (b->position)
                for (auto& r : b->position->tensor_requests()) out.push_back(r);
        return out;
    }
    void load_weights(const std::string& model_file) {
        SafetensorsFile file(model_file);
        check_manifest(tensor_requests(), file);
        embedding->load(file, dtype);
        if (embedding_position) embedding_position->load(file, dtype);
        for (auto& b : blocks)
            for (Part* p : b->parts()) p->load(file, dtype);
        final_norm->load(file, dtype);
        lm_head->load_head(file, dtype, embedding->table());
        EG_CUDA(cudaDeviceSynchronize());
    }
    // cache id -> what the entry that writes it needs
    std::map<int, CacheNeed> cache_needs() const {
        std::map<int, CacheNeed> needs;
        auto need_of = [&](int layer) { return blocks[layer]->mixer ? blocks[layer]->mixer->cache_need() : CacheNeed(); };
        for (auto& e : spec.run_order)
            if (e.writes_cache) needs[e.cache] = need_of(e.layer);
        for (auto& e : spec.run_order)
            if (!e.writes_cache && !(need_of(e.layer) == needs[e.cache]))
                throw std::invalid_argument("a run entry of layer " + std::to_string(e.layer) + " reads cache " + std::to_string(e.cache) +
                                            ", whose shape differs from its own");
        return needs;
    }
    // bytes of weights a step reads once each (embedding rows not counted)
    size_t weight_bytes_per_step() const {
        size_t total = 0;
        for (auto& e : spec.run_order)
            for (Part* p : blocks[e.layer]->parts()) total += p->weight_bytes();
        return total + final_norm->weight_bytes() + lm_head->weight_bytes();
    }
    // Upper bounds of the activation memory of a step of T tokens with R wanted rows: what lives for the whole step
    // (residual stream, shared tables, normalised rows and logits of the wanted places) and what one sub-layer takes.
    ArenaSizes activation_bytes(long long T, long long R) const {
        long long widths = 4 * spec.hidden_size, head_dim = 0;
        for (Part* p : all_parts()) {
            if (p->params.has("intermediate_size")) widths = std::max(widths, 2 * spec.hidden_size + 3 * p->params.integer("intermediate_size"));
            if (p->params.has("num_heads")) {
                const long long hd = p->params.integer("head_dim"), q = p->params.integer("num_heads") * hd;
                widths = std::max(widths, 2 * spec.hidden_size + 2 * q + 2 * p->params.integer("num_kv_heads") * hd);
                head_dim = std::max(head_dim, hd);
            }
        }
        ArenaSizes sizes;
        // partial results of an attention whose keys are shared by several CTAs: capped for prompt portions, and bounded by
        // the CTAs of a few waves for single tokens
        const size_t partials = plans::PREFILL_PARTS_SCRATCH_BYTES + (size_t)(4 * plans::sm_count() + 64) * 128 * (size_t)(head_dim + 2) * 4;
        sizes.sub = (size_t)T * (size_t)widths * 4 + partials + (4u << 20);
        sizes.step = (size_t)T * (size_t)(3 * spec.hidden_size + std::max<long long>(head_dim, 64)) * 4 + (size_t)R * (size_t)(spec.vocab_size + spec.hidden_size) * 4 +
                     (4u << 20);
        return sizes;
    }

    // The decode step of `ctx` (single tokens, logits for all of them) as a program for the fused decode kernel, if
    // every part of the model can say what it does as operations of it; otherwise an empty program.  The activations
    // come from the step arena, in the same order at every call, so the program stays valid while the arenas do.
    struct FusedProgram {
        std::vector<EgFusedTemplate> tmpls;
        std::vector<EgFusedOp> ops;
        int tokens = 0, stages = 0, xs_bytes = 0, grid = 0;
        float* logits = nullptr;
        bool ok() const { return !ops.empty(); }
    };
    FusedProgram fused_program(StepContext& ctx, StepArenas& arenas, const std::function<CacheView(int cache, bool writes)>& view) const {
        FusedProgram none;
        const int T = ctx.num_tokens;
        if (dtype != DType::BF16 || !ctx.all_decode || T <= 0 || T > EGF_MAX_TOKENS || embedding_position || spec.hidden_size % 16) return none;
        FusedBuilder b;
        b.ctx = &ctx;
        arenas.reset();
        b.arena = &arenas.step;
        b.tokens = T;
        b.hidden = (int)spec.hidden_size;
        b.grid = plans::sm_count();
        if (!embedding->fused_gather(&b.embed_table, &b.vocab)) return none;
        b.residual = b.arena->take_n<float>((size_t)T * b.hidden);
        const float* gain = nullptr;
        float eps = 0.f;
        for (auto& e : spec.run_order) {
            const Block& block = *blocks[e.layer];
            for (auto& sub : block.sublayers) {
                if (!sub.plain_pre_norm || !sub.norm->rms_parameters(&gain, &eps) || sub.norm->size() != b.hidden) return none;
                const bool ok = sub.mixer ? sub.mixer->emit_fused(b, gain, eps, view(e.cache, e.writes_cache)) : sub.feed_forward->emit_fused(b, gain, eps);
                if (!ok) return none;
            }
        }
        if (b.embed_table) return none;                 // nothing took the embedding as its input
        if (!final_norm->rms_parameters(&gain, &eps) || !lm_head->emit_fused(b, gain, eps) || !b.logits) return none;
        // the ring of weight stages takes the shared memory that is left
        int stages = 12;
        while (stages >= 3 && eg_decode_fused_smem(stages, b.xs_bytes, (int)b.ops.size(), (int)b.tmpls.size()) > 227 * 1024) --stages;
        if (stages < 3) return none;
        FusedProgram prog;
        prog.tmpls = std::move(b.tmpls);
        prog.ops = std::move(b.ops);
        prog.tokens = T;
        prog.stages = stages;
        prog.xs_bytes = b.xs_bytes;
        prog.grid = b.grid;
        prog.logits = b.logits;
        return prog;
    }

    // Runs the batch through every run entry; returns float32 logits [R, vocab] at logit_rows (token indices into the
    // batch; nullptr with all_rows: rows 0..T-1 in order, a decode step), or nullptr when none is wanted.
    float* forward(StepContext& ctx, StepArenas& arenas, const std::function<CacheView(int cache, bool writes)>& view, const int* logit_rows, int num_rows,
                   bool all_rows) const {
        const int T = ctx.num_tokens;
        const int H = (int)spec.hidden_size;
        ctx.shared.clear();
        arenas.reset();
        ctx.step_arena = ctx.arena = &arenas.step;
        int turn = 0;
        Block::Stream s;
        s.residual = ctx.take<float>((size_t)T * H);
        s.spare = ctx.take<float>((size_t)T * H);
        void* work = ctx.take_rows(T, H, dtype);
        embedding->forward(ctx, s.residual);
        if (embedding_position) embedding_position->add_to_embedding(s.residual, ctx);
        const auto& order = spec.run_order;
        for (size_t i = 0; i < order.size(); ++i) {
            const Norm* next_norm = (i + 1 < order.size()) ? blocks[order[i + 1].layer]->first_norm() : final_norm.get();
            s = blocks[order[i].layer]->forward(ctx, arenas, &turn, s, view(order[i].cache, order[i].writes_cache), work, next_norm);
        }
        ctx.arena = &arenas.step;                // the head's rows and logits live for the step
        if (num_rows <= 0) return nullptr;
        PendingNorm pending(ctx, final_norm.get(), s.residual, s.delta, s.spare, work, T, all_rows ? nullptr : logit_rows, num_rows,
                            plans::fused_norm_max_tokens(H));
        PartInput in;
        if (s.delta.has_pre()) {
            // the part in front prepared the final norm's rows for a product that folds the scale in; the head does not:
            // finish the norm here from the residual, which already holds the sum
            final_norm->forward(ctx, s.residual, nullptr, dtype, work, dtype, all_rows ? T : num_rows, all_rows ? nullptr : logit_rows);
            in.rows = Rows{work, dtype, all_rows ? T : num_rows, H, H};
        } else {
            in.pending = &pending;
        }
        return lm_head->forward(ctx, in, all_rows ? T : num_rows);
    }

    ModelSpec spec;
    DType dtype;
    std::shared_ptr<Embedding> embedding;
    std::shared_ptr<PositionEncoding> embedding_position;
    std::vector<std::unique_ptr<Block>> blocks;
    std::shared_ptr<Norm> final_norm;
    std::shared_ptr<Head> lm_head;
};

}  // namespace easygpt::engine
