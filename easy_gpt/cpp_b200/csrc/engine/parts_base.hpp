// Interfaces of the parts a layer is put together from, and what a step hands to them.
//
// A *mixer* moves information between the tokens of a request (attention here); a *feed-forward* works
// on each token alone; a *norm* normalises the residual stream; a *position encoding* is handed to the
// mixer that wants one (or works on the residual stream right after the embedding).  Every part is built
// from PartSpec::params (its sizes and constants) and its prefix (where its tensors live) and never
// learns which model it sits in.
//
// The residual stream is float32 in both precisions.  A block hands each part the normalised input in
// the compute dtype and gets back a *delta* in the compute dtype; the next norm adds the delta to the
// residual in float32 while it normalises (one fused kernel).  Two offers let a part fold neighbouring
// work into its own kernels: a PendingNorm stands for "norm(residual + delta), not computed yet", and a
// FollowingNorm for the add and the norm that come right after the part.
//
// To add a part: derive from the matching base, implement tensor_requests / load / forward (and
// cache_need for a mixer that keeps something per request), and register a factory under a kind.
#pragma once
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "device.hpp"
#include "../decode_fused.h"
#include "kernels_api.h"
#include "plans.hpp"
#include "spec.hpp"
#include "weights.hpp"

namespace easygpt::engine {

// ---- what a mixer needs the cache manager to keep for it -----------------------------------------------
struct CacheNeed {
    enum Kind { None, PagedKV, State } kind = None;
    int num_kv_heads = 0, head_dim = 0;
    long long window = -1;                  // PagedKV: < 0 keeps all keys
    std::vector<long long> state_shape;     // State: a tensor of this shape per live request, zeroed when a request starts
    DType state_dtype = DType::F32;
    bool operator==(const CacheNeed& o) const {
        return kind == o.kind && num_kv_heads == o.num_kv_heads && head_dim == o.head_dim && window == o.window &&
               state_shape == o.state_shape && state_dtype == o.state_dtype;
    }
    static CacheNeed paged(int kv_heads, int head_dim, long long window) {
        CacheNeed n;
        n.kind = PagedKV;
        n.num_kv_heads = kv_heads;
        n.head_dim = head_dim;
        n.window = window;
        return n;
    }
    static CacheNeed state(std::vector<long long> shape, DType dtype = DType::F32) {
        CacheNeed n;
        n.kind = State;
        n.state_shape = std::move(shape);
        n.state_dtype = dtype;
        return n;
    }
};

// ---- what a step hands to the parts ------------------------------------------------------------------------
struct GroupTables {
    int page_size = 0;
    const int* block_table = nullptr;   // int32 [num_seqs, table_width]: page id per logical page, -1 where none
    int table_width = 0;
    const int* slot_map = nullptr;      // int32 [T]: page * page_size + offset where the token's key/value is stored
};

// Memory that kernels need beyond their inputs and outputs and that outlives a step: ticket counters and work
// queues, which every kernel leaves at zero.  Allocated once with the engine.
struct KernelScratch {
    DeviceBuffer skinny_partials, skinny_counters, attention_counters, prefill_queue, argmax_counters;
    static constexpr size_t SKINNY_FLOATS = 1u << 22, SKINNY_COUNTERS = 1u << 14, ATTENTION_COUNTERS = 1u << 16, ARGMAX_ROWS = 4096;
    KernelScratch()
        : skinny_partials(SKINNY_FLOATS * 4), skinny_counters(SKINNY_COUNTERS * 4, true), attention_counters(ATTENTION_COUNTERS * 4, true),
          prefill_queue(16, true), argmax_counters(ARGMAX_ROWS * 4, true) {}
};

struct StepContext {
    DType dtype = DType::BF16;
    cudaStream_t stream = nullptr;
    // Activation memory.  `arena` is the current sub-layer's: a part takes what it needs from it, and what it hands back
    // (its delta, prepared rows) stays valid until the sub-layer after the next one starts (two arenas take turns).
    // `step_arena` holds what lives for the whole step (the residual stream, tables that layers share, the logits).
    Arena* arena = nullptr;
    Arena* step_arena = nullptr;
    Blas* blas = nullptr;
    KernelScratch* scratch = nullptr;
    int num_tokens = 0, num_seqs = 0;
    const int *token_ids = nullptr, *positions = nullptr, *token_seq = nullptr, *seq_starts = nullptr, *seq_context = nullptr,
              *seq_slots = nullptr;
    int* status = nullptr;              // device status word the kernels OR their complaints into
    std::vector<GroupTables> groups;
    // host twins for parts that plan their launches on the host (null inside a captured step: such parts are not capturable)
    const int *host_seq_starts = nullptr, *host_seq_context = nullptr, *host_seq_slots = nullptr;
    int max_query_len = 0;
    long long max_context_len = 0;      // longest context + query of the batch
    bool all_decode = false;
    const int* query_tiles = nullptr;   // int32 [num_tiles, 3] = (entry, first token, count) of the prompt portions' tiles
    int num_tiles = 0;
    const int* small_tokens = nullptr;  // token indices of the entries too short for tiles
    int num_small = 0;
    std::map<std::string, void*> shared;    // per-step data that parts share between layers (cleared at every forward)

    template <class T> T* take(size_t n) const { return arena->take_n<T>(n); }
    template <class T> T* take_for_step(size_t n) const { return step_arena->take_n<T>(n); }
    void* take_rows(size_t rows, size_t cols, DType t) const { return arena->take(rows * cols * dtype_size(t)); }
};

struct CacheView {
    int group = -1;                     // index into StepContext::groups (paged) ...
    void *k = nullptr, *v = nullptr;    // element (page, kv head, offset, d) at k[page * page_stride + head * head_stride + offset * head_dim + d]
    long long page_stride = 0, head_stride = 0;
    int num_pages = 0, page_size = 0;
    void* state = nullptr;              // [max_slots, state elements] for a mixer with fixed-size state
    size_t state_bytes_per_slot = 0;
    bool writes = true;                 // false: read another entry's cache, store nothing
};

// rows of activations on the device
struct Rows {
    void* p = nullptr;
    DType dtype = DType::BF16;
    int rows = 0, cols = 0;
    long long ld = 0;
};

// ---- the parts ----------------------------------------------------------------------------------------------
using HostTensors = SafetensorsFile;

class Part {
public:
    Part(const Params& params, const std::string& prefix) : params(params), prefix(prefix) {}
    virtual ~Part() = default;
    virtual std::vector<TensorRequest> tensor_requests() const { return {}; }
    // takes this part's tensors (host, stored precision) to the device in the form its kernels want
    virtual void load(const HostTensors&, DType) {}
    virtual size_t weight_bytes() const { return 0; }       // bytes of weights one forward reads (roofline arithmetic)
    // true if forward() only launches device work whose shape depends on the batch's size alone (no reads of the
    // batch's contents on the host): then decode steps may be captured in a CUDA graph
    virtual bool capturable() const { return false; }
    Params params;
    std::string prefix;
};

struct HalfRotation {
    const float* inv_freq = nullptr;    // float32 [rotary_dim / 2] on the device
    int rotary_dim = 0;
    std::string key;                    // equal keys mean equal tables: consumers may share what they derive from one
};

// How positions reach the model: any of three offers, each with a default that does nothing.
class PositionEncoding : public Part {
public:
    using Part::Part;
    // a half rotation of queries and keys that attention kernels can apply themselves (fused with the cache write)
    virtual bool half_rotation(HalfRotation*) const { return false; }
    // changes q [T, heads, head_dim] and k [T, kv heads, head_dim] in place (rows ld elements apart); called only when
    // half_rotation() says no
    virtual void apply_to_query_key(void* /*q*/, void* /*k*/, long long /*ld*/, int /*heads*/, int /*kv_heads*/, int /*head_dim*/, const StepContext&) const {}
    // adds to the float32 residual stream [T, hidden] right after the token embedding
    virtual void add_to_embedding(float* /*residual*/, const StepContext&) const {}
};

class Norm : public Part {
public:
    using Part::Part;
    // (gain float32 [size] on the device, eps) if this norm is a plain RMSNorm that a consumer's kernel may fold in
    virtual bool rms_parameters(const float** /*gain*/, float* /*eps*/) const { return false; }
    // residual += delta (float32, in place, unless rows is given); the normalised rows go to out (out_dtype).
    // With rows only those rows are normalised, into out[0 .. num_rows), and the residual is left as it is.
    virtual void forward(const StepContext& ctx, float* residual, const void* delta, DType delta_dtype, void* out, DType out_dtype, int num_rows,
                         const int* rows) const = 0;
    virtual int size() const = 0;
};

// Left by a part in place of its delta when it took a FollowingNorm over: the residual already holds the sum v;
// rows is (compute dtype) gain * v and ss_parts float32 [parts, padded T] the partial sums of v^2 per token.
struct PreNormed {
    const Norm* norm = nullptr;
    void* rows = nullptr;
    float* ss_parts = nullptr;
    int parts = 0;
};

// What a part hands back: a delta to be added to the residual stream, or a PreNormed, or nothing.
struct Delta {
    void* p = nullptr;
    DType dtype = DType::BF16;
    PreNormed pre;
    bool has_delta() const { return p != nullptr; }
    bool has_pre() const { return pre.norm != nullptr; }
};

// An add and an RMSNorm that a part's first kernel is to do itself, in one of two forms: residual (+ delta, the sum
// then also written to residual_out) with gain and eps; or prepared rows and partial sums, where only the scale is missing.
struct NormInFront {
    float eps = 0.f;
    const float* gain = nullptr;
    const float* residual = nullptr;
    const void* delta = nullptr;
    float* residual_out = nullptr;
    const void* prepared_rows = nullptr;
    const float* prepared_sums = nullptr;
    int prepared_parts = 0;
};

// x = norm(residual + delta), not computed yet.
class PendingNorm {
public:
    PendingNorm(const StepContext& ctx, const Norm* norm, float* residual, const Delta& delta, float* spare, void* work, int tokens,
                const int* rows, int num_rows, int max_fused_rows)
        : ctx_(ctx), norm_(norm), residual_(residual), delta_(delta), spare_(spare), work_(work), tokens_(tokens), rows_(rows), num_rows_(num_rows) {
        residual_after = residual;
        spare_after = spare;
        has_rms_ = norm->rms_parameters(&gain_, &eps_);
        fusable = has_rms_ && rows == nullptr && ctx.dtype == DType::BF16 && tokens > 0 && tokens <= max_fused_rows &&
                  (!delta.has_delta() || delta.dtype == DType::BF16);
    }
    // the norm as a kernel of its own; returns the normalised rows (ctx.dtype)
    Rows materialize() {
        consumed = true;
        const int n = rows_ ? num_rows_ : tokens_;
        if (delta_.has_pre()) throw DeviceError("prepared rows cannot be turned back into a plain norm");
        norm_->forward(ctx_, residual_, delta_.p, delta_.dtype, work_, ctx_.dtype, n, rows_);
        return Rows{work_, ctx_.dtype, n, norm_->size(), norm_->size()};
    }
    // hands the add and the norm over to the part, whose first kernel does both
    NormInFront fused() {
        consumed = true;
        NormInFront f;
        f.eps = eps_;
        if (delta_.has_pre()) {
            f.prepared_rows = delta_.pre.rows;
            f.prepared_sums = delta_.pre.ss_parts;
            f.prepared_parts = delta_.pre.parts;
            return f;
        }
        f.gain = gain_;
        f.residual = residual_;
        if (delta_.has_delta()) {
            f.delta = delta_.p;
            f.residual_out = spare_;
            residual_after = spare_;
            spare_after = residual_;
        }
        return f;
    }
    bool fusable = false, consumed = false;
    float *residual_after, *spare_after;
    int tokens() const { return tokens_; }
    int width() const { return norm_->size(); }

private:
    const StepContext& ctx_;
    const Norm* norm_;
    float* residual_;
    Delta delta_;
    float* spare_;
    void* work_;
    int tokens_;
    const int* rows_;
    int num_rows_;
    bool has_rms_ = false;
    const float* gain_ = nullptr;
    float eps_ = 0.f;
};

// The add and the norm that come right after a part (a plain RMSNorm).  A part that fuses such things may let its last
// kernel add its output to `residual()` in place and prepare the norm, and hand back a PreNormed instead of a delta.
struct FollowingNorm {
    const Norm* norm = nullptr;
    const float* gain = nullptr;
    float eps = 0.f;
    PendingNorm* pending = nullptr;
    float* residual() const { return pending->residual_after; }     // valid once the part's own input norm has run
};

// The input of a mixer or feed-forward: rows already normalised, or a PendingNorm that stands for them.
struct PartInput {
    Rows rows;
    PendingNorm* pending = nullptr;
};

// ---- a decode step as one program (csrc/decode_fused.cu) ---------------------------------------------------------
// A part that can say what it does in a decode step as operations of that program does so in emit_fused(); a model all
// of whose parts can is stepped by ONE persistent kernel for small batches instead of a chain of kernels.  The builder
// holds the step's buffers and collects the operations; what a part needs beyond them it takes from `arena`.
struct FusedBuilder {
    const StepContext* ctx = nullptr;
    Arena* arena = nullptr;
    int tokens = 0, hidden = 0, grid = 0;
    float* residual = nullptr;                      // float32 [tokens, hidden]
    const void* embed_table = nullptr;              // set until the first linear operation has taken the embedding as its input
    int vocab = 0;
    std::vector<EgFusedTemplate> tmpls;
    std::vector<EgFusedOp> ops;
    int xs_bytes = 0;                               // shared memory for the widest input rows (and the attention's key tiles)
    int next_offset = 0;
    float* logits = nullptr;

    static EgFusedTemplate blank() {
        EgFusedTemplate t;
        std::memset(&t, 0, sizeof t);
        return t;
    }
    int intern(const EgFusedTemplate& t) {
        for (size_t i = 0; i < tmpls.size(); ++i)
            if (std::memcmp(&tmpls[i], &t, sizeof t) == 0) return (int)i;
        tmpls.push_back(t);
        return (int)tmpls.size() - 1;
    }
    static int input_row_bytes(int K) { return ((K * 2 + 127) / 128) * 128 + 64; }
    // a linear operation over weights [N, K]; gain/eps: the RMSNorm in front (input rows x otherwise)
    bool linear(EgFusedTemplate t, const void* W, long long ldw, const float* bias, const float* gain, void* k_cache = nullptr, void* v_cache = nullptr) {
        t.type = EGF_LINEAR;
        if (t.K % 16 || t.N % t.group_rows || ldw % 8 || (uintptr_t)W % 16) return false;
        if (t.input == EGF_IN_ROWS && (t.ldx % 8 || (uintptr_t)t.x % 16)) return false;
        t.num_units = t.N / t.group_rows * t.units_per_group;
        if (t.input != EGF_IN_ROWS) {
            t.residual = residual;
            if (embed_table) {
                t.input = EGF_IN_EMBED_NORM;
                t.embed_table = embed_table;
                t.token_ids = ctx->token_ids;
                t.vocab = vocab;
                embed_table = nullptr;
            }
        }
        if (t.output == EGF_OUT_RESIDUAL) t.residual = residual;
        EgFusedOp op;
        std::memset(&op, 0, sizeof op);
        op.tmpl = intern(t);
        op.unit_offset = next_offset;
        op.W = W;
        op.ldw = ldw;
        op.bias = bias;
        op.gain = gain;
        op.k_cache = k_cache;
        op.v_cache = v_cache;
        ops.push_back(op);
        next_offset = (next_offset + t.num_units) % grid;
        xs_bytes = std::max(xs_bytes, EGF_MAX_TOKENS * input_row_bytes(t.K));
        return true;
    }
    void attention(EgFusedTemplate t, void* k_cache, void* v_cache) {
        t.type = EGF_ATTENTION;
        EgFusedOp op;
        std::memset(&op, 0, sizeof op);
        op.tmpl = intern(t);
        op.unit_offset = next_offset;
        op.k_cache = k_cache;
        op.v_cache = v_cache;
        ops.push_back(op);
        next_offset = (next_offset + tokens * t.num_kv_heads * t.splits) % grid;
        xs_bytes = std::max(xs_bytes, (int)EGF_KV_BYTES);
    }
};

class Mixer : public Part {
public:
    Mixer(const Params& params, const std::string& prefix, std::shared_ptr<PositionEncoding> position) : Part(params, prefix), position(std::move(position)) {}
    virtual bool accepts_pending_norm() const { return false; }
    virtual bool fuses_following_norm() const { return false; }
    virtual CacheNeed cache_need() const { return CacheNeed(); }
    // x [T, hidden] normalised input -> delta [T, hidden], both in ctx.dtype
    virtual Delta forward(const StepContext& ctx, PartInput x, const CacheView& cache, const FollowingNorm* follow) = 0;
    // x = x + this(rmsnorm(x; gain, eps)) as operations of a fused decode program; false: this part cannot say it so
    virtual bool emit_fused(FusedBuilder&, const float* /*gain*/, float /*eps*/, const CacheView&) const { return false; }
    std::shared_ptr<PositionEncoding> position;
};

class FeedForward : public Part {
public:
    using Part::Part;
    virtual bool accepts_pending_norm() const { return false; }
    virtual bool fuses_following_norm() const { return false; }
    virtual Delta forward(const StepContext& ctx, PartInput x, const FollowingNorm* follow) = 0;
    virtual bool emit_fused(FusedBuilder&, const float* /*gain*/, float /*eps*/) const { return false; }
};

class Embedding : public Part {
public:
    using Part::Part;
    virtual void forward(const StepContext& ctx, float* residual) = 0;      // residual[t] = table[token_ids[t]]
    virtual const void* table() const = 0;
    // a plain gather from a bfloat16 table [vocab, hidden] that a fused decode program's first operation can do itself
    virtual bool fused_gather(const void** /*table*/, int* /*vocab*/) const { return false; }
};

class Head : public Part {
public:
    using Part::Part;
    virtual void load_head(const HostTensors&, DType, const void* /*tied_table*/) = 0;
    // normalised rows or a pending norm -> float32 logits [R, vocab] (from the arena)
    virtual float* forward(const StepContext& ctx, PartInput x, int rows) = 0;
    virtual int vocab() const = 0;
    // logits = this(rmsnorm(x; gain, eps)) as the last operation of a fused decode program (sets FusedBuilder::logits)
    virtual bool emit_fused(FusedBuilder&, const float* /*gain*/, float /*eps*/) const { return false; }
};

// ---- registries ---------------------------------------------------------------------------------------------
struct PartRegistry {
    using MixerFactory = std::function<std::shared_ptr<Mixer>(const Params&, const std::string&, std::shared_ptr<PositionEncoding>)>;
    template <class T> using Factory = std::function<std::shared_ptr<T>(const Params&, const std::string&)>;
    std::map<std::string, MixerFactory> mixers;
    std::map<std::string, Factory<FeedForward>> feed_forwards;
    std::map<std::string, Factory<Norm>> norms;
    std::map<std::string, Factory<PositionEncoding>> positions;
    std::map<std::string, Factory<Embedding>> embeddings;
    std::map<std::string, Factory<Head>> heads;

    static PartRegistry& instance() {
        static PartRegistry r;
        return r;
    }
    template <class Map> static const typename Map::mapped_type& find(const Map& m, const char* role, const std::string& kind) {
        auto it = m.find(kind);
        if (it == m.end()) {
            std::string known;
            for (auto& kv : m) known += (known.empty() ? "" : ", ") + kv.first;
            throw std::invalid_argument(std::string("no ") + role + " part of kind '" + kind + "' is registered (known: " + known + ")");
        }
        return it->second;
    }
};

}  // namespace easygpt::engine
