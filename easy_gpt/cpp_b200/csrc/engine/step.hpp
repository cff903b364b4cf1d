// The cache manager's device side and the step function.
//
// DeviceCache: the bookkeeping of csrc/host/cache_core.hpp (pages, block tables, slots) with the device memory it
// addresses: per group of caches with the same needs one tensor [caches, pages + 1, 2 (k, v), kv_heads, page_size,
// head_dim] in the engine's dtype (the extra page is the scratch page that padding rows of a captured batch write
// to), and per cache that asked for fixed-size state one tensor [slots + 1, elements], zeroed when a request takes a slot
// (the extra slot is the scratch slot that padding rows of a captured batch use).
//
// StepRunner: one batch of (request, its next tokens) through the model.  A batch is any mix of prompt portions and
// single decoded tokens, cut anywhere.  run() reserves cache pages for the new tokens (all or nothing), packs the
// batch's metadata into one pinned host buffer, copies it to the device once, runs the model over exactly the tokens
// it was given (reading everything earlier from the cache) and returns float32 logits at the wanted places, in the
// order of the entries and of each entry's `want`.  Steps whose shape repeats are captured as CUDA graphs (decode steps
// per bucket of batch size and context length, other shapes when they have come often enough) and replayed: one copy
// and one graph launch per step; nothing is allocated inside a step.
// (The reference has two entry points that never mix, one for padded prompts and one for single tokens,
// src/models/gpt_model.cpp:375-419, and computes logits at every position, :203-211.)
#pragma once
#include <array>
#include <set>

#include "../host/step_pack.hpp"
#include "model.hpp"

namespace easygpt::engine {

struct StepError : std::runtime_error {
    using std::runtime_error::runtime_error;
};
struct OutOfPages : std::runtime_error {
    using std::runtime_error::runtime_error;
};
struct OutOfSlots : std::runtime_error {
    using std::runtime_error::runtime_error;
};

inline std::string describe_status(int word) {
    std::string out;
    auto add = [&](int bit, const char* text) {
        if (word & bit) out += (out.empty() ? "" : "; ") + std::string(text);
    };
    add(1, "a token id lies outside the vocabulary");
    add(2, "a block table entry needed by attention is not a valid page");
    add(4, "a cache write position lies outside the pool");
    add(8, "a bounded wait inside a kernel gave up");
    return out.empty() ? "ok" : out;
}

class DeviceCache {
public:
    struct Group {
        int index;
        CacheNeed need;
        std::vector<int> cache_ids;
        DeviceBuffer kv;
        int num_pages;
        int scratch_page;
        size_t layer_elems;             // elements of one cache's [pages + 1, 2, kv_heads, page_size, head_dim]
    };
    struct State {
        DeviceBuffer memory;
        size_t bytes_per_slot;
    };

    DeviceCache(const std::map<int, CacheNeed>& needs, int page_size, int num_pages, int max_slots, long long max_tokens_per_request, DType dtype)
        : core(page_size, max_slots, (int)((max_tokens_per_request + page_size - 1) / page_size)), page_size(page_size), max_slots(max_slots), dtype(dtype) {
        if (page_size <= 0 || max_slots <= 0 || max_tokens_per_request <= 0) throw std::invalid_argument("page_size, max_slots and max_tokens_per_request must be positive");
        if (num_pages <= 0) throw std::invalid_argument("a page pool needs at least one page");
        for (auto& kv : needs) {
            const CacheNeed& need = kv.second;
            if (need.kind == CacheNeed::PagedKV) {
                Group* g = nullptr;
                for (auto& have : groups)
                    if (have->need == need) g = have.get();
                if (!g) {
                    groups.emplace_back(new Group());
                    g = groups.back().get();
                    g->index = core.add_group(num_pages, need.window < 0 ? -1 : (int)need.window);
                    g->need = need;
                    g->num_pages = num_pages;
                    g->scratch_page = num_pages;
                    g->layer_elems = (size_t)(num_pages + 1) * 2 * need.num_kv_heads * page_size * need.head_dim;
                }
                g->cache_ids.push_back(kv.first);
                group_of_cache[kv.first] = g->index;
            } else if (need.kind == CacheNeed::State) {
                size_t elems = 1;
                for (long long s : need.state_shape) elems *= (size_t)s;
                State st;
                st.bytes_per_slot = elems * dtype_size(need.state_dtype);
                st.memory.allocate(st.bytes_per_slot * (size_t)(max_slots + 1), true);     // one slot more: the scratch slot of padding rows
                states.emplace(kv.first, std::move(st));
            }
        }
        for (auto& g : groups) g->kv.allocate(g->layer_elems * g->cache_ids.size() * dtype_size(dtype), true);
        fresh_.resize(max_slots);
    }

    CacheView view(int cache_id, bool writes) const {
        CacheView v;
        v.writes = writes;
        auto it = group_of_cache.find(cache_id);
        if (it != group_of_cache.end()) {
            const Group& g = *groups[it->second];
            const size_t which = std::find(g.cache_ids.begin(), g.cache_ids.end(), cache_id) - g.cache_ids.begin();
            const size_t es = dtype_size(dtype);
            char* base = g.kv.as<char>() + which * g.layer_elems * es;
            const long long plane = (long long)g.need.num_kv_heads * page_size * g.need.head_dim;
            v.group = g.index;
            v.k = base;
            v.v = base + (size_t)plane * es;
            v.page_stride = 2 * plane;
            v.head_stride = (long long)page_size * g.need.head_dim;
            v.num_pages = g.num_pages + 1;
            v.page_size = page_size;
            return v;
        }
        auto st = states.find(cache_id);
        if (st != states.end()) {
            v.state = st->second.memory.get();
            v.state_bytes_per_slot = st->second.bytes_per_slot;
        }
        return v;
    }
    // Clears the state of every slot that a request has taken since the last call, whoever began the request.  The step
    // function calls it before every forward pass, captured or not.
    void zero_fresh_state(cudaStream_t stream) {
        const int n = core.take_fresh_slots(fresh_.data(), max_slots);
        if (states.empty()) return;
        for (int i = 0; i < n; ++i)
            for (auto& kv : states)
                EG_CUDA(cudaMemsetAsync(kv.second.memory.as<char>() + (size_t)fresh_[i] * kv.second.bytes_per_slot, 0, kv.second.bytes_per_slot, stream));
    }
    size_t kv_bytes_per_token() const {
        size_t total = 0;
        for (auto& g : groups) total += g->cache_ids.size() * 2 * g->need.num_kv_heads * g->need.head_dim * dtype_size(dtype);
        return total;
    }

    host::CacheCore core;
    int page_size, max_slots;
    DType dtype;
    std::vector<std::unique_ptr<Group>> groups;
    std::map<int, int> group_of_cache;
    std::map<int, State> states;

private:
    std::vector<int> fresh_;
};

struct StepEntry {
    int64_t request;
    std::vector<int64_t> tokens;
    std::vector<int64_t> want;          // indices into tokens whose logits are asked for
};

constexpr int kDecodeBuckets[] = {1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256};
constexpr long long kMinContextBucket = 512;    // tokens: shorter contexts share the smallest captured step

inline int decode_bucket_for(int n) {
    for (int b : kDecodeBuckets)
        if (n <= b) return b;
    return -1;
}
// Block-table width (pages) of the captured step that serves requests of up to `tokens` tokens: the next power of two
// of tokens, at least kMinContextBucket, at most what a request may hold.
inline int context_pages(long long tokens, int page_size, int most) {
    long long bucket = kMinContextBucket;
    while (bucket < tokens) bucket *= 2;
    return (int)std::max<long long>(1, std::min<long long>(most, (bucket + page_size - 1) / page_size));
}

class StepRunner {
public:
    struct Options {
        int page_size = 16;
        int num_pages = 0;
        int max_slots = 16;
        long long max_tokens_per_request = 0;   // 0: min(max positions, pool)
        long long max_batch_tokens = 2048;      // the eager arena is made for steps of up to this many tokens
        bool use_graphs = true;
    };

    StepRunner(Model& model, const Options& opt)
        : model(model), options(opt),
          cache(model.cache_needs(), opt.page_size, opt.num_pages, opt.max_slots,
                opt.max_tokens_per_request > 0 ? opt.max_tokens_per_request
                                               : std::min<long long>(model.spec.max_positions, (long long)opt.num_pages * opt.page_size),
                model.dtype),
          status_(sizeof(int), true) {
        EG_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
        EG_CUDA(cudaMallocHost((void**)&status_host_, sizeof(int)));
        use_graphs = opt.use_graphs && model.capturable();
        if (const char* env = std::getenv("EASY_GPT_FUSED_DECODE")) fused_decode = std::atoi(env) != 0;
        for (auto& e : ring_events_) EG_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    }
    ~StepRunner() {
        graphs_.clear();
        for (auto& e : ring_events_) cudaEventDestroy(e);
        if (status_host_) cudaFreeHost(status_host_);
        if (stream) cudaStreamDestroy(stream);
    }
    StepRunner(const StepRunner&) = delete;
    StepRunner& operator=(const StepRunner&) = delete;

    void end(int64_t request) {
        if (cache.core.find(request)) cache.core.end_request(request);
    }

    struct Result {
        float* logits = nullptr;        // [rows, vocab] float32 on the device, valid until the next step; nullptr if nothing was wanted
        int rows = 0;
        bool captured = false;
    };

    // With `check` the device status word is read back (a synchronisation) and a complaint of a kernel becomes an
    // exception.  With `commit` the requests' cached lengths advance here; a scheduler that keeps its own count passes
    // false (its pages are reserved already: `reserved` true) and commits itself.
    Result run(const std::vector<StepEntry>& entries, bool check = true, bool commit = true, bool reserved = false) {
        validate(entries);
        const int n = (int)entries.size();
        std::vector<int64_t> rids(n), counts(n);
        for (int i = 0; i < n; ++i) {
            rids[i] = entries[i].request;
            counts[i] = (int64_t)entries[i].tokens.size();
        }
        if (!reserved) reserve(entries, rids, counts);
        Result r;
        bool decode = use_graphs;
        for (auto& e : entries)
            if (e.tokens.size() != 1 || e.want.size() != 1 || e.want[0] != 0) decode = false;
        CapturedStep* graph = decode ? decode_graph(n, context_after(rids, 1)) : nullptr;
        if (!graph && use_graphs) graph = signature_graph(entries, rids);
        if (graph) {
            std::vector<int32_t> tokens;
            for (auto& e : entries)
                for (int64_t t : e.tokens) tokens.push_back((int32_t)t);
            r.logits = graph->replay(*this, rids, tokens.data());
            r.rows = graph->padded ? n : graph->rows();
            r.captured = true;
            last_graph = graph;
            ++graph_replays;
            if (graph->is_fused()) ++fused_steps;
        } else {
            r = run_eager(entries, rids, counts);
        }
        if (commit)
            for (int i = 0; i < n; ++i) cache.core.commit(rids[i], counts[i]);
        ++steps_run;
        if (check) check_status();
        return r;
    }

    void check_status() {
        EG_CUDA(cudaMemcpyAsync(status_host_, status_.get(), sizeof(int), cudaMemcpyDeviceToHost, stream));
        EG_CUDA(cudaStreamSynchronize(stream));
        const int word = *status_host_;
        if (word) {
            EG_CUDA(cudaMemsetAsync(status_.get(), 0, sizeof(int), stream));
            throw StepError("a kernel reported: " + describe_status(word));
        }
    }
    int* status() const { return status_.as<int>(); }

    // ---- captured steps ---------------------------------------------------------------------------------------------
    // A step is a fixed sequence of launches once it is known how many tokens every entry brings and where logits are
    // wanted (its *signature*); the only changing inputs are small integer arrays (token ids, positions, cache positions,
    // block tables).  The sequence is captured once over static buffers; a step then costs one host-to-device copy of
    // the arrays and one graph launch.  Decode steps (every entry brings one token) are captured per bucket of batch
    // size and padded with rows that touch only the scratch page; any other signature is captured when it has come
    // often enough.  (The reference captures a graph only for the attention of one layer at batch 1 and re-captures
    // whenever a pointer changes, src/cuda/ops/self_attn.cu:750-828.)
    class CapturedStep {
    public:
        // counts: tokens per entry; wants: per entry the places whose logits are wanted; padded: fewer entries than the
        // signature's may be replayed (decode buckets); table_width: pages per block-table row that the step carries
        CapturedStep(StepRunner& r, std::vector<int32_t> counts, const std::vector<std::vector<int64_t>>& wants, bool padded, int table_width)
            : entries((int)counts.size()), table_width(table_width), padded(padded), counts_(std::move(counts)) {
            DeviceCache& cache = r.cache;
            const int G = (int)cache.groups.size();
            const int n = entries;
            std::vector<int32_t> starts(n + 1, 0), token_seq, rows, tiles, small;
            for (int i = 0; i < n; ++i) {
                starts[i + 1] = starts[i] + counts_[i];
                for (int k = 0; k < counts_[i]; ++k) token_seq.push_back(i);
                for (int64_t w : wants[i]) rows.push_back(starts[i] + (int32_t)w);
                if (counts_[i] > plans::SMALL_ENTRY_TOKENS)
                    for (int o = 0; o < counts_[i]; o += plans::QUERY_TILE) {
                        tiles.push_back(i);
                        tiles.push_back(starts[i] + o);
                        tiles.push_back(std::min(plans::QUERY_TILE, counts_[i] - o));
                    }
                else
                    for (int k = 0; k < counts_[i]; ++k) small.push_back(starts[i] + k);
            }
            tokens = starts[n];
            num_rows_ = (int)rows.size();
            all_rows_ = num_rows_ == tokens;
            for (int i = 0; all_rows_ && i < tokens; ++i) all_rows_ = rows[i] == i;
            num_tiles_ = (int)tiles.size() / 3;
            num_small_ = num_tiles_ ? (int)small.size() : 0;
            max_query_ = *std::max_element(counts_.begin(), counts_.end());
            auto section = [&](long long size) {
                const long long at = size_;
                size_ += host::pad4(size);
                return at;
            };
            // what changes from step to step comes first (one copy), what depends on the signature alone behind it
            off_tokens_ = section(tokens);
            off_positions_ = section(tokens);
            off_context_ = section(n);
            off_slots_ = section(n);
            for (int g = 0; g < G; ++g) {
                off_slot_map_.push_back(section(tokens));
                off_table_.push_back(section((long long)n * table_width));
            }
            changing_ = size_;
            off_token_seq_ = section(tokens);
            off_starts_ = section(n + 1);
            off_rows_ = section(num_rows_);
            off_tiles_ = section((long long)tiles.size());
            off_small_ = section((long long)small.size());
            meta_.allocate((size_t)size_ * 4, true);
            for (auto& st : staging_) st.ensure((size_t)size_ * 4);
            for (auto& e : events_) EG_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
            r.ensure_arenas(r.model.activation_bytes(tokens, num_rows_));      // before anything of this step is captured: growing drops every captured step
            int32_t* hv = staging_[0].as<int32_t>();
            std::fill(hv, hv + size_, 0);
            std::copy(token_seq.begin(), token_seq.end(), hv + off_token_seq_);
            std::copy(starts.begin(), starts.end(), hv + off_starts_);
            std::copy(rows.begin(), rows.end(), hv + off_rows_);
            std::copy(tiles.begin(), tiles.end(), hv + off_tiles_);
            std::copy(small.begin(), small.end(), hv + off_small_);
            fill_padding(r, hv, 0);                  // every row reads and writes the scratch page until a replay says otherwise
            EG_CUDA(cudaMemcpyAsync(meta_.get(), hv, (size_t)size_ * 4, cudaMemcpyHostToDevice, r.stream));
            EG_CUDA(cudaStreamSynchronize(r.stream));
            for (auto& st : staging_)
                if (st.as<int32_t>() != hv) std::memcpy(st.as<int32_t>(), hv, (size_t)size_ * 4);
            // small decode steps: the whole step as one persistent kernel, if the model's parts can say it so
            if (padded && tokens <= EGF_MAX_TOKENS && r.fused_decode) {
                StepContext ctx = context(r);
                Model::FusedProgram prog = r.model.fused_program(ctx, *r.arenas_, [&](int c, bool w) { return r.cache.view(c, w); });
                if (prog.ok()) {
                    const size_t tb = prog.tmpls.size() * sizeof(EgFusedTemplate), ob = prog.ops.size() * sizeof(EgFusedOp);
                    fused_tmpls_.allocate(tb);
                    fused_ops_.allocate(ob);
                    fused_sync_.allocate(256, true);
                    EG_CUDA(cudaMemcpy(fused_tmpls_.get(), prog.tmpls.data(), tb, cudaMemcpyHostToDevice));
                    EG_CUDA(cudaMemcpy(fused_ops_.get(), prog.ops.data(), ob, cudaMemcpyHostToDevice));
                    fused_ = prog;
                    if (std::getenv("EASY_GPT_FUSED_TRACE")) fused_trace_.allocate(prog.ops.size() * 4 * sizeof(unsigned long long), true);
                }
            }
            // run once eagerly (library plans come into being), then capture
            forward(r);
            EG_CUDA(cudaStreamSynchronize(r.stream));
            EG_CUDA(cudaStreamBeginCapture(r.stream, cudaStreamCaptureModeThreadLocal));
            try {
                logits_ = forward(r);
            } catch (...) {
                cudaGraph_t broken = nullptr;
                cudaStreamEndCapture(r.stream, &broken);
                if (broken) cudaGraphDestroy(broken);
                throw;
            }
            cudaGraph_t graph = nullptr;
            EG_CUDA(cudaStreamEndCapture(r.stream, &graph));
            size_t nodes = 0;
            cudaGraphGetNodes(graph, nullptr, &nodes);
            launches = (int)nodes;
            const cudaError_t e = cudaGraphInstantiate(&exec_, graph, 0);
            cudaGraphDestroy(graph);
            cuda_check(e, "cudaGraphInstantiate");
        }
        ~CapturedStep() {
            if (exec_) cudaGraphExecDestroy(exec_);
            for (auto& e : events_) cudaEventDestroy(e);
        }
        CapturedStep(const CapturedStep&) = delete;
        CapturedStep& operator=(const CapturedStep&) = delete;

        // rids: the live requests of this step in the signature's order (fewer than the signature's only if it is padded);
        // pages for their new tokens are reserved.  token_ids: their token ids, flat, in order, or nullptr if the device
        // already holds them (see token_ids()).  Returns the logits [rows, vocab]; rows of padding entries are to be ignored.
        float* replay(StepRunner& r, const std::vector<int64_t>& rids, const int32_t* token_ids) {
            const int n = (int)rids.size();
            const int turn = next_++ % (int)staging_.size();
            if (used_[turn]) EG_CUDA(cudaEventSynchronize(events_[turn]));
            int32_t* hv = staging_[turn].as<int32_t>();
            int live_tokens = 0;
            for (int i = 0; i < n; ++i) live_tokens += counts_[i];
            if (token_ids) std::memcpy(hv + off_tokens_, token_ids, (size_t)live_tokens * 4);
            const int rc = host::pack_replay(r.cache.core, n, rids.data(), counts_.data(), hv, off_positions_, off_context_, off_slots_,
                                             off_slot_map_.data(), off_table_.data(), table_width);
            if (rc != host::OK)
                throw StepError(rc == host::NO_PAGE ? "a token of a captured step has no cache page"
                                                    : "packing a captured step failed with status " + std::to_string(rc));
            if (n < entries) fill_padding(r, hv, n);
            // token ids, when they are on the device already (the sampler's output was copied in), stay as they are
            const long long first = token_ids ? 0 : off_positions_;
            EG_CUDA(cudaMemcpyAsync(meta_.as<int32_t>() + first, hv + first, (size_t)(changing_ - first) * 4, cudaMemcpyHostToDevice, r.stream));
            EG_CUDA(cudaEventRecord(events_[turn], r.stream));
            used_[turn] = true;
            r.cache.zero_fresh_state(r.stream);
            EG_CUDA(cudaGraphLaunch(exec_, r.stream));
            return logits_;
        }
        int32_t* token_ids() const { return meta_.as<int32_t>() + off_tokens_; }
        size_t meta_bytes() const { return (size_t)changing_ * 4; }      // what a replay copies to the device
        int rows() const { return num_rows_; }
        const int entries, table_width;
        const bool padded;
        int tokens = 0;
        int launches = 0;               // nodes of the captured graph: the kernels one replay launches

    private:
        // rows from first_row on are padding (every entry of a padded signature brings one token)
        void fill_padding(StepRunner& r, int32_t* hv, int first_row) {
            int first_token = 0;
            for (int i = 0; i < first_row; ++i) first_token += counts_[i];
            for (int t = first_token; t < tokens; ++t) hv[off_tokens_ + t] = hv[off_positions_ + t] = 0;
            for (int i = first_row; i < entries; ++i) {
                hv[off_context_ + i] = 0;
                hv[off_slots_ + i] = r.cache.max_slots;           // the scratch slot: no request's state
            }
            for (size_t g = 0; g < r.cache.groups.size(); ++g) {
                const int scratch = r.cache.groups[g]->scratch_page;
                for (int t = first_token; t < tokens; ++t) hv[off_slot_map_[g] + t] = scratch * r.cache.page_size;
                std::fill(hv + off_table_[g] + (long long)first_row * table_width, hv + off_table_[g] + (long long)entries * table_width, scratch);
            }
        }
        float* forward(StepRunner& r) {
            if (fused_.ok()) {
                launch_check(eg_decode_fused(r.stream, fused_tmpls_.get(), (int)fused_.tmpls.size(), fused_ops_.get(), (int)fused_.ops.size(), fused_.tokens,
                                             fused_.stages, fused_.xs_bytes, fused_.grid, fused_sync_.as<unsigned>(), r.status(),
                                             fused_trace_.get() ? fused_trace_.as<unsigned long long>() : nullptr), "decode_fused");
                return fused_.logits;
            }
            StepContext ctx = context(r);
            return r.model.forward(ctx, *r.arenas_, [&](int c, bool w) { return r.cache.view(c, w); }, all_rows_ ? nullptr : ctx_rows(), num_rows_, all_rows_);
        }
        const int* ctx_rows() const { return meta_.as<int32_t>() + off_rows_; }
        StepContext context(StepRunner& r) {
            StepContext ctx;
            ctx.dtype = r.model.dtype;
            ctx.stream = r.stream;
            ctx.blas = &r.blas_;
            ctx.scratch = &r.scratch_;
            ctx.num_tokens = tokens;
            ctx.num_seqs = entries;
            const int32_t* m = meta_.as<int32_t>();
            ctx.token_ids = m + off_tokens_;
            ctx.positions = m + off_positions_;
            ctx.token_seq = m + off_token_seq_;
            ctx.seq_starts = m + off_starts_;
            ctx.seq_context = m + off_context_;
            ctx.seq_slots = m + off_slots_;
            ctx.status = r.status();
            for (size_t g = 0; g < r.cache.groups.size(); ++g)
                ctx.groups.push_back(GroupTables{r.cache.page_size, m + off_table_[g], table_width, m + off_slot_map_[g]});
            ctx.max_query_len = max_query_;
            ctx.max_context_len = (long long)table_width * r.cache.page_size;
            ctx.all_decode = max_query_ == 1;
            if (num_tiles_) {
                ctx.query_tiles = m + off_tiles_;
                ctx.num_tiles = num_tiles_;
                if (num_small_) {
                    ctx.small_tokens = m + off_small_;
                    ctx.num_small = num_small_;
                }
            }
            return ctx;
        }

        long long size_ = 0, changing_ = 0, off_tokens_ = 0, off_positions_ = 0, off_context_ = 0, off_slots_ = 0, off_token_seq_ = 0, off_starts_ = 0,
                  off_rows_ = 0, off_tiles_ = 0, off_small_ = 0;
        std::vector<long long> off_slot_map_, off_table_;
        std::vector<int32_t> counts_;
        int num_rows_ = 0, num_tiles_ = 0, num_small_ = 0, max_query_ = 1;
        bool all_rows_ = false;
        DeviceBuffer meta_;
        std::array<PinnedBuffer, 4> staging_;
        std::array<cudaEvent_t, 4> events_{};
        std::array<bool, 4> used_{};
        int next_ = 0;
        cudaGraphExec_t exec_ = nullptr;
        float* logits_ = nullptr;
        Model::FusedProgram fused_;
        DeviceBuffer fused_tmpls_, fused_ops_, fused_sync_, fused_trace_;
    public:
        bool is_fused() const { return fused_.ok(); }
        // The stamps of the fused kernel's last run (EASY_GPT_FUSED_TRACE=1), one row per operation: when the last CTA
        // entered it, had its input rows, had its products, left it (GPU nanoseconds), and what kind of operation it was;
        // the rows are cleared for the next run.
        std::vector<std::array<unsigned long long, 5>> fused_trace(cudaStream_t stream) {
            std::vector<std::array<unsigned long long, 5>> rows;
            if (!fused_trace_.get()) return rows;
            std::vector<unsigned long long> raw(fused_.ops.size() * 4);
            EG_CUDA(cudaStreamSynchronize(stream));
            EG_CUDA(cudaMemcpy(raw.data(), fused_trace_.get(), raw.size() * 8, cudaMemcpyDeviceToHost));
            EG_CUDA(cudaMemset(fused_trace_.get(), 0, raw.size() * 8));
            for (size_t i = 0; i < fused_.ops.size(); ++i) {
                const EgFusedTemplate& t = fused_.tmpls[fused_.ops[i].tmpl];
                const unsigned long long kind = t.type == EGF_ATTENTION ? 100ull : (unsigned long long)(t.input * 10 + t.output);
                rows.push_back({raw[4 * i], raw[4 * i + 1], raw[4 * i + 2], raw[4 * i + 3], kind});
            }

            return rows;
        }
    };
    using DecodeGraph = CapturedStep;

    // tokens the longest of these requests holds once the step's tokens are in
    long long context_after(const std::vector<int64_t>& rids, long long most_new_tokens) const {
        long long longest = 0;
        for (int64_t rid : rids)
            if (const host::CachedRequest* c = cache.core.find(rid)) longest = std::max(longest, c->length);
        return longest + most_new_tokens;
    }
    // the captured step for n single-token entries whose requests hold up to `context` tokens after it; nullptr if n is
    // beyond the buckets
    DecodeGraph* decode_graph(int n, long long context) {
        if (!use_graphs) return nullptr;
        int b = decode_bucket_for(n);
        if (b < 0 || b > cache.max_slots) b = n <= cache.max_slots ? cache.max_slots : -1;
        if (b < 0) return nullptr;
        const int width = context_pages(context, cache.page_size, cache.core.max_pages_per_request());
        auto key = std::make_pair(b, width);
        auto it = graphs_.find(key);
        if (it == graphs_.end())
            it = graphs_.emplace(key, std::unique_ptr<CapturedStep>(new CapturedStep(*this, std::vector<int32_t>(b, 1), std::vector<std::vector<int64_t>>(b, {0}), true, width))).first;
        last_graph = it->second.get();
        return last_graph;
    }

    // The captured step for this exact batch shape (and context bucket), once the shape has come often enough; nullptr
    // before that.  A capture costs about as much as six eager steps.  One request's portions come again and again; a
    // batch of several requests rarely comes twice in the same shape, so it has to show that it does before it is captured.
    CapturedStep* signature_graph(const std::vector<StepEntry>& entries, const std::vector<int64_t>& rids) {
        if (!use_graphs) return nullptr;
        Signature sig;
        long long total = 0, most = 0;
        for (auto& e : entries) {
            sig.counts.push_back((int32_t)e.tokens.size());
            sig.wants.push_back(e.want);
            total += (long long)e.tokens.size();
            most = std::max<long long>(most, (long long)e.tokens.size());
        }
        sig.width = context_pages(context_after(rids, most), cache.page_size, cache.core.max_pages_per_request());
        auto it = signature_graphs_.find(sig);
        if (it != signature_graphs_.end()) {
            it->second.last_used = ++signature_clock_;
            return it->second.graph.get();
        }
        const int seen = ++signature_seen_[sig];
        if (signature_seen_.size() > 4096) signature_seen_.clear();
        if (seen < (entries.size() == 1 ? kCaptureAfter : kCaptureMixedAfter) || total > 16384) return nullptr;
        if (signature_graphs_.size() >= kMaxSignatureGraphs) {          // the least recently used goes
            auto oldest = signature_graphs_.begin();
            for (auto i = signature_graphs_.begin(); i != signature_graphs_.end(); ++i)
                if (i->second.last_used < oldest->second.last_used) oldest = i;
            EG_CUDA(cudaStreamSynchronize(stream));
            signature_graphs_.erase(oldest);
        }
        SignatureGraph made;
        made.graph.reset(new CapturedStep(*this, sig.counts, sig.wants, false, sig.width));
        made.last_used = ++signature_clock_;
        return signature_graphs_.emplace(sig, std::move(made)).first->second.graph.get();
    }
    // One set of arenas serves every step, captured or not: steps run one after the other on one stream.  It is made
    // for steps of max_batch_tokens tokens; a larger step makes it grow, which takes every captured step with it (their
    // graphs hold addresses inside the old arenas).
    void ensure_arenas(const ArenaSizes& need) {
        if (arenas_ && arenas_->holds(need)) return;
        EG_CUDA(cudaStreamSynchronize(stream));
        graphs_.clear();
        signature_graphs_.clear();
        last_graph = nullptr;
        const ArenaSizes usual = model.activation_bytes(options.max_batch_tokens, std::max(options.max_slots, 256));
        arenas_.reset();
        arenas_.reset(new StepArenas(ArenaSizes{std::max(need.step, usual.step), std::max(need.sub, usual.sub)}));
    }
    // (Measured with 64 requests of 128 to 4096 prompt tokens in portions of 512 beside decoding requests, at the 0.5B
    // sizes: 1.09 s without captures of mixed shapes, 1.18 s when they were captured at their fourth coming: launching
    // from C++ is not what such steps wait for, and every capture costs about three steps.)
    static constexpr int kCaptureAfter = 2, kCaptureMixedAfter = 16;
    static constexpr size_t kMaxSignatureGraphs = 48;
    size_t signature_graph_count() const { return signature_graphs_.size(); }

    Model& model;
    Options options;
    DeviceCache cache;
    cudaStream_t stream = nullptr;
    bool use_graphs = false;
    // Decode steps of up to EGF_MAX_TOKENS tokens as one persistent kernel (csrc/decode_fused.cu) instead of a chain of
    // kernels.  Off unless EASY_GPT_FUSED_DECODE=1: measured on B200 at the Qwen2.5-0.5B sizes it takes 1.38 ms a step
    // where the chain takes 0.85 (a barrier across the grid costs 2.8 us, a launch boundary of the chain 0.9).
    bool fused_decode = false;
    long long steps_run = 0, graph_replays = 0, fused_steps = 0;      // fused_steps: replays that ran as one persistent kernel
    DecodeGraph* last_graph = nullptr;

private:
    void validate(const std::vector<StepEntry>& entries) const {
        if (entries.empty()) throw StepError("a step needs at least one entry");
        std::set<int64_t> seen;
        for (auto& e : entries) {
            if (!seen.insert(e.request).second) throw StepError("request " + std::to_string(e.request) + " appears twice in one step");
            if (e.tokens.empty()) throw StepError("request " + std::to_string(e.request) + " brings no tokens");
            for (int64_t w : e.want)
                if (w < 0 || w >= (int64_t)e.tokens.size())
                    throw StepError("request " + std::to_string(e.request) + ": wanted place " + std::to_string(w) + " is outside its " +
                                    std::to_string(e.tokens.size()) + " tokens");
            for (int64_t t : e.tokens)
                if (t < INT32_MIN || t > INT32_MAX) throw StepError("token ids do not fit 32 bits");
        }
    }
    // begins the step's new requests and takes the pages for every entry's tokens: all of it, or an exception with nothing changed
    void reserve(const std::vector<StepEntry>& entries, const std::vector<int64_t>& rids, const std::vector<int64_t>& counts) {
        int info[3] = {0, 0, 0};
        const int rc = host::reserve_step(cache.core, (int)rids.size(), rids.data(), counts.data(), info);
        if (rc == host::OK) return;
        if (rc == host::OUT_OF_PAGES)
            throw OutOfPages("group " + std::to_string(info[0]) + ": the step needs " + std::to_string(info[1]) + " new pages, " + std::to_string(info[2]) + " are free");
        if (rc == host::TOO_LONG)
            throw OutOfPages("request " + std::to_string(entries[info[0]].request) + " would hold more tokens than a request may hold (" +
                             std::to_string((long long)cache.core.max_pages_per_request() * cache.page_size) + ")");
        if (rc == host::OUT_OF_SLOTS) throw OutOfSlots("all " + std::to_string(cache.max_slots) + " request slots are taken");
        throw StepError("reserving the step's pages failed with status " + std::to_string(rc));
    }

    Result run_eager(const std::vector<StepEntry>& entries, const std::vector<int64_t>& rids, const std::vector<int64_t>& counts) {
        const int n = (int)entries.size();
        const int G = (int)cache.groups.size();
        long long T = 0, R = 0;
        std::vector<int64_t> token_ids, want_offsets(n + 1, 0), wants;
        for (int i = 0; i < n; ++i) {
            T += counts[i];
            token_ids.insert(token_ids.end(), entries[i].tokens.begin(), entries[i].tokens.end());
            wants.insert(wants.end(), entries[i].want.begin(), entries[i].want.end());
            want_offsets[i + 1] = (int64_t)wants.size();
        }
        R = (long long)wants.size();
        const long long bound = host::packed_step_bound(cache.core, n, T, R, plans::QUERY_TILE);
        // pinned staging buffers in a ring: a buffer is rewritten only after the copy that read it has finished
        const int turn = ring_next_++ % (int)ring_.size();
        if (ring_used_[turn]) EG_CUDA(cudaEventSynchronize(ring_events_[turn]));
        ring_[turn].ensure((size_t)bound * 4);
        if (dev_meta_.bytes() < (size_t)bound * 4) {
            EG_CUDA(cudaStreamSynchronize(stream));
            size_t cap = 1u << 16;
            while (cap < (size_t)bound * 4) cap *= 2;
            dev_meta_.allocate(cap);
        }
        std::vector<long long> layout(2 * (host::FIXED_SECTIONS + 2 * G));
        std::vector<int> widths(std::max(G, 1));
        host::PackedStep packed;
        if (wants.empty()) wants.push_back(0);
        const int rc = host::pack_step(cache.core, n, rids.data(), counts.data(), token_ids.data(), want_offsets.data(), wants.data(), plans::QUERY_TILE,
                                       plans::SMALL_ENTRY_TOKENS, ring_[turn].as<int32_t>(), bound, layout.data(), widths.data(), &packed);
        if (rc != host::OK) throw StepError("packing the step failed with status " + std::to_string(rc));
        EG_CUDA(cudaMemcpyAsync(dev_meta_.get(), ring_[turn].as<int32_t>(), (size_t)packed.total * 4, cudaMemcpyHostToDevice, stream));
        EG_CUDA(cudaEventRecord(ring_events_[turn], stream));
        ring_used_[turn] = true;

        ensure_arenas(model.activation_bytes(T, R));
        const int32_t* m = dev_meta_.as<int32_t>();
        const int32_t* hv = ring_[turn].as<int32_t>();
        auto at = [&](int section) { return m + layout[2 * section]; };
        StepContext ctx;
        ctx.dtype = model.dtype;
        ctx.stream = stream;
        ctx.blas = &blas_;
        ctx.scratch = &scratch_;
        ctx.num_tokens = (int)T;
        ctx.num_seqs = n;
        ctx.token_ids = at(host::TOKEN_IDS);
        ctx.positions = at(host::POSITIONS);
        ctx.token_seq = at(host::TOKEN_SEQ);
        ctx.seq_starts = at(host::SEQ_STARTS);
        ctx.seq_context = at(host::SEQ_CONTEXT);
        ctx.seq_slots = at(host::SEQ_SLOTS);
        ctx.host_seq_starts = hv + layout[2 * host::SEQ_STARTS];
        ctx.host_seq_context = hv + layout[2 * host::SEQ_CONTEXT];
        ctx.host_seq_slots = hv + layout[2 * host::SEQ_SLOTS];
        ctx.status = status();
        for (int g = 0; g < G; ++g)
            ctx.groups.push_back(GroupTables{cache.page_size, at(host::FIXED_SECTIONS + 2 * g + 1), widths[g], at(host::FIXED_SECTIONS + 2 * g)});
        ctx.max_query_len = (int)packed.max_query_len;
        ctx.max_context_len = packed.max_context_len;
        ctx.all_decode = packed.all_decode != 0;
        if (packed.num_tiles) {
            ctx.query_tiles = at(host::QUERY_TILES);
            ctx.num_tiles = packed.num_tiles;
            if (packed.num_small) {
                ctx.small_tokens = at(host::SMALL_TOKENS);
                ctx.num_small = packed.num_small;
            }
        }
        cache.zero_fresh_state(stream);         // slots taken since the last step (by this step or by the scheduler)
        Result r;
        r.logits = model.forward(ctx, *arenas_, [&](int c, bool w) { return cache.view(c, w); }, R ? at(host::LOGIT_ROWS) : nullptr, (int)R, false);
        r.rows = (int)R;
        return r;
    }

    DeviceBuffer status_;
    int* status_host_ = nullptr;
    Blas blas_;
    KernelScratch scratch_;
    std::unique_ptr<StepArenas> arenas_;
    std::array<PinnedBuffer, 4> ring_;
    std::array<cudaEvent_t, 4> ring_events_{};
    std::array<bool, 4> ring_used_{};
    int ring_next_ = 0;
    DeviceBuffer dev_meta_;
    std::map<std::pair<int, int>, std::unique_ptr<CapturedStep>> graphs_;
    struct Signature {
        std::vector<int32_t> counts;
        std::vector<std::vector<int64_t>> wants;
        int width = 0;
        bool operator<(const Signature& o) const { return std::tie(counts, wants, width) < std::tie(o.counts, o.wants, o.width); }
    };
    struct SignatureGraph {
        std::unique_ptr<CapturedStep> graph;
        long long last_used = 0;
    };
    std::map<Signature, SignatureGraph> signature_graphs_;
    std::map<Signature, int> signature_seen_;
    long long signature_clock_ = 0;
};

}  // namespace easygpt::engine
