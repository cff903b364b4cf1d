// GptEngine: the entry point.  Token ids in, token ids out.
//
// It mirrors the reference's GptEngine::run (include/gpt_engine.hpp:15-29, src/gpt_engine.cpp:33-43): add the inputs, run
// the model until every request has ended, hand back the outputs — but through the scheduler (csrc/host/scheduler_core.hpp),
// the one step function and the sampling kernels, on the device.  Sampling numbers are keyed by (seed, request, token
// index), so a request's tokens do not depend on what else was in its batches (the reference shares one mt19937 over
// the batch, src/models/gpt_model.cpp:128-129).
#pragma once
#include <chrono>
#include <cstdio>
#include <unordered_map>

#include "../host/scheduler_core.hpp"
#include "step.hpp"

namespace easygpt::engine {

// Sampling options of one request.  Names and meanings are the reference's command line (src/cli_options.cpp:23-47,
// 105-198): temperature > 0, top_p in (0, 1], top_k >= 0 (0 disables), seed >= 0, greedy overrides sampling.
struct SamplingParams {
    float temperature = 0.8f, top_p = 0.95f;
    int top_k = 20;
    long long seed = 42;
    bool greedy = false;
    void validate() const {
        if (!greedy && !(temperature > 0.0f)) throw std::invalid_argument("Temperature must be greater than 0");
        if (!(top_p > 0.0f && top_p <= 1.0f)) throw std::invalid_argument("Top-p must be in (0, 1]");
        if (top_k < 0) throw std::invalid_argument("Top-k must be >= 0");
        if (seed < 0) throw std::invalid_argument("Seed must be >= 0");
    }
    bool is_greedy() const { return greedy || temperature <= 0.0f; }      // src/sampler.cpp:43-49
};

// Counter-based uniform number keyed by (seed, request, token index): three rounds of the splitmix64 finaliser; the top
// 24 bits give a float32-exact number in [0, 1).
inline float uniform_from_counter(uint64_t seed, uint64_t request, uint64_t index) {
    auto mix = [](uint64_t z) {
        z += 0x9E3779B97F4A7C15ull;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    };
    uint64_t z = mix(seed);
    z = mix(z ^ request);
    z = mix(z ^ index);
    return (float)(z >> 40) / 16777216.0f;
}

// --max-steps caps prompt + generated tokens; at least one token is generated (src/continuous_batch_server.cpp:313)
inline long long max_new_tokens_from_max_steps(long long max_steps, long long prompt_len) { return std::max<long long>(1, max_steps - prompt_len + 1); }

struct EngineOptions {
    int page_size = 16;
    long long cache_tokens = 0;             // 0: max_active * min(max positions, 4096)
    int max_active = 16, prefill_batch = 4;
    long long max_batch_tokens = 2048, chunk_size = 512, max_tokens_per_request = 0;
    bool use_graphs = true;
};

struct RequestRecord {
    int64_t id = 0;
    std::vector<int64_t> prompt, output;
    SamplingParams params;
    long long max_new_tokens = 0;
    double added_at = 0;
};

class GptEngine {
public:
    GptEngine(const std::string& model_dir, DType dtype, const EngineOptions& opt) : options(opt) {
        int devices = 0;
        if (cudaGetDeviceCount(&devices) != cudaSuccess || devices == 0) throw DeviceError("GptEngine needs a CUDA device; there is no CPU path");
        model = Model::from_dir(model_dir, dtype);
        const ModelSpec& spec = model->spec;
        long long cache_tokens = opt.cache_tokens > 0 ? opt.cache_tokens : (long long)opt.max_active * std::min<long long>(spec.max_positions, 4096);
        StepRunner::Options ro;
        ro.page_size = opt.page_size;
        ro.num_pages = (int)((cache_tokens + opt.page_size - 1) / opt.page_size);
        ro.max_slots = opt.max_active;
        ro.max_tokens_per_request = opt.max_tokens_per_request > 0 ? opt.max_tokens_per_request
                                                                   : std::min<long long>(spec.max_positions, (long long)ro.num_pages * opt.page_size);
        ro.max_batch_tokens = opt.max_batch_tokens;
        ro.use_graphs = opt.use_graphs;
        runner.reset(new StepRunner(*model, ro));
        host::SchedulerOptions so;
        so.max_batch_tokens = opt.max_batch_tokens;
        so.chunk_size = opt.chunk_size;
        so.max_active = opt.max_active;
        so.prefill_batch = opt.prefill_batch;
        so.eos_token_id = spec.eos_token_id;
        so.max_positions = spec.max_positions;
        if (so.max_batch_tokens <= 0 || so.chunk_size <= 0 || so.max_active <= 0 || so.prefill_batch <= 0) throw std::invalid_argument("scheduler limits must be positive");
        scheduler.reset(new host::SchedulerCore(&runner->cache.core, so));
        const size_t rows = (size_t)std::max(opt.max_active, 1);
        sample_params_dev_.allocate(4 * rows * 4);
        sample_out_dev_.allocate(rows * 4);
        sample_params_host_.ensure(4 * rows * 4);
        sample_out_host_.ensure(rows * 4);
        max_rows_ = rows;
    }

    int64_t add_request(const std::vector<int64_t>& prompt, const SamplingParams& params, long long max_new_tokens) {
        params.validate();
        if (max_new_tokens <= 0) throw std::invalid_argument("max_new_tokens must be positive");
        for (int64_t t : prompt)
            if (t < 0 || t >= model->spec.vocab_size)
                throw std::invalid_argument("token id " + std::to_string(t) + " is outside the vocabulary of " + std::to_string(model->spec.vocab_size));
        RequestRecord r;
        r.id = scheduler->add((long long)prompt.size(), max_new_tokens);
        r.prompt = prompt;
        r.params = params;
        r.max_new_tokens = max_new_tokens;
        r.added_at = now();
        const int64_t id = r.id;
        requests.emplace(id, std::move(r));
        return id;
    }

    // One scheduler round and one model step.  Returns the ids of the requests that finished.
    std::vector<int64_t> step() {
        std::vector<host::ScheduledEntry> batch;
        scheduler->schedule(batch);
        std::vector<int64_t> finished;
        if (batch.empty()) return finished;
        std::vector<StepEntry> entries;
        entries.reserve(batch.size());
        for (auto& s : batch) {
            const RequestRecord& r = requests.at(s.id);
            StepEntry e;
            e.request = s.id;
            e.tokens.resize((size_t)s.count);
            const long long n = (long long)r.prompt.size();
            for (long long k = 0; k < s.count; ++k) {
                const long long pos = s.start + k;
                e.tokens[(size_t)k] = pos < n ? r.prompt[(size_t)pos] : r.output.at((size_t)(pos - n));
            }
            if (s.samples) e.want.push_back(s.count - 1);
            entries.push_back(std::move(e));
        }
        const StepRunner::Result result = runner->run(entries, /*check=*/false, /*commit=*/false, /*reserved=*/true);
        const int rc = scheduler->launched(batch.data(), (int)batch.size());
        if (rc != host::OK) throw StepError("the scheduler failed with status " + std::to_string(rc));
        std::vector<const host::ScheduledEntry*> sampling;
        for (auto& s : batch)
            if (s.samples) sampling.push_back(&s);
        if (!sampling.empty()) {
            const std::vector<long long> tokens = sample(result.logits, sampling);
            std::vector<int> actions(sampling.size());
            const int k = scheduler->resolve(batch.data(), (int)batch.size(), tokens.data(), actions.data());
            if (k < 0) throw StepError("the scheduler failed with status " + std::to_string(k));
            for (size_t i = 0; i < sampling.size(); ++i) {
                if (actions[i] == 0) continue;
                requests.at(sampling[i]->id).output.push_back(tokens[i]);
                if (actions[i] == 2) finished.push_back(sampling[i]->id);
            }
        }
        return finished;
    }

    void run_to_completion() {
        while (scheduler->has_work()) {
            const long long before = scheduler->stats().steps;
            const std::vector<int64_t> done = step();
            if (scheduler->stats().steps == before && done.empty() && scheduler->has_work())
                throw StepError("the scheduler made no progress although requests are waiting");
        }
        runner->check_status();
    }

    // generates for every prompt (lists of token ids) and returns the new tokens of each
    std::vector<std::vector<int64_t>> generate(const std::vector<std::vector<int64_t>>& prompts, const SamplingParams& params, long long max_new_tokens,
                                               long long max_steps) {
        std::vector<int64_t> ids;
        for (auto& p : prompts)
            ids.push_back(add_request(p, params, max_new_tokens > 0 ? max_new_tokens : max_new_tokens_from_max_steps(max_steps > 0 ? max_steps : 100, (long long)p.size())));
        run_to_completion();
        std::vector<std::vector<int64_t>> outputs;
        std::string error;
        for (int64_t id : ids) {
            outputs.push_back(requests.at(id).output);
            const host::SchedRequest* r = scheduler->find(id);
            if (r && r->error && error.empty()) error = "request " + std::to_string(id) + ": " + error_text(id, r->error);
            forget(id);
        }
        if (!error.empty()) throw std::runtime_error(error);
        return outputs;
    }

    std::string error_text(int64_t id, int code) const {
        const size_t n = requests.count(id) ? requests.at(id).prompt.size() : 0;
        if (code == 0) return "";
        if (code == host::ERROR_NO_ROOM_UNDER_MAX_POSITIONS)
            return "prompt of " + std::to_string(n) + " tokens leaves no room under max_position_embeddings=" + std::to_string(model->spec.max_positions);
        if (code == host::ERROR_PROMPT_CANNOT_FIT) return "prompt of " + std::to_string(n) + " tokens cannot fit the cache even alone";
        return "the cache cannot hold this request even alone";
    }
    // drops the record of a finished request (a long-running caller that has read its output)
    void forget(int64_t id) {
        const host::SchedRequest* r = scheduler->find(id);
        if (r && r->state == host::FINISHED) {
            scheduler->forget(id);
            requests.erase(id);
        }
    }

    EngineOptions options;
    std::unique_ptr<Model> model;
    std::unique_ptr<StepRunner> runner;
    std::unique_ptr<host::SchedulerCore> scheduler;
    std::unordered_map<int64_t, RequestRecord> requests;

private:
    static double now() { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); }

    // one kernel launch for the whole batch, greedy rows and sampled rows together; the tokens come back to the host
    std::vector<long long> sample(const float* logits, const std::vector<const host::ScheduledEntry*>& sampling) {
        const size_t rows = sampling.size();
        if (rows > max_rows_) throw StepError("more sampling rows than live requests");
        const int vocab = model->lm_head->vocab();
        cudaStream_t stream = runner->stream;
        bool all_greedy = true;
        for (auto* s : sampling) all_greedy = all_greedy && requests.at(s->id).params.is_greedy();
        int* out = sample_out_dev_.as<int>();
        if (all_greedy) {
            const int blocks = std::max(1, std::min(32, vocab / 4096));
            if (blocks > 1 && rows > KernelScratch::ARGMAX_ROWS) throw StepError("more rows than the argmax kernel's counters");
            if (blocks > 1 && argmax_parts_.bytes() < rows * 32 * 8) argmax_parts_.allocate(std::max(rows, max_rows_) * 32 * 8);
            float* vals = blocks > 1 ? argmax_parts_.as<float>() : nullptr;
            int* idxs = blocks > 1 ? (int*)(argmax_parts_.as<float>() + std::max(rows, max_rows_) * 32) : nullptr;
            launch_check(eg_argmax(stream, logits, vocab, (int)rows, vocab, out, blocks, vals, idxs, blocks > 1 ? scratch_counters() : nullptr), "argmax");
        } else {
            float* h = sample_params_host_.as<float>();
            for (size_t r = 0; r < rows; ++r) {
                const RequestRecord& req = requests.at(sampling[r]->id);
                const SamplingParams& p = req.params;
                const host::SchedRequest* sr = scheduler->find(req.id);
                const uint64_t index = (uint64_t)req.output.size() + (uint64_t)(sr ? sr->pending - 1 : 0);
                h[r] = p.is_greedy() ? 0.0f : p.temperature;
                h[max_rows_ + r] = p.top_p;
                h[2 * max_rows_ + r] = p.is_greedy() ? 0.0f : uniform_from_counter((uint64_t)p.seed, (uint64_t)req.id, index);
                ((int*)h)[3 * max_rows_ + r] = p.top_k;
            }
            EG_CUDA(cudaMemcpyAsync(sample_params_dev_.get(), h, 4 * max_rows_ * 4, cudaMemcpyHostToDevice, stream));
            const float* d = sample_params_dev_.as<float>();
            launch_check(eg_sample(stream, logits, vocab, (int)rows, vocab, d, (const int*)(d + 3 * max_rows_), d + max_rows_, d + 2 * max_rows_, out), "sample");
        }
        EG_CUDA(cudaMemcpyAsync(sample_out_host_.as<int>(), out, rows * 4, cudaMemcpyDeviceToHost, stream));
        EG_CUDA(cudaStreamSynchronize(stream));
        std::vector<long long> tokens(rows);
        for (size_t r = 0; r < rows; ++r) tokens[r] = sample_out_host_.as<int>()[r];
        return tokens;
    }
    int* scratch_counters() {
        if (!argmax_counters_.get()) argmax_counters_.allocate(KernelScratch::ARGMAX_ROWS * 4, true);
        return argmax_counters_.as<int>();
    }

    DeviceBuffer sample_params_dev_, sample_out_dev_, argmax_parts_, argmax_counters_;
    PinnedBuffer sample_params_host_, sample_out_host_;
    size_t max_rows_ = 0;
};

}  // namespace easygpt::engine
