// C interface of the native engine (libeasygpt_engine.so) for the Python face (native.py), bin/trace_run and any other
// caller.  Handles are opaque pointers.  Functions return 0 or a non-negative result on success and -1 on failure, with the
// error text in the caller's buffer.  Nothing here is specific to one architecture: the model class is chosen by config.json.
#include <dlfcn.h>

#include <cstring>

#include "engine.hpp"

using namespace easygpt::engine;
namespace host = easygpt::host;

#define EGE_API extern "C" __attribute__((visibility("default")))

namespace {
void put_error(char* buffer, int cap, const std::string& text) {
    if (!buffer || cap <= 0) return;
    std::strncpy(buffer, text.c_str(), (size_t)cap - 1);
    buffer[cap - 1] = 0;
}
DType dtype_from(const char* name) {
    const std::string s = name ? name : "";
    if (s == "bfloat16" || s == "bf16") return DType::BF16;
    if (s == "float32" || s == "fp32") return DType::F32;
    throw std::invalid_argument("dtype must be bfloat16 or float32, not '" + s + "'");
}
template <class F> long long guarded(char* error, int cap, F f) {
    try {
        return f();
    } catch (const std::exception& e) {
        put_error(error, cap, e.what());
        return -1;
    }
}
struct Runner {
    std::unique_ptr<Model> model;
    std::unique_ptr<StepRunner> runner;
    std::vector<float> host_logits;
};
}  // namespace

// ---- plugins: parts and architectures from outside the library ------------------------------------------------------------
// A plugin is a shared library built against the engine's headers (csrc/engine/plugin.hpp) that exports
//     extern "C" void easygpt_register(easygpt::engine::PartRegistry*, easygpt::engine::ArchitectureRegistry*);
// It is loaded once, stays loaded, and adds its mixers, feed-forwards, norms, position encodings, embeddings, heads and
// architectures to the registries that models are built from.  Nothing of the library's sources changes for it.
EGE_API long long ege_load_plugin(const char* path, char* error, int cap) {
    return guarded(error, cap, [&]() {
        register_builtin_parts();
        register_builtin_architectures();
        void* handle = dlopen(path, RTLD_NOW | RTLD_LOCAL);
        if (!handle) throw std::runtime_error(std::string("cannot load the plugin ") + path + ": " + dlerror());
        using RegisterFn = void (*)(PartRegistry*, ArchitectureRegistry*);
        RegisterFn fn = reinterpret_cast<RegisterFn>(dlsym(handle, "easygpt_register"));
        if (!fn) throw std::runtime_error(std::string(path) + " exports no easygpt_register");
        fn(&PartRegistry::instance(), &ArchitectureRegistry::instance());
        return 0;
    });
}

// ---- the engine ---------------------------------------------------------------------------------------------------
// options (8 long longs): page_size, cache_tokens (0: default), max_active, prefill_batch, max_batch_tokens, chunk_size,
// max_tokens_per_request (0: default), use_graphs
EGE_API void* ege_engine_create(const char* model_dir, const char* dtype, const long long* options, char* error, int cap) {
    GptEngine* engine = nullptr;
    guarded(error, cap, [&]() {
        EngineOptions o;
        o.page_size = (int)options[0];
        o.cache_tokens = options[1];
        o.max_active = (int)options[2];
        o.prefill_batch = (int)options[3];
        o.max_batch_tokens = options[4];
        o.chunk_size = options[5];
        o.max_tokens_per_request = options[6];
        o.use_graphs = options[7] != 0;
        engine = new GptEngine(model_dir, dtype_from(dtype), o);
        return 0;
    });
    return engine;
}
EGE_API void ege_engine_destroy(void* e) { delete static_cast<GptEngine*>(e); }

EGE_API long long ege_engine_add_request(void* e, const long long* prompt, long long n, float temperature, float top_p, int top_k, long long seed,
                                         int greedy, long long max_new_tokens, char* error, int cap) {
    return guarded(error, cap, [&]() {
        SamplingParams p;
        p.temperature = temperature;
        p.top_p = top_p;
        p.top_k = top_k;
        p.seed = seed;
        p.greedy = greedy != 0;
        return (long long)static_cast<GptEngine*>(e)->add_request(std::vector<int64_t>(prompt, prompt + n), p, max_new_tokens);
    });
}
// one scheduler round and one model step; the ids of the requests that finished go to `finished` (at most cap_finished)
EGE_API long long ege_engine_step(void* e, long long* finished, int cap_finished, char* error, int cap) {
    return guarded(error, cap, [&]() {
        const std::vector<int64_t> done = static_cast<GptEngine*>(e)->step();
        for (size_t i = 0; i < done.size() && (int)i < cap_finished; ++i) finished[i] = done[i];
        return (long long)done.size();
    });
}
EGE_API int ege_engine_has_work(void* e) { return static_cast<GptEngine*>(e)->scheduler->has_work() ? 1 : 0; }
EGE_API long long ege_engine_run_to_completion(void* e, char* error, int cap) {
    return guarded(error, cap, [&]() {
        static_cast<GptEngine*>(e)->run_to_completion();
        return 0;
    });
}
// the tokens generated so far for a request; returns how many there are, writes what fits
EGE_API long long ege_engine_output(void* e, long long id, long long* out, long long cap_out) {
    GptEngine* g = static_cast<GptEngine*>(e);
    auto it = g->requests.find(id);
    if (it == g->requests.end()) return -1;
    const auto& tokens = it->second.output;
    for (size_t i = 0; i < tokens.size() && (long long)i < cap_out; ++i) out[i] = tokens[i];
    return (long long)tokens.size();
}
// out (10 long longs): prompt length, output length, max new tokens, computed, state (0 waiting, 1 running, 2 finished),
// finish reason (1 empty, 2 eos, 3 length, 4 max positions, 5 error), error code, pending, preemptions, admission counter
EGE_API int ege_engine_request(void* e, long long id, long long* out, char* error_text, int cap) {
    GptEngine* g = static_cast<GptEngine*>(e);
    const host::SchedRequest* r = g->scheduler->find(id);
    if (!r) return -1;
    out[0] = r->prompt_len; out[1] = r->output_len; out[2] = r->max_new_tokens; out[3] = r->computed; out[4] = r->state;
    out[5] = r->reason; out[6] = r->error; out[7] = r->pending; out[8] = r->preemptions; out[9] = r->admitted_at;
    put_error(error_text, cap, g->error_text(id, r->error));
    return 0;
}
EGE_API void ege_engine_forget(void* e, long long id) { static_cast<GptEngine*>(e)->forget(id); }
// out (12 long longs): scheduler steps, prompt tokens, decode tokens, preemptions, finished, failed, captured-step replays,
// steps run, live requests, free pages of group 0, vocabulary, bytes of weights a step reads
EGE_API void ege_engine_stats(void* e, long long* out) {
    GptEngine* g = static_cast<GptEngine*>(e);
    const host::SchedulerStats& st = g->scheduler->stats();
    out[0] = st.steps; out[1] = st.prompt_tokens; out[2] = st.decode_tokens; out[3] = st.preemptions; out[4] = st.finished; out[5] = st.failed;
    out[6] = g->runner->graph_replays;
    out[7] = g->runner->steps_run;
    out[8] = (long long)g->runner->cache.core.live_count();
    out[9] = g->runner->cache.groups.empty() ? 0 : g->runner->cache.core.group(0).pool.free_count();
    out[10] = g->model->spec.vocab_size;
    out[11] = (long long)g->model->weight_bytes_per_step();
}
// further figures for roofline arithmetic: what == 0: cache bytes per token, 1: bytes of metadata the last captured step
// copied to the device, 2: tokens of request `id` in the cache (-1 if it is not live), 3: kernels one replay of the last
// captured step launches (the nodes of its graph)
EGE_API long long ege_engine_figure(void* e, int what, long long id) {
    GptEngine* g = static_cast<GptEngine*>(e);
    if (what == 0) return (long long)g->runner->cache.kv_bytes_per_token();
    if (what == 1) return g->runner->last_graph ? (long long)g->runner->last_graph->meta_bytes() : 0;
    if (what == 2) {
        const host::CachedRequest* r = g->runner->cache.core.find(id);
        return r ? r->length : -1;
    }
    if (what == 3) return g->runner->last_graph ? g->runner->last_graph->launches : 0;
    if (what == 4) return g->runner->fused_steps;
    return -1;
}
// The fused decode kernel's stamps of the last step (see CapturedStep::fused_trace): rows of five numbers into `out`;
// returns the number of rows (0 if the last step was not a fused one or EASY_GPT_FUSED_TRACE is not set).
EGE_API long long ege_engine_fused_trace(void* e, unsigned long long* out, long long cap_rows) {
    GptEngine* g = static_cast<GptEngine*>(e);
    if (!g->runner->last_graph) return 0;
    const auto rows = g->runner->last_graph->fused_trace(g->runner->stream);
    long long n = 0;
    for (auto& r : rows) {
        if (n >= cap_rows) break;
        for (int k = 0; k < 5; ++k) out[n * 5 + k] = r[k];
        ++n;
    }
    return n;
}
// Runs `steps` calls of step() and times them: out[0] device milliseconds between CUDA events recorded on the engine's
// stream before the first and after the last step, out[1] wall-clock milliseconds until the last step's tokens are on the
// host.  Returns the number of requests that finished meanwhile.
EGE_API long long ege_engine_time_steps(void* e, int steps, double* out, char* error, int cap) {
    return guarded(error, cap, [&]() {
        GptEngine* g = static_cast<GptEngine*>(e);
        cudaEvent_t start, stop;
        EG_CUDA(cudaEventCreate(&start));
        EG_CUDA(cudaEventCreate(&stop));
        EG_CUDA(cudaStreamSynchronize(g->runner->stream));
        long long finished = 0;
        const auto t0 = std::chrono::steady_clock::now();
        EG_CUDA(cudaEventRecord(start, g->runner->stream));
        for (int i = 0; i < steps; ++i) finished += (long long)g->step().size();
        EG_CUDA(cudaEventRecord(stop, g->runner->stream));
        EG_CUDA(cudaEventSynchronize(stop));
        out[1] = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        float ms = 0.f;
        EG_CUDA(cudaEventElapsedTime(&ms, start, stop));
        out[0] = ms;
        cudaEventDestroy(start);
        cudaEventDestroy(stop);
        return finished;
    });
}
EGE_API void ege_engine_sync(void* e) { cudaStreamSynchronize(static_cast<GptEngine*>(e)->runner->stream); }

// ---- the bare step function (trace replay, tests) ---------------------------------------------------------------------
EGE_API void* ege_runner_create(const char* model_dir, const char* dtype, int page_size, int num_pages, int max_slots, long long max_tokens_per_request,
                                int use_graphs, char* error, int cap) {
    Runner* r = nullptr;
    guarded(error, cap, [&]() {
        std::unique_ptr<Runner> made(new Runner());
        made->model = Model::from_dir(model_dir, dtype_from(dtype));
        StepRunner::Options o;
        o.page_size = page_size;
        o.num_pages = num_pages;
        o.max_slots = max_slots;
        o.max_tokens_per_request = max_tokens_per_request;
        o.use_graphs = use_graphs != 0;
        made->runner.reset(new StepRunner(*made->model, o));
        r = made.release();
        return 0;
    });
    return r;
}
EGE_API void ege_runner_destroy(void* r) { delete static_cast<Runner*>(r); }
// One step: n entries; entry i is request rids[i] with counts[i] tokens (flat in `tokens`) and wants[want_offsets[i] ..
// want_offsets[i + 1]) as the places among its tokens whose logits are asked for.  The logits [rows, vocab] are copied to
// `logits` (host, float32) if it holds them (cap_floats); returns the number of rows.  device_ms (optional): the step's time
// on the device in milliseconds.
EGE_API long long ege_runner_step(void* r, int n, const long long* rids, const long long* counts, const long long* tokens, const long long* want_offsets,
                                  const long long* wants, float* logits, long long cap_floats, double* device_ms, char* error, int cap) {
    return guarded(error, cap, [&]() {
        Runner* run = static_cast<Runner*>(r);
        cudaEvent_t start = nullptr, stop = nullptr;
        if (device_ms) {                        // the step's time on the device, between events on the runner's stream
            EG_CUDA(cudaEventCreate(&start));
            EG_CUDA(cudaEventCreate(&stop));
            EG_CUDA(cudaStreamSynchronize(run->runner->stream));
            EG_CUDA(cudaEventRecord(start, run->runner->stream));
        }
        std::vector<StepEntry> entries((size_t)n);
        long long at = 0;
        for (int i = 0; i < n; ++i) {
            entries[i].request = rids[i];
            entries[i].tokens.assign(tokens + at, tokens + at + counts[i]);
            entries[i].want.assign(wants + want_offsets[i], wants + want_offsets[i + 1]);
            at += counts[i];
        }
        const StepRunner::Result res = run->runner->run(entries, /*check=*/false, /*commit=*/true);
        if (device_ms) EG_CUDA(cudaEventRecord(stop, run->runner->stream));
        const long long vocab = run->model->lm_head->vocab();
        if (res.rows > 0) {
            if ((long long)res.rows * vocab > cap_floats) throw std::invalid_argument("the caller's logits buffer is too small");
            EG_CUDA(cudaMemcpyAsync(logits, res.logits, (size_t)res.rows * vocab * 4, cudaMemcpyDeviceToHost, run->runner->stream));
        }
        run->runner->check_status();           // synchronises the stream: the logits are on the host
        if (device_ms) {
            float ms = 0.f;
            EG_CUDA(cudaEventElapsedTime(&ms, start, stop));
            *device_ms = ms;
            cudaEventDestroy(start);
            cudaEventDestroy(stop);
        }
        return (long long)res.rows;
    });
}
EGE_API void ege_runner_end(void* r, long long rid) { static_cast<Runner*>(r)->runner->end(rid); }
// what: 0 vocabulary, 1 live requests, 2 captured-step replays, 3 free pages of group `arg`, 4 pages of group `arg`, 5 pages handed
// out over the life of group `arg`'s pool, 6 number of groups, 7 books in order (1) or not (0), 8 captured steps of shapes other
// than decode buckets, 9 steps that ran as one fused kernel
EGE_API long long ege_runner_info(void* r, int what, int arg) {
    Runner* run = static_cast<Runner*>(r);
    DeviceCache& cache = run->runner->cache;
    switch (what) {
        case 0: return run->model->lm_head->vocab();
        case 1: return (long long)cache.core.live_count();
        case 2: return run->runner->graph_replays;
        case 3: return cache.core.group(arg).pool.free_count();
        case 4: return cache.core.group(arg).pool.num_pages();
        case 5: return cache.core.group(arg).pool.total_allocated();
        case 6: return cache.core.num_groups();
        case 7: {
            std::string why;
            return cache.core.check(&why) == host::OK ? 1 : 0;
        }
        case 8: return (long long)run->runner->signature_graph_count();
        case 9: return run->runner->fused_steps;
    }
    return -1;
}

// A launch plan as this library computes it, for the test that compares the rules with their twins in the PyTorch face.
// what 0: the decode product's plan for (rows, width, head size or 0) -> (row blocks, K slices, K parts); 1: the decode
// attention's splits for (tokens, heads, KV heads, longest context, head size); 2: the most tokens whose norm rides in
// a decode product's prologue, for (width); 3: the prompt attention's (most parts, fewest key tiles of a part) for
// (query tiles, heads, head size, longest context); 4: the SM count the plans hang off.
EGE_API void ege_plan(int what, const long long* in, long long* out) {
    switch (what) {
        case 0: {
            const plans::SkinnyPlan plan = plans::skinny_plan((int)in[0], (int)in[1], (int)in[2]);
            out[0] = plan.row_blocks;
            out[1] = plan.k_slices;
            out[2] = plan.k_split;
            break;
        }
        case 1: out[0] = plans::attention_paged_splits((int)in[0], (int)in[1], (int)in[2], in[3], (int)in[4]); break;
        case 2: out[0] = plans::fused_norm_max_tokens((int)in[0]); break;
        case 3: {
            int parts = 0, part_tiles = 0;
            plans::attention_prefill_parts((int)in[0], (int)in[1], (int)in[2], in[3], &parts, &part_tiles);
            out[0] = parts;
            out[1] = part_tiles;
            break;
        }
        case 4: out[0] = plans::sm_count(); break;
    }
}
