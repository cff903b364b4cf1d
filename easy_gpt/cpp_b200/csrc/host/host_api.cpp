// C interface of the host runtime (page pools, cache bookkeeping, step packing, scheduler) for the
// Python bindings.  Handles are opaque pointers; functions return 0 or a positive result, or a
// negative Status.  Nothing here touches a GPU.
#include <cstring>

#include "bpe_tokenizer.hpp"
#include "cache_core.hpp"
#include "scheduler_core.hpp"
#include "step_pack.hpp"

using namespace easygpt::host;

#define EGH_API extern "C" __attribute__((visibility("default")))

// -- page pool ----------------------------------------------------------------------------------
EGH_API void* egh_pool_create(int num_pages) { return num_pages > 0 ? new PagePool(num_pages) : nullptr; }
EGH_API void egh_pool_destroy(void* p) { delete static_cast<PagePool*>(p); }
EGH_API int egh_pool_alloc(void* p, int n, int32_t* out) { return static_cast<PagePool*>(p)->alloc(n, out); }
EGH_API int egh_pool_free(void* p, const int32_t* pages, int n, int* bad) { return static_cast<PagePool*>(p)->free(pages, n, bad); }
EGH_API int egh_pool_check(void* p) { return static_cast<PagePool*>(p)->check(); }
// what: 0 pages, 1 free, 2 high-water mark, 3 pages handed out over the pool's life
EGH_API long long egh_pool_stat(void* p, int what) {
    const PagePool* pool = static_cast<PagePool*>(p);
    switch (what) {
        case 0: return pool->num_pages();
        case 1: return pool->free_count();
        case 2: return pool->high_water();
        case 3: return pool->total_allocated();
    }
    return BAD_ARGUMENT;
}

// -- cache bookkeeping ----------------------------------------------------------------------------
EGH_API void* egh_cache_create(int page_size, int max_slots, int max_pages_per_request) {
    if (page_size <= 0 || max_slots <= 0 || max_pages_per_request <= 0) return nullptr;
    return new CacheCore(page_size, max_slots, max_pages_per_request);
}
EGH_API void egh_cache_destroy(void* c) { delete static_cast<CacheCore*>(c); }
EGH_API int egh_cache_add_group(void* c, int num_pages, int window) {
    return num_pages > 0 ? static_cast<CacheCore*>(c)->add_group(num_pages, window) : BAD_ARGUMENT;
}
// borrowed: lives as long as the cache
EGH_API void* egh_cache_group_pool(void* c, int g) { return &static_cast<CacheCore*>(c)->group(g).pool; }
EGH_API int32_t* egh_cache_group_table(void* c, int g) { return static_cast<CacheCore*>(c)->group(g).tables.data(); }
EGH_API int egh_cache_begin(void* c, long long rid) { return static_cast<CacheCore*>(c)->begin_request(rid); }
EGH_API int egh_cache_take_fresh(void* c, int* out, int cap) { return static_cast<CacheCore*>(c)->take_fresh_slots(out, cap); }
EGH_API int egh_cache_end(void* c, long long rid) { return static_cast<CacheCore*>(c)->end_request(rid); }
// what: 0 slot, 1 tokens committed, 2 tokens reserved
EGH_API long long egh_cache_query(void* c, long long rid, int what) {
    const CachedRequest* r = static_cast<CacheCore*>(c)->find(rid);
    if (!r) return UNKNOWN_REQUEST;
    return what == 0 ? r->slot : what == 1 ? r->length : r->reserved;
}
// the most tokens committed to the cache among the given requests (one that is not live holds none)
EGH_API long long egh_cache_max_length(void* c, int n, const long long* rids) {
    long long most = 0;
    for (int i = 0; i < n; ++i) {
        const CachedRequest* r = static_cast<CacheCore*>(c)->find(rids[i]);
        if (r && r->length > most) most = r->length;
    }
    return most;
}
EGH_API int egh_cache_pages_needed(void* c, long long rid, long long new_tokens, int* out) {
    return static_cast<CacheCore*>(c)->pages_needed(rid, new_tokens, out);
}
EGH_API int egh_cache_can_reserve(void* c, long long rid, long long new_tokens, int spare) {
    return static_cast<CacheCore*>(c)->can_reserve(rid, new_tokens, spare);
}
EGH_API int egh_cache_reserve(void* c, long long rid, long long new_tokens, int* info) {
    return static_cast<CacheCore*>(c)->reserve(rid, new_tokens, info);
}
EGH_API int egh_cache_commit(void* c, long long rid, long long new_tokens) { return static_cast<CacheCore*>(c)->commit(rid, new_tokens); }
EGH_API int egh_cache_free_slots(void* c) { return static_cast<CacheCore*>(c)->free_slot_count(); }
EGH_API int egh_cache_slot_positions(void* c, int g, long long rid, long long start, int count, int32_t* out) {
    return static_cast<CacheCore*>(c)->slot_positions(g, rid, start, count, out);
}
// ids of the live requests into out (at most cap); returns how many are live
EGH_API int egh_cache_live(void* c, long long* out, int cap) {
    int n = 0;
    static_cast<CacheCore*>(c)->for_each_request([&](int64_t rid, const CachedRequest&) {
        if (n < cap) out[n] = rid;
        ++n;
    });
    return n;
}
EGH_API int egh_cache_check(void* c, char* why, int cap) {
    std::string msg;
    const int rc = static_cast<CacheCore*>(c)->check(&msg);
    if (why && cap > 0) {
        std::strncpy(why, msg.c_str(), cap - 1);
        why[cap - 1] = 0;
    }
    return rc;
}

// -- a step's pages and packed metadata ---------------------------------------------------------------
EGH_API int egh_step_reserve(void* c, int n, const long long* rids, const long long* counts, int* info) {
    return reserve_step(*static_cast<CacheCore*>(c), n, (const int64_t*)rids, (const int64_t*)counts, info);
}
EGH_API long long egh_step_bound(void* c, int n, long long tokens, long long wanted, int query_tile) {
    return packed_step_bound(*static_cast<CacheCore*>(c), n, tokens, wanted, query_tile);
}
// scalars (8 long longs): ints used, tokens, wanted rows, longest entry, longest context, all entries
// bring one token, query tiles, tokens outside tiles
EGH_API int egh_step_pack(void* c, int n, const long long* rids, const long long* counts, const long long* token_ids,
                          const long long* want_offsets, const long long* wants, int query_tile, int small_entry_tokens,
                          int32_t* buf, long long cap, long long* layout, int* widths, long long* scalars) {
    PackedStep out;
    const int rc = pack_step(*static_cast<CacheCore*>(c), n, (const int64_t*)rids, (const int64_t*)counts, (const int64_t*)token_ids,
                             (const int64_t*)want_offsets, (const int64_t*)wants, query_tile, small_entry_tokens, buf, cap,
                             layout, widths, &out);
    if (rc != OK) return rc;
    scalars[0] = out.total; scalars[1] = out.tokens; scalars[2] = out.rows; scalars[3] = out.max_query_len;
    scalars[4] = out.max_context_len; scalars[5] = out.all_decode; scalars[6] = out.num_tiles; scalars[7] = out.num_small;
    return OK;
}
EGH_API int egh_replay_pack(void* c, int n, const long long* rids, const int32_t* counts, int32_t* buf, long long off_positions,
                            long long off_context, long long off_slots, const long long* off_slot_map, const long long* off_table,
                            int table_width) {
    return pack_replay(*static_cast<CacheCore*>(c), n, (const int64_t*)rids, counts, buf, off_positions, off_context, off_slots,
                       off_slot_map, off_table, table_width);
}

// -- scheduler ------------------------------------------------------------------------------------------
// A batch crosses this interface as 4 long longs per entry: request id, start, count, samples.
namespace {
std::vector<ScheduledEntry> entries_of(const long long* flat, int n) {
    std::vector<ScheduledEntry> out(n);
    for (int i = 0; i < n; ++i) out[i] = {flat[4 * i], flat[4 * i + 1], flat[4 * i + 2], (int)flat[4 * i + 3]};
    return out;
}
}  // namespace

// the cache must outlive the scheduler
EGH_API void* egh_sched_create(void* cache, long long max_batch_tokens, long long chunk_size, int max_active, int prefill_batch,
                               long long eos_token_id, long long max_positions) {
    if (!cache || max_batch_tokens <= 0 || chunk_size <= 0 || max_active <= 0 || prefill_batch <= 0) return nullptr;
    SchedulerOptions opt;
    opt.max_batch_tokens = max_batch_tokens;
    opt.chunk_size = chunk_size;
    opt.max_active = max_active;
    opt.prefill_batch = prefill_batch;
    opt.eos_token_id = eos_token_id;
    opt.max_positions = max_positions;
    return new SchedulerCore(static_cast<CacheCore*>(cache), opt);
}
EGH_API void egh_sched_destroy(void* s) { delete static_cast<SchedulerCore*>(s); }
EGH_API long long egh_sched_add(void* s, long long prompt_len, long long max_new_tokens) {
    if (prompt_len < 0 || max_new_tokens <= 0) return BAD_ARGUMENT;
    return static_cast<SchedulerCore*>(s)->add(prompt_len, max_new_tokens);
}
EGH_API int egh_sched_has_work(void* s) { return static_cast<SchedulerCore*>(s)->has_work() ? 1 : 0; }
// The next step's batch into out, 5 long longs per entry (id, start, count, samples, and the request's tokens
// that are still on the device), at most cap entries; returns the number of entries.
EGH_API int egh_sched_schedule(void* s, long long* out, int cap) {
    std::vector<ScheduledEntry> batch;
    SchedulerCore* sc = static_cast<SchedulerCore*>(s);
    sc->schedule(batch);
    if ((int)batch.size() > cap) return BAD_ARGUMENT;
    for (size_t i = 0; i < batch.size(); ++i) {
        out[5 * i] = batch[i].id;
        out[5 * i + 1] = batch[i].start;
        out[5 * i + 2] = batch[i].count;
        out[5 * i + 3] = batch[i].samples;
        out[5 * i + 4] = sc->find(batch[i].id)->pending;
    }
    return (int)batch.size();
}
EGH_API int egh_sched_launched(void* s, const long long* batch, int n) {
    const auto entries = entries_of(batch, n);
    return static_cast<SchedulerCore*>(s)->launched(entries.data(), n);
}
EGH_API int egh_sched_resolve(void* s, const long long* batch, int n, const long long* tokens, int* actions) {
    const auto entries = entries_of(batch, n);
    return static_cast<SchedulerCore*>(s)->resolve(entries.data(), n, tokens, actions);
}
EGH_API int egh_sched_advance(void* s, long long id, long long n) { return static_cast<SchedulerCore*>(s)->advance(id, n); }
// out (10 long longs): prompt length, output length, max new tokens, computed, state, finish reason, error,
// pending, preemptions, admission counter
EGH_API int egh_sched_request(void* s, long long id, long long* out) {
    const SchedRequest* r = static_cast<SchedulerCore*>(s)->find(id);
    if (!r) return UNKNOWN_REQUEST;
    out[0] = r->prompt_len; out[1] = r->output_len; out[2] = r->max_new_tokens; out[3] = r->computed; out[4] = r->state;
    out[5] = r->reason; out[6] = r->error; out[7] = r->pending; out[8] = r->preemptions; out[9] = r->admitted_at;
    return OK;
}
// which: 0 waiting (queue order), 1 running (admission order), 2 finished (in the order they ended); returns the count
EGH_API int egh_sched_list(void* s, int which, long long* out, int cap) {
    const SchedulerCore* sc = static_cast<SchedulerCore*>(s);
    int n = 0;
    auto put = [&](int64_t id) { if (n < cap) out[n] = id; ++n; };
    if (which == 0) for (int64_t id : sc->waiting()) put(id);
    else if (which == 1) for (int64_t id : sc->running()) put(id);
    else for (int64_t id : sc->finished()) put(id);
    return n;
}
// out (6 long longs): steps, prompt tokens, decode tokens, preemptions, finished, failed
EGH_API void egh_sched_stats(void* s, long long* out) {
    const SchedulerStats& st = static_cast<SchedulerCore*>(s)->stats();
    out[0] = st.steps; out[1] = st.prompt_tokens; out[2] = st.decode_tokens; out[3] = st.preemptions; out[4] = st.finished; out[5] = st.failed;
}
EGH_API void egh_sched_forget(void* s, long long id) { static_cast<SchedulerCore*>(s)->forget(id); }

// -- tokenizer --------------------------------------------------------------------------------------------
// Strings cross this interface as UTF-8 bytes: lists of them as one blob with n + 1 offsets.
EGH_API void* egh_bpe_create() { return new BpeTokenizer(); }
EGH_API void egh_bpe_destroy(void* t) { delete static_cast<BpeTokenizer*>(t); }
EGH_API void egh_bpe_add_tokens(void* t, const char* blob, const long long* offsets, const int32_t* ids, int n) {
    for (int i = 0; i < n; ++i) static_cast<BpeTokenizer*>(t)->add_token(std::string(blob + offsets[i], blob + offsets[i + 1]), ids[i]);
}
EGH_API void egh_bpe_add_merges(void* t, const char* left, const long long* left_offsets, const char* right,
                                const long long* right_offsets, int n) {
    for (int i = 0; i < n; ++i)
        static_cast<BpeTokenizer*>(t)->add_merge(std::string(left + left_offsets[i], left + left_offsets[i + 1]),
                                                 std::string(right + right_offsets[i], right + right_offsets[i + 1]));
}
// longest first
EGH_API void egh_bpe_add_specials(void* t, const char* blob, const long long* offsets, int n) {
    for (int i = 0; i < n; ++i) static_cast<BpeTokenizer*>(t)->add_special(std::string(blob + offsets[i], blob + offsets[i + 1]));
}
EGH_API void egh_bpe_set_bos(void* t, int id) { static_cast<BpeTokenizer*>(t)->set_bos(id); }
// The three below return how much there is; what fits cap is written (a caller that got more than cap asks again).
EGH_API long long egh_bpe_encode(void* t, const char* text, long long length, int32_t* out, long long cap) {
    const std::vector<int32_t> ids = static_cast<BpeTokenizer*>(t)->encode(std::string(text, text + length));
    for (size_t i = 0; i < ids.size() && (long long)i < cap; ++i) out[i] = ids[i];
    return (long long)ids.size();
}
// tokens as UTF-8, each followed by a zero byte
EGH_API long long egh_bpe_tokenize(void* t, const char* text, long long length, char* out, long long cap) {
    std::string joined;
    for (const std::string& token : static_cast<BpeTokenizer*>(t)->tokenize(std::string(text, text + length))) {
        joined += token;
        joined += '\0';
    }
    std::memcpy(out, joined.data(), (size_t)std::min<long long>(cap, (long long)joined.size()));
    return (long long)joined.size();
}
EGH_API long long egh_bpe_decode(void* t, const int32_t* ids, long long n, char* out, long long cap) {
    const std::string raw = static_cast<BpeTokenizer*>(t)->decode(ids, (size_t)n);
    std::memcpy(out, raw.data(), (size_t)std::min<long long>(cap, (long long)raw.size()));
    return (long long)raw.size();
}
