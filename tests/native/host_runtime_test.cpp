// The host runtime used from C++ alone, without Python: pools, cache bookkeeping with a window,
// all-or-nothing reservation of a step, and the scheduler driven to completion over a pool that is
// too small for all requests at once (so that it preempts).  Exits 0 if every check holds.
#include <cstdio>
#include <cstdlib>
#include <map>
#include <string>
#include <vector>

#include "bpe_tokenizer.hpp"
#include "cache_core.hpp"
#include "scheduler_core.hpp"
#include "step_pack.hpp"

using namespace easygpt::host;

#define CHECK(cond)                                                          \
    do {                                                                     \
        if (!(cond)) {                                                       \
            std::fprintf(stderr, "%s:%d: check failed: %s\n", __FILE__, __LINE__, #cond); \
            std::exit(1);                                                    \
        }                                                                    \
    } while (0)

static void pools() {
    PagePool p(4);
    int32_t a[4];
    CHECK(p.alloc(3, a) == OK && a[0] == 0 && a[1] == 1 && a[2] == 2 && p.free_count() == 1);
    int32_t one[] = {1};
    int bad = -1;
    CHECK(p.free(one, 1, &bad) == OK);
    CHECK(p.alloc(1, a) == OK && a[0] == 1);              // a page given back is the next one handed out
    CHECK(p.alloc(2, a) == OUT_OF_PAGES && p.free_count() == 1);
    int32_t twice[] = {0, 0};
    CHECK(p.free(twice, 2, &bad) == FREED_TWICE && bad == 0 && p.used_count() == 3);
    int32_t far[] = {9};
    CHECK(p.free(far, 1, &bad) == NOT_OF_POOL && bad == 9);
    CHECK(p.check() == OK);
}

static void cache_with_a_window() {
    CacheCore cache(4, 2, 64);
    const int full = cache.add_group(32, -1), win = cache.add_group(32, 10);
    CHECK(cache.begin_request(7) == 0 && cache.begin_request(7) == ALREADY_LIVE);
    for (int pos = 0; pos < 40; ++pos) {
        CHECK(cache.reserve(7, 1, nullptr) == OK && cache.commit(7, 1) == OK);
        // the next token sits at pos + 1 and sees keys pos + 1 - 9 .. pos + 1: pages below are given back
        const int first_key = pos + 1 - 10 + 1 > 0 ? pos + 1 - 10 + 1 : 0;
        const int32_t* row = cache.group(win).tables.data();
        for (int i = 0; i < 64; ++i) CHECK((row[i] >= 0) == (i >= first_key / 4 && i <= pos / 4));
        CHECK(cache.group(full).tables[0] >= 0);
        CHECK(cache.group(win).pool.used_count() <= 4);
    }
    CHECK(cache.commit(7, 1) == EXCEEDS_RESERVED);
    std::string why;
    CHECK(cache.check(&why) == OK);
    CHECK(cache.end_request(7) == OK && cache.end_request(7) == UNKNOWN_REQUEST);
    CHECK(cache.group(full).pool.free_count() == 32 && cache.group(win).pool.free_count() == 32);
}

static void a_step_is_reserved_whole_or_not_at_all() {
    CacheCore cache(4, 3, 16);
    cache.add_group(6, -1);
    const int64_t rids[] = {1, 2, 3};
    const int64_t fits[] = {8, 8, 8}, too_much[] = {8, 8, 9};
    int info[3] = {0, 0, 0};
    CHECK(reserve_step(cache, 3, rids, too_much, info) == OUT_OF_PAGES && info[1] == 7 && info[2] == 6);
    CHECK(cache.live_count() == 0 && cache.group(0).pool.free_count() == 6 && cache.free_slot_count() == 3);
    CHECK(reserve_step(cache, 3, rids, fits, info) == OK && cache.group(0).pool.free_count() == 0);
    const int64_t tokens[24] = {0}, want_offsets[] = {0, 1, 1, 2}, wants[] = {7, 0};
    std::vector<int32_t> buf(packed_step_bound(cache, 3, 24, 2, 128));
    long long layout[2 * (FIXED_SECTIONS + 2)];
    int widths[1];
    PackedStep out;
    CHECK(pack_step(cache, 3, rids, fits, tokens, want_offsets, wants, 128, 4, buf.data(), (long long)buf.size(), layout, widths,
                    &out) == OK);
    CHECK(out.tokens == 24 && out.rows == 2 && out.num_tiles == 3 && out.num_small == 0 && widths[0] == 2 && !out.all_decode);
    CHECK(buf[layout[2 * LOGIT_ROWS]] == 7 && buf[layout[2 * LOGIT_ROWS] + 1] == 16);
    CHECK(buf[layout[2 * POSITIONS] + 9] == 1 && buf[layout[2 * TOKEN_SEQ] + 9] == 1);
}

static void the_scheduler_finishes_everything_although_pages_run_out() {
    CacheCore cache(4, 4, 64);
    cache.add_group(24, -1);
    SchedulerOptions opt;
    opt.max_batch_tokens = 24;
    opt.chunk_size = 10;
    opt.max_active = 4;
    opt.prefill_batch = 2;
    opt.eos_token_id = 3;
    SchedulerCore sched(&cache, opt);
    std::map<int64_t, long long> want_new;
    for (int i = 0; i < 6; ++i) want_new[sched.add(5 + 7 * i, 12 + i)] = 12 + i;
    CHECK(sched.find(sched.add(0, 5))->reason == FINISHED_EMPTY);
    std::vector<ScheduledEntry> batch;
    unsigned rng = 12345;
    int rounds = 0;
    while (sched.has_work()) {
        CHECK(++rounds < 10000);
        sched.schedule(batch);
        CHECK(!batch.empty());
        long long total = 0;
        std::vector<long long> tokens;
        for (const ScheduledEntry& e : batch) {
            const SchedRequest* r = sched.find(e.id);
            CHECK(e.start == r->computed && cache.find(e.id)->length == r->computed);
            CHECK((e.samples != 0) == (e.start + e.count == r->known()));
            total += e.count;
            rng = rng * 1664525u + 1013904223u;
            if (e.samples) tokens.push_back(4 + (rng >> 16) % 40);       // never the EOS id
        }
        CHECK(total <= opt.max_batch_tokens);
        CHECK(sched.launched(batch.data(), (int)batch.size()) == OK);
        std::vector<int> actions(tokens.size() + 1);
        CHECK(sched.resolve(batch.data(), (int)batch.size(), tokens.data(), actions.data()) == (int)tokens.size());
        std::string why;
        CHECK(cache.check(&why) == OK);
    }
    CHECK(sched.stats().preemptions > 0 && sched.stats().failed == 0 && sched.stats().finished == 7);
    for (auto& kv : want_new) {
        const SchedRequest* r = sched.find(kv.first);
        CHECK(r->state == FINISHED && r->reason == FINISHED_LENGTH && r->output_len == kv.second);
    }
    CHECK(cache.live_count() == 0 && cache.group(0).pool.free_count() == 24);
}

static void the_tokenizer_follows_the_rules() {
    BpeTokenizer tok;
    const std::string sp = "\xC4\xA0";                       // the stand-in of the space byte (U+0120)
    const std::vector<std::string> vocab = {"h", "e", "l", "o", "w", "r", "d", sp, "he", "ll", "hell", "hello", sp + "w", "or",
                                            sp + "wor", "ld", "!"};
    for (size_t i = 0; i < vocab.size(); ++i) tok.add_token(vocab[i], (int32_t)i);
    tok.add_token("<|im_end|>", 101);
    const std::pair<std::string, std::string> merges[] = {{"h", "e"}, {"l", "l"}, {"he", "ll"}, {"hell", "o"}, {sp, "w"},
                                                          {"o", "r"}, {sp + "w", "or"}, {"l", "d"}};
    for (auto& m : merges) tok.add_merge(m.first, m.second);
    tok.add_special("<|im_end|>");
    CHECK((tok.tokenize("hello   \n world") == std::vector<std::string>{"hello", sp + "wor", "ld"}));
    CHECK((tok.encode("hello world") == std::vector<int32_t>{11, 14, 15}));
    CHECK((tok.encode("hello<|im_end|>world") == std::vector<int32_t>{11, 101, 4, 13, 15}));      // no space between specials and text
    CHECK((tok.encode("hello <|im_end|> world") == std::vector<int32_t>{11, 101, 14, 15}));
    CHECK((tok.encode("hello xyz") == std::vector<int32_t>{11, 7}));                              // unknown pieces are dropped
    const std::vector<int32_t> ids = {11, 14, 15, 101};
    CHECK(tok.decode(ids.data(), ids.size()) == "hello world<|im_end|>");
    tok.set_bos(9);
    CHECK(tok.encode("hello").front() == 9);
}

int main() {
    the_tokenizer_follows_the_rules();
    pools();
    cache_with_a_window();
    a_step_is_reserved_whole_or_not_at_all();
    the_scheduler_finishes_everything_although_pages_run_out();
    std::puts("host runtime: all checks passed");
    return 0;
}
