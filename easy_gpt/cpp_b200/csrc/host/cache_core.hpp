// Bookkeeping of the paged cache: one page pool and one block table per group of caches with the
// same needs, request slots, and per request the tokens committed and reserved.  A group that keeps
// all keys holds ceil(length / page_size) pages per request; a group with a window gives a page back
// as soon as every position in it has left the window of all tokens still to come.  Host code only:
// device memory belongs to the caller, which addresses it with the page ids kept here.
//
// (The reference has no pages: its per-sample caches grow by concatenation,
// src/models/self_attn.cpp:369-389, and its slots are a stack of free indices,
// src/continuous_batch_server.cpp:44-47.)
#pragma once
#include <cstdint>
#include <cstdio>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "page_pool.hpp"

namespace easygpt::host {

struct CacheGroup {
    PagePool pool;
    int window;                         // < 0: all keys are kept
    std::vector<int32_t> tables;        // [max_slots][max_pages_per_request], -1 where no page is held
    CacheGroup(int num_pages, int window_, size_t table_ints) : pool(num_pages), window(window_), tables(table_ints, -1) {}
};

struct CachedRequest {
    int slot = -1;
    long long length = 0;               // tokens committed to the cache
    long long reserved = 0;             // tokens for which pages exist (>= length)
    std::vector<int> first_live_page;   // per group: logical pages below were given back
};

class CacheCore {
public:
    CacheCore(int page_size, int max_slots, int max_pages_per_request)
        : page_size_(page_size), max_slots_(max_slots), max_pages_(max_pages_per_request) {
        for (int s = max_slots - 1; s >= 0; --s) free_slots_.push_back(s);   // slot 0 first
        slot_is_fresh_.assign(max_slots, 0);
    }

    int add_group(int num_pages, int window) {
        groups_.emplace_back(new CacheGroup(num_pages, window, (size_t)max_slots_ * max_pages_));
        for (auto& kv : requests_) kv.second.first_live_page.push_back(0);
        return (int)groups_.size() - 1;
    }

    int page_size() const { return page_size_; }
    int max_slots() const { return max_slots_; }
    int max_pages_per_request() const { return max_pages_; }
    int num_groups() const { return (int)groups_.size(); }
    CacheGroup& group(int g) { return *groups_[g]; }
    const CacheGroup& group(int g) const { return *groups_[g]; }
    int free_slot_count() const { return (int)free_slots_.size(); }
    size_t live_count() const { return requests_.size(); }
    const CachedRequest* find(int64_t rid) const {
        auto it = requests_.find(rid);
        return it == requests_.end() ? nullptr : &it->second;
    }
    template <class F> void for_each_request(F f) const { for (auto& kv : requests_) f(kv.first, kv.second); }
    // the smallest pool, in tokens (what a single request can hold at most)
    long long pool_tokens() const {
        if (groups_.empty()) return 1LL << 60;
        long long least = 1LL << 60;
        for (auto& g : groups_) if (g->pool.num_pages() < least) least = g->pool.num_pages();
        return least * page_size_;
    }

    int begin_request(int64_t rid) {
        if (requests_.count(rid)) return ALREADY_LIVE;
        if (free_slots_.empty()) return OUT_OF_SLOTS;
        CachedRequest r;
        r.slot = free_slots_.back();
        free_slots_.pop_back();
        r.first_live_page.assign(groups_.size(), 0);
        if (!slot_is_fresh_[r.slot]) {
            slot_is_fresh_[r.slot] = 1;
            fresh_slots_.push_back(r.slot);
        }
        requests_.emplace(rid, std::move(r));
        return requests_[rid].slot;
    }

    // Slots that requests have taken since the last call (each once), whoever began them: the owner of
    // per-request state of fixed size clears those slots before the next step runs.  Writes at most cap
    // of them to out and forgets what it wrote; returns how many were written.
    int take_fresh_slots(int* out, int cap) {
        int n = 0;
        while (n < cap && !fresh_slots_.empty()) {
            const int s = fresh_slots_.back();
            fresh_slots_.pop_back();
            slot_is_fresh_[s] = 0;
            out[n++] = s;
        }
        return n;
    }

    int end_request(int64_t rid) {
        auto it = requests_.find(rid);
        if (it == requests_.end()) return UNKNOWN_REQUEST;
        const int slot = it->second.slot;
        std::vector<int32_t> held;
        for (auto& g : groups_) {
            int32_t* row = g->tables.data() + (size_t)slot * max_pages_;
            held.clear();
            for (int i = 0; i < max_pages_; ++i)
                if (row[i] >= 0) { held.push_back(row[i]); row[i] = -1; }
            int bad = 0;
            const int rc = g->pool.free(held.data(), (int)held.size(), &bad);
            if (rc != OK) return rc;
        }
        free_slots_.push_back(slot);
        requests_.erase(it);
        return OK;
    }

    static long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }

    // pages each group would have to hand out so that new_tokens more tokens fit
    int pages_needed(int64_t rid, long long new_tokens, int* out) const {
        const CachedRequest* r = find(rid);
        if (!r) return UNKNOWN_REQUEST;
        const long long target = r->length + new_tokens;
        for (size_t g = 0; g < groups_.size(); ++g) {
            const long long have = ceil_div(r->reserved, page_size_), want = ceil_div(target, page_size_);
            out[g] = (int)(want > have ? want - have : 0);
        }
        return OK;
    }

    // 1 yes, 0 no, < 0 error
    int can_reserve(int64_t rid, long long new_tokens, int spare) const {
        const CachedRequest* r = find(rid);
        if (!r) return UNKNOWN_REQUEST;
        if (ceil_div(r->length + new_tokens, page_size_) > max_pages_) return 0;
        std::vector<int> need(groups_.size());
        pages_needed(rid, new_tokens, need.data());
        for (size_t g = 0; g < groups_.size(); ++g)
            if (groups_[g]->pool.free_count() - spare < need[g]) return 0;
        return 1;
    }

    // Pages for positions length .. length + new_tokens - 1 in every group, or an error with nothing
    // changed.  info (3 ints, optional): group, pages wanted, pages free of the group that fell short.
    int reserve(int64_t rid, long long new_tokens, int* info) {
        auto it = requests_.find(rid);
        if (it == requests_.end()) return UNKNOWN_REQUEST;
        CachedRequest& r = it->second;
        const long long target = r.length + new_tokens;
        if (ceil_div(target, page_size_) > max_pages_) return TOO_LONG;
        std::vector<int> need(groups_.size());
        pages_needed(rid, new_tokens, need.data());
        for (size_t g = 0; g < groups_.size(); ++g)
            if (groups_[g]->pool.free_count() < need[g]) {
                if (info) { info[0] = (int)g; info[1] = need[g]; info[2] = groups_[g]->pool.free_count(); }
                return OUT_OF_PAGES;
            }
        const long long have = ceil_div(r.reserved, page_size_);
        for (size_t g = 0; g < groups_.size(); ++g)
            groups_[g]->pool.alloc(need[g], groups_[g]->tables.data() + (size_t)r.slot * max_pages_ + have);
        if (target > r.reserved) r.reserved = target;
        return OK;
    }

    // The step has written new_tokens more tokens; pages that no coming token can see any more (a
    // window has passed them) are given back.
    int commit(int64_t rid, long long new_tokens) {
        auto it = requests_.find(rid);
        if (it == requests_.end()) return UNKNOWN_REQUEST;
        CachedRequest& r = it->second;
        if (new_tokens < 0) return BAD_ARGUMENT;
        if (r.length + new_tokens > r.reserved) return EXCEEDS_RESERVED;
        r.length += new_tokens;
        for (size_t g = 0; g < groups_.size(); ++g) {
            CacheGroup& grp = *groups_[g];
            if (grp.window < 0) continue;
            const long long first_key = r.length - grp.window + 1 > 0 ? r.length - grp.window + 1 : 0;
            const int first = (int)(first_key / page_size_), old = r.first_live_page[g];
            if (first > old) {
                int32_t* row = grp.tables.data() + (size_t)r.slot * max_pages_;
                int bad = 0;
                const int rc = grp.pool.free(row + old, first - old, &bad);
                if (rc != OK) return rc;
                for (int i = old; i < first; ++i) row[i] = -1;
                r.first_live_page[g] = first;
            }
        }
        return OK;
    }

    // physical cache positions (page * page_size + offset) of logical positions start .. start + count - 1
    int slot_positions(int g, int64_t rid, long long start, int count, int32_t* out) const {
        const CachedRequest* r = find(rid);
        if (!r) return UNKNOWN_REQUEST;
        if (start < 0 || count < 0 || ceil_div(start + count, page_size_) > max_pages_) return NO_PAGE;
        const int32_t* row = groups_[g]->tables.data() + (size_t)r->slot * max_pages_;
        for (int i = 0; i < count; ++i) {
            const long long pos = start + i;
            const int page = row[pos / page_size_];
            if (page < 0) return NO_PAGE;
            out[i] = (int32_t)((long long)page * page_size_ + pos % page_size_);
        }
        return OK;
    }

    // No page lost, none held twice: the pages in all block tables are exactly the pages the pools
    // consider held, free slots hold nothing, and slots add up.
    int check(std::string* why) const {
        std::vector<char> live(max_slots_, 0);
        for (auto& kv : requests_) {
            if (kv.second.slot < 0 || kv.second.slot >= max_slots_ || live[kv.second.slot]) return fail(why, "two requests share a slot");
            live[kv.second.slot] = 1;
        }
        for (size_t gi = 0; gi < groups_.size(); ++gi) {
            const CacheGroup& g = *groups_[gi];
            if (g.pool.check() != OK) return fail(why, "group " + std::to_string(gi) + ": a page is lost, or both held and free");
            std::vector<char> seen(g.pool.num_pages(), 0);
            int held = 0;
            for (int s = 0; s < max_slots_; ++s)
                for (int i = 0; i < max_pages_; ++i) {
                    const int p = g.tables[(size_t)s * max_pages_ + i];
                    if (p < 0) continue;
                    if (!live[s]) return fail(why, "group " + std::to_string(gi) + ": free slot " + std::to_string(s) + " still holds pages");
                    if (p >= g.pool.num_pages() || seen[p]) return fail(why, "group " + std::to_string(gi) + ": a page is in two places of the block tables");
                    seen[p] = 1;
                    ++held;
                }
            if (held != g.pool.used_count())
                return fail(why, "group " + std::to_string(gi) + ": " + std::to_string(g.pool.used_count()) + " pages held, " + std::to_string(held) + " in tables");
        }
        std::vector<char> free_seen(max_slots_, 0);
        for (int s : free_slots_) {
            if (s < 0 || s >= max_slots_ || free_seen[s] || live[s]) return fail(why, "a slot is free twice, or free and taken");
            free_seen[s] = 1;
        }
        if (free_slots_.size() + requests_.size() != (size_t)max_slots_) return fail(why, "slots do not add up");
        return OK;
    }

private:
    static int fail(std::string* why, const std::string& msg) {
        if (why) *why = msg;
        return BOOKS_WRONG;
    }
    int page_size_, max_slots_, max_pages_;
    std::vector<std::unique_ptr<CacheGroup>> groups_;
    std::vector<int> free_slots_;
    std::vector<int> fresh_slots_;          // taken since take_fresh_slots() was last called
    std::vector<char> slot_is_fresh_;
    std::unordered_map<int64_t, CachedRequest> requests_;
};

}  // namespace easygpt::host
