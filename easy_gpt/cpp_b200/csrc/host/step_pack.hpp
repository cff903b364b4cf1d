// Packs a step's integer metadata into one buffer (the caller's pinned staging memory), from which
// a single copy takes it to the device: token ids, positions, the token -> entry map, entry starts,
// cached lengths and slots, the rows whose logits are wanted, query tiles for the prompt attention,
// and per cache group the cache position of every token and the entries' block-table rows.
// Also the reservation of a whole step's pages, all or nothing.
#pragma once
#include <algorithm>
#include <climits>
#include <cstdint>
#include <vector>

#include "cache_core.hpp"

namespace easygpt::host {

// sections of the packed buffer, in this order; then, for every group g, SLOT_MAP and TABLE
enum Section : int { TOKEN_IDS, POSITIONS, TOKEN_SEQ, SEQ_STARTS, SEQ_CONTEXT, SEQ_SLOTS, LOGIT_ROWS, QUERY_TILES, SMALL_TOKENS, FIXED_SECTIONS };

struct PackedStep {
    long long total = 0;                // ints used
    long long tokens = 0, rows = 0;
    long long max_query_len = 0, max_context_len = 0;
    int all_decode = 0, num_tiles = 0, num_small = 0;
};

inline long long pad4(long long n) { return (n + 3) & ~3LL; }

// Begins the requests of a step that are not live yet and reserves pages for every entry's new tokens:
// everything, or nothing at all (requests begun here are ended again) with the Status of the first
// obstacle.  info (3 ints, optional): group, pages the step needs there, pages free.
inline int reserve_step(CacheCore& cache, int n, const int64_t* rids, const int64_t* counts, int* info) {
    std::vector<int64_t> started;
    auto undo = [&](int rc) {
        for (int64_t r : started) cache.end_request(r);
        return rc;
    };
    for (int i = 0; i < n; ++i)
        if (!cache.find(rids[i])) {
            const int rc = cache.begin_request(rids[i]);
            if (rc < 0) return undo(rc);
            started.push_back(rids[i]);
        }
    const int G = cache.num_groups();
    std::vector<long long> need(G, 0);
    std::vector<int> one(G);
    for (int i = 0; i < n; ++i) {
        const CachedRequest* r = cache.find(rids[i]);
        if (CacheCore::ceil_div(r->length + counts[i], cache.page_size()) > cache.max_pages_per_request()) {
            if (info) { info[0] = i; info[1] = 0; info[2] = 0; }
            return undo(TOO_LONG);
        }
        cache.pages_needed(rids[i], counts[i], one.data());
        for (int g = 0; g < G; ++g) need[g] += one[g];
    }
    for (int g = 0; g < G; ++g)
        if (need[g] > cache.group(g).pool.free_count()) {
            if (info) { info[0] = g; info[1] = (int)need[g]; info[2] = cache.group(g).pool.free_count(); }
            return undo(OUT_OF_PAGES);
        }
    for (int i = 0; i < n; ++i) {
        const int rc = cache.reserve(rids[i], counts[i], nullptr);
        if (rc != OK) return undo(rc);            // cannot happen after the checks above
    }
    return OK;
}

// Upper bound of the ints a packed step takes (to size the staging buffer before packing).
inline long long packed_step_bound(const CacheCore& cache, int n, long long tokens, long long wanted, int query_tile) {
    const long long tiles = tokens / query_tile + n;
    long long total = 3 * pad4(tokens) + pad4(n + 1) + 2 * pad4(n) + pad4(wanted) + pad4(3 * tiles) + pad4(tokens);
    total += (long long)cache.num_groups() * (pad4(tokens) + pad4((long long)n * cache.max_pages_per_request()));
    return total;
}

// The requests are live and their pages reserved.  layout: (offset, size) of every section, 2 ints
// each, FIXED_SECTIONS + 2 * groups of them; widths: block-table columns per group.
inline int pack_step(const CacheCore& cache, int n, const int64_t* rids, const int64_t* counts, const int64_t* token_ids,
                     const int64_t* want_offsets, const int64_t* wants, int query_tile, int small_entry_tokens,
                     int32_t* buf, long long cap, long long* layout, int* widths, PackedStep* out) {
    const int G = cache.num_groups();
    const int ps = cache.page_size();
    long long T = 0, max_q = 0, max_ctx = 0;
    std::vector<const CachedRequest*> req(n);
    int all_decode = 1;
    for (int i = 0; i < n; ++i) {
        req[i] = cache.find(rids[i]);
        if (!req[i]) return UNKNOWN_REQUEST;
        if (counts[i] <= 0) return BAD_ARGUMENT;
        T += counts[i];
        if (counts[i] > max_q) max_q = counts[i];
        if (req[i]->length + counts[i] > max_ctx) max_ctx = req[i]->length + counts[i];
        if (counts[i] != 1) all_decode = 0;
    }
    const long long R = want_offsets[n];
    // tiles of the entries that bring more than small_entry_tokens tokens; the other entries' tokens one by one
    std::vector<int32_t> tiles, small;
    {
        long long s0 = 0;
        for (int i = 0; i < n; ++i) {
            if (counts[i] > small_entry_tokens)
                for (long long o = 0; o < counts[i]; o += query_tile) {
                    tiles.push_back(i);
                    tiles.push_back((int32_t)(s0 + o));
                    tiles.push_back((int32_t)(counts[i] - o < query_tile ? counts[i] - o : query_tile));
                }
            else
                for (long long t = 0; t < counts[i]; ++t) small.push_back((int32_t)(s0 + t));
            s0 += counts[i];
        }
    }
    const long long width = CacheCore::ceil_div(max_ctx, ps);
    long long off = 0;
    auto section = [&](int index, long long size) {
        layout[2 * index] = off;
        layout[2 * index + 1] = size;
        off += pad4(size);
    };
    section(TOKEN_IDS, T);
    section(POSITIONS, T);
    section(TOKEN_SEQ, T);
    section(SEQ_STARTS, n + 1);
    section(SEQ_CONTEXT, n);
    section(SEQ_SLOTS, n);
    section(LOGIT_ROWS, R);
    section(QUERY_TILES, (long long)tiles.size());
    section(SMALL_TOKENS, (long long)small.size());
    for (int g = 0; g < G; ++g) {
        widths[g] = (int)width;
        section(FIXED_SECTIONS + 2 * g, T);
        section(FIXED_SECTIONS + 2 * g + 1, (long long)n * width);
    }
    if (off > cap) return BAD_ARGUMENT;

    int32_t* ids = buf + layout[2 * TOKEN_IDS];
    int32_t* pos = buf + layout[2 * POSITIONS];
    int32_t* seq = buf + layout[2 * TOKEN_SEQ];
    int32_t* starts = buf + layout[2 * SEQ_STARTS];
    int32_t* context = buf + layout[2 * SEQ_CONTEXT];
    int32_t* slots = buf + layout[2 * SEQ_SLOTS];
    int32_t* rows = buf + layout[2 * LOGIT_ROWS];
    long long t = 0;
    for (int i = 0; i < n; ++i) {
        starts[i] = (int32_t)t;
        context[i] = (int32_t)req[i]->length;
        slots[i] = req[i]->slot;
        for (long long k = 0; k < counts[i]; ++k, ++t) {
            const int64_t id = token_ids[t];
            if (id < INT32_MIN || id > INT32_MAX) return BAD_ARGUMENT;
            ids[t] = (int32_t)id;
            pos[t] = (int32_t)(req[i]->length + k);
            seq[t] = i;
        }
        for (long long w = want_offsets[i]; w < want_offsets[i + 1]; ++w) {
            if (wants[w] < 0 || wants[w] >= counts[i]) return BAD_ARGUMENT;
            rows[w] = (int32_t)(starts[i] + wants[w]);
        }
    }
    starts[n] = (int32_t)T;
    std::copy(tiles.begin(), tiles.end(), buf + layout[2 * QUERY_TILES]);
    std::copy(small.begin(), small.end(), buf + layout[2 * SMALL_TOKENS]);
    for (int g = 0; g < G; ++g) {
        int32_t* slot_map = buf + layout[2 * (FIXED_SECTIONS + 2 * g)];
        int32_t* table = buf + layout[2 * (FIXED_SECTIONS + 2 * g + 1)];
        const int32_t* all = cache.group(g).tables.data();
        long long tt = 0;
        for (int i = 0; i < n; ++i) {
            const int32_t* row = all + (size_t)req[i]->slot * cache.max_pages_per_request();
            for (long long k = 0; k < counts[i]; ++k, ++tt) {
                const long long p = req[i]->length + k;
                const int page = row[p / ps];
                if (page < 0) return NO_PAGE;
                slot_map[tt] = (int32_t)((long long)page * ps + p % ps);
            }
            std::copy(row, row + width, table + (size_t)i * width);
        }
    }
    out->total = off;
    out->tokens = T;
    out->rows = R;
    out->max_query_len = max_q;
    out->max_context_len = max_ctx;
    out->all_decode = all_decode;
    out->num_tiles = (int)tiles.size() / 3;
    out->num_small = (int)small.size();
    return OK;
}

// A captured step's changing inputs: the signature (counts, starts, offsets inside entries) is fixed;
// positions, cached lengths, slots, cache positions and block-table rows of the n live entries are
// written at the given offsets of the graph's staging buffer.  Rows beyond n (padding of a decode
// bucket) are filled by the caller.
inline int pack_replay(const CacheCore& cache, int n, const int64_t* rids, const int32_t* counts, int32_t* buf,
                       long long off_positions, long long off_context, long long off_slots, const long long* off_slot_map,
                       const long long* off_table, int table_width) {
    const int ps = cache.page_size();
    long long t = 0;
    std::vector<const CachedRequest*> req(n);
    for (int i = 0; i < n; ++i) {
        req[i] = cache.find(rids[i]);
        if (!req[i]) return UNKNOWN_REQUEST;
        // the graph's block table is as wide as the context bucket it was captured for
        if ((req[i]->length + counts[i] + ps - 1) / ps > table_width) return TOO_LONG;
        buf[off_context + i] = (int32_t)req[i]->length;
        buf[off_slots + i] = req[i]->slot;
        for (int k = 0; k < counts[i]; ++k, ++t) buf[off_positions + t] = (int32_t)(req[i]->length + k);
    }
    for (int g = 0; g < cache.num_groups(); ++g) {
        const int32_t* all = cache.group(g).tables.data();
        long long tt = 0;
        for (int i = 0; i < n; ++i) {
            const int32_t* row = all + (size_t)req[i]->slot * cache.max_pages_per_request();
            for (int k = 0; k < counts[i]; ++k, ++tt) {
                const long long p = req[i]->length + k;
                if (p / ps >= cache.max_pages_per_request()) return NO_PAGE;
                const int page = row[p / ps];
                if (page < 0) return NO_PAGE;
                buf[off_slot_map[g] + tt] = (int32_t)((long long)page * ps + p % ps);
            }
            std::copy(row, row + table_width, buf + off_table[g] + (size_t)i * table_width);
        }
    }
    return OK;
}

}  // namespace easygpt::host
