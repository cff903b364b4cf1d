// Allocator of page ids for one cache group: a LIFO stack of free ids, so that a page given
// back is the next one handed out (a small pool uses its ids again at once).  Host code; it
// owns no device memory.
#pragma once
#include <cstdint>
#include <vector>

namespace easygpt::host {

enum Status : int {
    OK = 0,
    OUT_OF_PAGES = -1,        // nothing was changed
    NOT_OF_POOL = -2,
    FREED_TWICE = -3,
    ALREADY_LIVE = -4,
    OUT_OF_SLOTS = -5,
    UNKNOWN_REQUEST = -6,
    TOO_LONG = -7,            // a request would hold more than max_pages_per_request pages
    EXCEEDS_RESERVED = -8,
    NO_PAGE = -9,             // a position that was asked for has no page
    BAD_ARGUMENT = -10,
    BOOKS_WRONG = -11,        // a consistency check failed
};

class PagePool {
public:
    explicit PagePool(int num_pages) : num_pages_(num_pages), held_(num_pages, 0) {
        free_.reserve(num_pages);
        for (int p = num_pages - 1; p >= 0; --p) free_.push_back(p);        // page 0 is handed out first
    }
    int num_pages() const { return num_pages_; }
    int free_count() const { return (int)free_.size(); }
    int used_count() const { return num_pages_ - (int)free_.size(); }
    int high_water() const { return high_water_; }
    long long total_allocated() const { return total_allocated_; }

    // n pages into out, or OUT_OF_PAGES with nothing changed
    int alloc(int n, int32_t* out) {
        if (n < 0) return BAD_ARGUMENT;
        if (n > (int)free_.size()) return OUT_OF_PAGES;
        for (int i = 0; i < n; ++i) {
            const int p = free_.back();
            free_.pop_back();
            held_[p] = 1;
            out[i] = p;
        }
        total_allocated_ += n;
        if (used_count() > high_water_) high_water_ = used_count();
        return OK;
    }

    // Gives pages back, all or none: a page that is not of this pool or not held (or named twice in
    // the call) refuses the whole call and is reported through *bad.
    int free(const int32_t* pages, int n, int* bad) {
        for (int i = 0; i < n; ++i) {
            const int p = pages[i];
            if (p < 0 || p >= num_pages_) { if (bad) *bad = p; return NOT_OF_POOL; }
            if (held_[p] != 1) {
                for (int j = 0; j < i; ++j) if (held_[pages[j]] == 2) held_[pages[j]] = 1;
                if (bad) *bad = p;
                return FREED_TWICE;
            }
            held_[p] = 2;                                                   // marked: catches a page named twice
        }
        for (int i = 0; i < n; ++i) held_[pages[i]] = 0;
        // pushed in reverse so that the lowest id of the batch comes out first again
        for (int i = n - 1; i >= 0; --i) free_.push_back(pages[i]);
        return OK;
    }

    // every page is either free once or held once
    int check() const {
        std::vector<char> seen(num_pages_, 0);
        for (int p : free_) {
            if (p < 0 || p >= num_pages_ || seen[p]) return BOOKS_WRONG;
            seen[p] = 1;
        }
        for (int p = 0; p < num_pages_; ++p)
            if ((held_[p] != 0) == (seen[p] != 0)) return BOOKS_WRONG;
        return OK;
    }

private:
    int num_pages_;
    std::vector<int32_t> free_;
    std::vector<char> held_;
    int high_water_ = 0;
    long long total_allocated_ = 0;
};

}  // namespace easygpt::host
