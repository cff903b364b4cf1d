// The scheduler's decisions: admits requests, cuts prompts into portions under a token budget,
// decodes, finishes and frees.  Host code over the cache bookkeeping; it knows requests by their
// lengths only (token ids stay with the caller) and never touches a device.
//
// It follows the rounds of the reference's ContinuousBatchServer (src/continuous_batch_server.cpp:71-86):
// a FIFO of waiting requests, at most prefill_batch admissions per round and at most max_active live
// requests (:88-101), every decoding request advances by one token per round (:160-200), a request
// ends on EOS, which is emitted, or at its length limit (:141-149, 189-197), and its slot and cache
// are given back at once (:222-260).  What the reference does not have: one mixed step instead of
// separate prefill and decode rounds, a token budget with portions of prompts, and pages that can
// run out.  When they do: at admission the request waits and nothing overtakes it; for a running
// request the most recently admitted running request is preempted (everything it holds is given back
// and it returns to the front of the queue with the tokens it has generated, to be computed again);
// a request that cannot fit even alone in an empty pool fails.
#pragma once
#include <algorithm>
#include <cstdint>
#include <deque>
#include <unordered_map>
#include <vector>

#include "cache_core.hpp"

namespace easygpt::host {

struct SchedulerOptions {
    long long max_batch_tokens = 2048;   // tokens per step
    long long chunk_size = 512;          // longest portion of a prompt in one step
    int max_active = 16;                 // live requests
    int prefill_batch = 4;               // admissions per step
    long long eos_token_id = -1;         // < 0: no EOS
    long long max_positions = 1LL << 30;
};

enum RequestState : int { WAITING = 0, RUNNING = 1, FINISHED = 2 };
enum FinishReason : int { NOT_FINISHED = 0, FINISHED_EMPTY, FINISHED_EOS, FINISHED_LENGTH, FINISHED_MAX_POSITIONS, FINISHED_ERROR };
enum RequestError : int { NO_REQUEST_ERROR = 0, ERROR_NO_ROOM_UNDER_MAX_POSITIONS, ERROR_PROMPT_CANNOT_FIT, ERROR_CANNOT_HOLD_ALONE };

struct SchedRequest {
    int64_t id = 0;
    long long prompt_len = 0, output_len = 0, max_new_tokens = 0;
    long long computed = 0;              // tokens whose keys and values are in the cache
    int state = WAITING, reason = NOT_FINISHED, error = NO_REQUEST_ERROR;
    int pending = 0;                     // tokens sampled on the device whose ids the host has not read yet
    int preemptions = 0;
    long long admitted_at = -1;          // admission counter, for "most recently admitted"
    long long known() const { return prompt_len + output_len + pending; }
};

struct ScheduledEntry {
    int64_t id;
    long long start, count;              // first position fed this step, tokens fed
    int samples;                         // the portion reaches the last known token: its logits give the next token
};

struct SchedulerStats {
    long long steps = 0, prompt_tokens = 0, decode_tokens = 0, preemptions = 0, finished = 0, failed = 0;
};

class SchedulerCore {
public:
    SchedulerCore(CacheCore* cache, const SchedulerOptions& opt) : cache_(cache), opt_(opt) {}

    const SchedulerOptions& options() const { return opt_; }
    const SchedulerStats& stats() const { return stats_; }
    bool has_work() const { return !waiting_.empty() || !running_.empty(); }
    const std::deque<int64_t>& waiting() const { return waiting_; }
    const std::vector<int64_t>& running() const { return running_; }
    const std::vector<int64_t>& finished() const { return finished_; }
    SchedRequest* find(int64_t id) {
        auto it = requests_.find(id);
        return it == requests_.end() ? nullptr : &it->second;
    }

    int64_t add(long long prompt_len, long long max_new_tokens) {
        SchedRequest r;
        r.id = next_id_++;
        r.prompt_len = prompt_len;
        r.max_new_tokens = max_new_tokens;
        requests_.emplace(r.id, r);
        if (prompt_len == 0)
            finish(r.id, FINISHED_EMPTY, NO_REQUEST_ERROR);      // the reference answers an empty prompt at once (:285-291)
        else
            waiting_.push_back(r.id);
        return r.id;
    }

    // A finished request's record may be dropped once the caller has read it.
    void forget(int64_t id) {
        SchedRequest* r = find(id);
        if (r && r->state == FINISHED) {
            finished_.erase(std::remove(finished_.begin(), finished_.end(), id), finished_.end());
            requests_.erase(id);
        }
    }

    // Decides the next step's batch and reserves its cache pages.
    void schedule(std::vector<ScheduledEntry>& batch) {
        batch.clear();
        long long budget = opt_.max_batch_tokens;

        // 1. every request that has all its known tokens but one in the cache decodes one token
        const std::vector<int64_t> snapshot = running_;
        for (int64_t id : snapshot) {
            SchedRequest& req = requests_[id];
            if (req.state != RUNNING || req.known() - req.computed != 1 || budget <= 0) continue;
            if (req.pending && (req.output_len + req.pending >= req.max_new_tokens || req.known() >= opt_.max_positions))
                continue;                    // its pending token is its last one: it ends when the token is read
            while (cache_->can_reserve(id, 1, 0) != 1) {
                const int64_t victim = most_recently_admitted();
                for (size_t i = 0; i < batch.size(); ++i)
                    if (batch[i].id == victim) {
                        budget += batch[i].count;
                        batch.erase(batch.begin() + i);
                        break;
                    }
                const bool only_one = running_.size() == 1;
                preempt(victim);
                if (victim == id) {
                    if (only_one) {          // alone and still too large: it can never go on
                        waiting_.pop_front();
                        finish(id, FINISHED_ERROR, ERROR_CANNOT_HOLD_ALONE);
                    }
                    break;
                }
            }
            if (req.state != RUNNING) continue;
            cache_->reserve(id, 1, nullptr);
            batch.push_back({id, req.computed, 1, 1});
            budget -= 1;
        }

        // 2. requests in the middle of their prompt (or being computed again) get their next portion
        for (int64_t id : running_) {
            SchedRequest& req = requests_[id];
            const long long left = req.known() - req.computed;
            if (left <= 1 || budget <= 0 || req.pending) continue;       // (a portion needs all its token ids on the host)
            const long long n = std::min({left, opt_.chunk_size, budget});
            if (cache_->can_reserve(id, n, 0) != 1) continue;            // waits for pages; decoding requests free some or are preempted
            cache_->reserve(id, n, nullptr);
            batch.push_back({id, req.computed, n, req.computed + n == req.known() ? 1 : 0});
            budget -= n;
        }

        // 3. admissions, FIFO, while slots, pages and budget last
        int admitted = 0;
        while (!waiting_.empty() && admitted < opt_.prefill_batch && (int)running_.size() < opt_.max_active && budget > 0 &&
               cache_->free_slot_count() > 0) {
            const int64_t id = waiting_.front();
            SchedRequest& req = requests_[id];
            if (req.pending) break;          // preempted while its last token was on its way: wait for it
            const int err = limit_error(req);
            if (err) {
                waiting_.pop_front();
                finish(id, FINISHED_ERROR, err);
                continue;
            }
            const long long n = std::min({req.known(), opt_.chunk_size, budget});
            // keep one page per running request in reserve, so that admissions do not starve decoding
            cache_->begin_request(id);
            if (cache_->can_reserve(id, n, (int)running_.size()) != 1) {
                cache_->end_request(id);
                break;
            }
            cache_->reserve(id, n, nullptr);
            waiting_.pop_front();
            req.state = RUNNING;
            req.admitted_at = admissions_++;
            running_.push_back(id);
            batch.push_back({id, 0, n, n == req.known() ? 1 : 0});
            budget -= n;
            ++admitted;
        }

        if (batch.empty()) {
            for (int64_t id : running_)
                if (requests_[id].pending) return;       // everything live waits for a token that is on its way
            if (!running_.empty()) {
                // nothing fits although requests are live (all stuck in their prompts): make room
                const int64_t victim = most_recently_admitted();
                if (running_.size() == 1)
                    finish(victim, FINISHED_ERROR, ERROR_CANNOT_HOLD_ALONE);
                else
                    preempt(victim);
                schedule(batch);
                return;
            }
            return;
        }
        ++stats_.steps;
    }

    // The step has been handed to the device: its tokens count as cached, and every sampling entry has
    // one token on its way whose id resolve() will bring.
    int launched(const ScheduledEntry* batch, int n) {
        for (int i = 0; i < n; ++i) {
            SchedRequest* req = find(batch[i].id);
            if (!req) return UNKNOWN_REQUEST;
            const int rc = cache_->commit(req->id, batch[i].count);
            if (rc != OK) return rc;
            req->computed += batch[i].count;
            if (batch[i].count == 1 && batch[i].start >= req->prompt_len)
                ++stats_.decode_tokens;
            else
                stats_.prompt_tokens += batch[i].count;
            if (batch[i].samples) ++req->pending;
        }
        return OK;
    }

    // The sampled tokens of a launched step have reached the host: tokens[k] belongs to the k-th sampling
    // entry.  actions[k]: 0 dropped (the request had ended meanwhile: its previous token was EOS while this
    // step was already on the device), 1 appended to the request's output, 2 appended and the request ended.
    int resolve(const ScheduledEntry* batch, int n, const long long* tokens, int* actions) {
        int k = 0;
        for (int i = 0; i < n; ++i) {
            if (!batch[i].samples) continue;
            SchedRequest* req = find(batch[i].id);
            if (!req) return UNKNOWN_REQUEST;
            const long long token = tokens[k];
            if (req->state == FINISHED) {
                actions[k++] = 0;
                continue;
            }
            --req->pending;
            ++req->output_len;
            int reason = NOT_FINISHED;
            if (opt_.eos_token_id >= 0 && token == opt_.eos_token_id)
                reason = FINISHED_EOS;                       // the EOS token itself is emitted
            else if (req->output_len >= req->max_new_tokens)
                reason = FINISHED_LENGTH;
            else if (req->known() + 1 > opt_.max_positions)
                reason = FINISHED_MAX_POSITIONS;
            if (reason != NOT_FINISHED) {
                req->pending = 0;
                finish(req->id, reason, NO_REQUEST_ERROR);
                actions[k++] = 2;
            } else {
                actions[k++] = 1;
            }
        }
        return k;
    }

    // Tokens that were decoded outside the scheduler (a benchmark loop that feeds the device itself):
    // n more tokens exist and all but the last are in the cache, which the caller has committed.
    int advance(int64_t id, long long n) {
        SchedRequest* req = find(id);
        if (!req || req->state != RUNNING || n <= 0) return BAD_ARGUMENT;
        req->output_len += n;
        req->computed += n;
        return OK;
    }

private:
    int64_t most_recently_admitted() const {
        int64_t best = running_.front();
        long long at = requests_.at(best).admitted_at;
        for (int64_t id : running_)
            if (requests_.at(id).admitted_at > at) { at = requests_.at(id).admitted_at; best = id; }
        return best;
    }

    void finish(int64_t id, int reason, int error) {
        SchedRequest& req = requests_[id];
        if (cache_->find(id)) cache_->end_request(id);
        if (req.state == RUNNING)
            running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
        else if (req.state == WAITING)
            waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
        req.state = FINISHED;
        req.reason = reason;
        req.error = error;
        finished_.push_back(id);
        if (error) ++stats_.failed; else ++stats_.finished;
    }

    void preempt(int64_t id) {
        SchedRequest& victim = requests_[id];
        cache_->end_request(id);
        running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
        victim.computed = 0;
        victim.state = WAITING;
        ++victim.preemptions;
        ++stats_.preemptions;
        waiting_.push_front(id);
    }

    int limit_error(const SchedRequest& req) const {
        const long long total = req.prompt_len + 1;
        if (total > opt_.max_positions) return ERROR_NO_ROOM_UNDER_MAX_POSITIONS;
        if (total > cache_->pool_tokens() || total > (long long)cache_->max_pages_per_request() * cache_->page_size())
            return ERROR_PROMPT_CANNOT_FIT;
        return NO_REQUEST_ERROR;
    }

    CacheCore* cache_;
    SchedulerOptions opt_;
    std::deque<int64_t> waiting_;
    std::vector<int64_t> running_, finished_;
    std::unordered_map<int64_t, SchedRequest> requests_;
    SchedulerStats stats_;
    long long admissions_ = 0;
    int64_t next_id_ = 0;
};

}  // namespace easygpt::host
