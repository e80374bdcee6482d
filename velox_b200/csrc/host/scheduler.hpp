// Continuous batching above the step function: admit, cut prompts into portions
// under a token budget, decode, finish and free.
//
// What is kept of the reference's BatchScheduler (src/paged/scheduler.rs:75-535):
// first come first served from a queue (:220-295), at most max_running requests
// holding cache (:239), requests in a step ordered by id (:311-312), one new token
// per decoding request per step (:337-343), the first token sampled from the step
// that completes the prompt (:407-421), an end-of-sequence token kept and counted
// (:426), finish reasons "stop", "length" and "cancelled" (:440-452, :465-484), and
// its counters with the last step's wall time (:95-105, :528-532).
//
// What differs, on purpose:
//   * Prompts are really cut.  The reference offers a request's whole remaining
//     prompt or defers it (src/paged/scheduler.rs:322-330), so one long prompt
//     still runs whole.  Here decoding requests go first (one token each), then
//     the budget max_batch_tokens is filled with portions of prompts in arrival
//     order, each at most chunk_size if that is set.
//   * Pages are taken step by step, not for prompt + max_tokens at admission
//     (src/paged/scheduler.rs:255).  So they can run out in mid-flight: then the
//     running request that was admitted last is preempted: its pages and slot are
//     given back, its tokens are kept, and it returns to the FRONT of the queue to
//     be recomputed (prompt and generated tokens as one prompt).  A request that
//     is alone and still cannot grow ends with reason "length".
//   * A request that could never fit (longer than the pool or than max_model_len)
//     is refused at submit; the reference would queue it forever
//     (src/paged/scheduler.rs:284-292).
//
// The scheduler decides and keeps books; it runs nothing on the device.  plan()
// reserves the pages of the step it returns; update() takes the sampled tokens.
#pragma once
#include <chrono>
#include <deque>
#include <map>
#include <memory>

#include "cache_book.hpp"

namespace vxh {

enum RequestStatus : int { WAITING = 0, RUNNING = 1, FINISHED = 2 };
enum FinishReason : int { NOT_FINISHED = 0, FINISH_STOP = 1, FINISH_LENGTH = 2, FINISH_CANCELLED = 3 };

struct Request {
    int64_t id = 0;
    std::vector<int> prompt, generated;
    int64_t max_tokens = 0;
    bool ignore_eos = false;
    std::vector<int> stop_ids;  // end-of-sequence and stop tokens alike end the request
    std::vector<std::vector<int>> stop_sequences;  // so does a run of generated tokens that equals one of these
    int status = WAITING;
    int finish_reason = NOT_FINISHED;
    int64_t admitted_at = -1;  // admission counter: the latest is preempted first
    int64_t preemptions = 0;
    int64_t num_tokens() const { return (int64_t)(prompt.size() + generated.size()); }
    int token_at(int64_t i) const {
        return i < (int64_t)prompt.size() ? prompt[i] : generated[i - (int64_t)prompt.size()];
    }
};

struct SchedulerStats {
    int64_t steps = 0, tokens_generated = 0, prompt_tokens = 0, requests_completed = 0, requests_refused = 0,
            preemptions = 0, last_batch_size = 0, last_batch_tokens = 0;
    // requests withdrawn by their caller (not counted as completed)
    int64_t requests_aborted = 0;
    // wall time from the start of plan() to the end of the update() that took the
    // step's tokens: planning, the device's work and the copy back of the sampled ids
    int64_t last_step_us = 0, total_step_us = 0;
};

struct PlanEntry {
    int64_t id;
    int64_t start;   // position of its first token in the request
    int64_t count;
    int wants_last;  // the portion ends the request's tokens: its last place is sampled
};

class Scheduler {
public:
    Scheduler(CacheBook* book, int max_running, int64_t max_batch_tokens, int64_t chunk_size, int64_t max_model_len)
        : book_(book), max_running_(max_running), max_batch_tokens_(max_batch_tokens), chunk_size_(chunk_size) {
        const int64_t limit = (int64_t)book->max_blocks() * book->page_size();
        max_model_len_ = max_model_len > 0 ? std::min(max_model_len, limit) : limit;
    }
    int64_t max_model_len() const { return max_model_len_; }
    SchedulerStats& stats() { return stats_; }
    const std::deque<Request*>& waiting() const { return waiting_; }
    const std::map<int64_t, Request*>& running() const { return running_; }
    const std::map<int64_t, Request*>& finished() const { return finished_; }
    Request* find(int64_t id) {
        auto it = all_.find(id);
        return it == all_.end() ? nullptr : it->second.get();
    }
    bool has_work() const { return !waiting_.empty() || !running_.empty(); }

    // The new request's id, or ERR_REFUSED.
    // stop_sequences: n_seqs runs of tokens, concatenated; seq_lens their lengths.
    int64_t submit(const int* prompt, int64_t n, int64_t max_tokens, bool ignore_eos, const int* stop_ids, int n_stop,
                   const int* stop_sequences = nullptr, const int* seq_lens = nullptr, int n_seqs = 0) {
        if (n <= 0) {  // the reference rejects an empty prompt too (src/paged/scheduler.rs:165-167)
            ++stats_.requests_refused;
            return fail(ERR_REFUSED, "empty prompt");
        }
        const int64_t total = n + max_tokens;
        if (total > max_model_len_) {
            ++stats_.requests_refused;
            return fail(ERR_REFUSED, "prompt (" + std::to_string(n) + ") + max_tokens (" + std::to_string(max_tokens) +
                                         ") exceeds the longest sequence " + std::to_string(max_model_len_));
        }
        const int64_t S = book_->page_size();
        const int64_t pages = (total + S - 1) / S;
        for (int g = 0; g < book_->num_groups(); ++g) {
            CacheGroup& grp = book_->group(g);
            int64_t need = pages;
            if (grp.window > 0)
                need = std::min(pages, (grp.window + std::min(portion_cap(), total) + S - 1) / S + 1);
            if (need > grp.pool.num_pages()) {
                ++stats_.requests_refused;
                return fail(ERR_REFUSED, "the request needs " + std::to_string(need) + " pages of a pool of " +
                                             std::to_string(grp.pool.num_pages()) + " and could never run");
            }
        }
        auto r = std::make_unique<Request>();
        r->id = next_id_++;
        r->prompt.assign(prompt, prompt + n);
        r->max_tokens = max_tokens;
        r->ignore_eos = ignore_eos;
        r->stop_ids.assign(stop_ids, stop_ids + n_stop);
        for (int q = 0; q < n_seqs; ++q) {
            if (seq_lens[q] > 0) r->stop_sequences.emplace_back(stop_sequences, stop_sequences + seq_lens[q]);
            stop_sequences += seq_lens[q];
        }
        Request* p = r.get();
        all_.emplace(p->id, std::move(r));
        waiting_.push_back(p);
        return p->id;
    }

    // The next step: its entries (pages already reserved), the requests that were
    // ended while planning (alone and out of pages), and those admitted (their
    // state slots are fresh).
    int plan() {
        plan_started_ = std::chrono::steady_clock::now();
        entries_.clear();
        ended_.clear();
        admitted_.clear();
        while (true) {
            if (int e = plan_once()) return e;
            if (!entries_.empty() || running_.empty()) return OK;
            // Requests hold cache but none can move (every one waits for pages the
            // others hold): the one admitted last makes room.
            Request* victim = latest_admitted();
            if (running_.size() == 1) {
                if (int e = finish(victim, FINISH_LENGTH)) return e;
                ended_.push_back(victim->id);
            } else if (int e = preempt(victim)) {
                return e;
            }
        }
    }
    const std::vector<PlanEntry>& entries() const { return entries_; }
    const std::vector<int64_t>& ended() const { return ended_; }
    const std::vector<std::pair<int64_t, int>>& admitted() const { return admitted_; }

    // Takes the tokens sampled for the entries that wanted one (in order).  out:
    // (request id, token, finished) per sampled token.
    int update(int n, const int64_t* ids, const int64_t* counts, const int* wants, const int* sampled, int n_sampled,
               int64_t* out_ids, int* out_tokens, int* out_finished) {
        ++stats_.steps;
        stats_.last_batch_size = n;
        stats_.last_batch_tokens = 0;
        int k = 0;
        for (int i = 0; i < n; ++i) stats_.last_batch_tokens += counts[i];
        for (int i = 0; i < n; ++i) {
            auto it = running_.find(ids[i]);
            if (it == running_.end()) return fail(ERR_UNKNOWN_REQUEST, "request " + std::to_string(ids[i]) + " is not running");
            Request* r = it->second;
            if (!wants[i]) {
                stats_.prompt_tokens += counts[i];
                continue;
            }
            if (k >= n_sampled) return fail(ERR_VALUE, "fewer sampled tokens than entries that wanted one");
            const int tok = sampled[k];
            if (counts[i] > 1 || r->generated.empty()) stats_.prompt_tokens += counts[i];
            r->generated.push_back(tok);
            ++stats_.tokens_generated;
            int reason = NOT_FINISHED;
            if (!r->ignore_eos && std::find(r->stop_ids.begin(), r->stop_ids.end(), tok) != r->stop_ids.end())
                reason = FINISH_STOP;
            else if (ends_with_stop_sequence(*r))
                reason = FINISH_STOP;
            else if ((int64_t)r->generated.size() >= r->max_tokens)
                reason = FINISH_LENGTH;
            else if (r->num_tokens() >= max_model_len_)
                reason = FINISH_LENGTH;
            if (reason)
                if (int e = finish(r, reason)) return e;
            out_ids[k] = r->id;
            out_tokens[k] = tok;
            out_finished[k] = reason != NOT_FINISHED;
            ++k;
        }
        stats_.last_step_us = std::chrono::duration_cast<std::chrono::microseconds>(
                                  std::chrono::steady_clock::now() - plan_started_).count();
        stats_.total_step_us += stats_.last_step_us;
        return k;
    }

    int finish(Request* r, int reason) {
        if (book_->find(r->id))
            if (int e = book_->release(r->id)) return e;
        running_.erase(r->id);
        r->status = FINISHED;
        r->finish_reason = reason;
        finished_[r->id] = r;
        ++(reason == FINISH_CANCELLED ? stats_.requests_aborted : stats_.requests_completed);
        return OK;
    }
    // Withdraws a request, waiting or running: what it holds of the cache is given
    // back at once, its tokens so far are kept, its reason is "cancelled"
    // (src/paged/scheduler.rs:440-452 ends a request whose client is gone so).
    // 1 if it was withdrawn, 0 if it had finished already.  To be called between
    // steps: a step that was planned with the request must have been taken by update().
    int cancel(int64_t id) {
        Request* r = find(id);
        if (!r) return fail(ERR_UNKNOWN_REQUEST, "no request " + std::to_string(id));
        if (r->status == FINISHED) return 0;
        if (r->status == WAITING) waiting_.erase(std::find(waiting_.begin(), waiting_.end(), r));
        if (int e = finish(r, FINISH_CANCELLED)) return e;
        return 1;
    }
    // Drops a finished request's record (its tokens have been read).
    void forget(int64_t id) {
        auto it = finished_.find(id);
        if (it == finished_.end()) return;
        finished_.erase(it);
        all_.erase(id);
    }

private:
    static bool ends_with_stop_sequence(const Request& r) {
        for (const auto& q : r.stop_sequences)
            if (q.size() <= r.generated.size() && std::equal(q.begin(), q.end(), r.generated.end() - (long)q.size()))
                return true;
        return false;
    }
    int64_t portion_cap() const { return chunk_size_ > 0 ? std::min(max_batch_tokens_, chunk_size_) : max_batch_tokens_; }
    int64_t remaining(const Request* r) { return r->num_tokens() - book_->find(r->id)->length; }
    Request* latest_admitted() {
        Request* best = nullptr;
        for (auto& kv : running_)
            if (!best || kv.second->admitted_at > best->admitted_at) best = kv.second;
        return best;
    }
    int preempt(Request* victim) {
        if (int e = book_->release(victim->id)) return e;
        running_.erase(victim->id);
        victim->status = WAITING;
        ++victim->preemptions;
        ++stats_.preemptions;
        waiting_.push_front(victim);
        return OK;
    }
    // The largest portion <= k whose pages can be reserved now (reserves it); < 0 on error.
    int64_t fit(int64_t id, int64_t k) {
        while (k > 0) {
            const int r = book_->reserve(id, k);
            if (r < 0) return r;
            if (r == 1) return k;
            // fewer pages: shrink to what the scarcest group can still hold
            k = std::min(k - 1, book_->room(*book_->find(id)));
        }
        return 0;
    }

    int plan_once() {
        int64_t budget = max_batch_tokens_;
        std::map<int64_t, int64_t> chosen;
        bool preempted = false;

        // 1. requests that decode: one token each, oldest id first
        std::vector<int64_t> ids;
        for (auto& kv : running_) ids.push_back(kv.first);
        for (int64_t id : ids) {
            auto it = running_.find(id);
            if (it == running_.end()) continue;  // preempted a moment ago
            Request* r = it->second;
            if (remaining(r) != 1 || r->generated.empty()) continue;
            if (budget <= 0) break;
            bool got = false;
            while (true) {
                const int res = book_->reserve(id, 1);
                if (res < 0) return res;
                if (res == 1) {
                    got = true;
                    break;
                }
                Request* victim = latest_admitted();
                if (victim == r && running_.size() == 1) {
                    if (int e = finish(r, FINISH_LENGTH)) return e;
                    ended_.push_back(r->id);
                    break;
                }
                chosen.erase(victim->id);
                if (int e = preempt(victim)) return e;
                preempted = true;
                if (victim == r) break;
            }
            if (got) {
                chosen[id] = 1;
                --budget;
            }
        }

        // 2. prompts under way (and recomputations), oldest id first
        for (auto& kv : running_) {
            const int64_t id = kv.first;
            Request* r = kv.second;
            if (chosen.count(id) || budget <= 0) continue;
            const int64_t rem = remaining(r);
            if (rem == 1 && !r->generated.empty()) continue;  // a decode that found no budget
            const int64_t k = fit(id, std::min({rem, budget, portion_cap()}));
            if (k < 0) return (int)k;
            if (k > 0) {
                chosen[id] = k;
                budget -= k;
            }
        }

        // 3. admissions, first come first served; none in a step that had to preempt
        // (the pages just freed are for those that stayed)
        while (!preempted && !waiting_.empty() && budget > 0 && (int)running_.size() < max_running_) {
            Request* r = waiting_.front();
            const int slot = book_->add(r->id);
            if (slot < -1) return slot;
            if (slot < 0) break;
            const int64_t k = fit(r->id, std::min({r->num_tokens(), budget, portion_cap()}));
            if (k < 0) return (int)k;
            if (k == 0) {
                if (int e = book_->release(r->id)) return e;
                if (running_.empty()) {  // nothing will ever free a page for it
                    waiting_.pop_front();
                    if (int e = finish(r, FINISH_LENGTH)) return e;
                    ended_.push_back(r->id);
                    continue;
                }
                break;  // head of the line waits; nobody overtakes it
            }
            waiting_.pop_front();
            r->status = RUNNING;
            r->admitted_at = admissions_++;
            running_[r->id] = r;
            admitted_.emplace_back(r->id, slot);
            chosen[r->id] = k;
            budget -= k;
        }

        for (auto& kv : chosen) {
            Request* r = running_.at(kv.first);
            const int64_t done = book_->find(r->id)->length;
            entries_.push_back({r->id, done, kv.second, done + kv.second == r->num_tokens() ? 1 : 0});
        }
        // a request admitted and preempted again within this planning round holds no slot any more
        admitted_.erase(std::remove_if(admitted_.begin(), admitted_.end(),
                                       [&](const std::pair<int64_t, int>& a) { return !running_.count(a.first); }),
                        admitted_.end());
        return OK;
    }

    CacheBook* book_;
    int max_running_;
    int64_t max_batch_tokens_, chunk_size_, max_model_len_ = 0;
    std::deque<Request*> waiting_;
    std::map<int64_t, Request*> running_, finished_;
    std::unordered_map<int64_t, std::unique_ptr<Request>> all_;
    SchedulerStats stats_;
    int64_t next_id_ = 0, admissions_ = 0;
    std::chrono::steady_clock::time_point plan_started_ = std::chrono::steady_clock::now();
    std::vector<PlanEntry> entries_;
    std::vector<int64_t> ended_;
    std::vector<std::pair<int64_t, int>> admitted_;
};

}  // namespace vxh
