// The cache manager's books: block tables per request in groups of layers with
// the same needs, and the state slot of each request.
//
// A group has its own page pool and, per request, its own block table: entry i
// is the page that holds positions [i*S, (i+1)*S), or -1.  Pages are taken when a
// step needs them (reserve), not for the worst case at admission as the
// reference does (src/paged/scheduler.rs:255).  They are given back when the
// request ends, and in a group with a window as soon as every position of a page
// lies before the window of the next query; the freed page is the next one
// handed out.  Beside the tables the book keeps, per group, a dense mirror
// [slot, block] (-1 where no page is held), from which the step builders copy
// whole rows.
//
// The device storage (the pools of keys and values, the state tensors) is not
// here: the book only knows ids.
#pragma once
#include <algorithm>
#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

#include "pages.hpp"

namespace vxh {

struct RequestCache {
    int slot = -1;
    int64_t length = 0;                     // positions whose keys/values (or state) are in the cache
    std::vector<std::vector<int>> tables;   // per group
};

struct CacheGroup {
    int window;
    PagePool pool;
    std::vector<int32_t> mirror;  // [max_requests, max_blocks]
    CacheGroup(int window_, int num_pages, size_t cells) : window(window_), pool(num_pages), mirror(cells, -1) {}
};

class CacheBook {
public:
    CacheBook(int n_groups, const int* windows, int page_size, int num_pages, int max_requests, int max_blocks)
        : page_size_(page_size), max_blocks_(max_blocks), max_requests_(max_requests), slots_(max_requests) {
        groups_.reserve(n_groups);
        for (int g = 0; g < n_groups; ++g)
            groups_.emplace_back(windows[g], num_pages, (size_t)max_requests * max_blocks);
    }
    int page_size() const { return page_size_; }
    int max_blocks() const { return max_blocks_; }
    int num_groups() const { return (int)groups_.size(); }
    CacheGroup& group(int g) { return groups_[g]; }
    SlotPool& slots() { return slots_; }
    size_t num_requests() const { return reqs_.size(); }

    RequestCache* find(int64_t rid) {
        auto it = reqs_.find(rid);
        return it == reqs_.end() ? nullptr : &it->second;
    }
    RequestCache* need(int64_t rid) {
        RequestCache* rc = find(rid);
        if (!rc) fail(ERR_UNKNOWN_REQUEST, "request " + std::to_string(rid) + " holds no cache");
        return rc;
    }

    // A state slot and empty block tables: the slot, -1 if none is free.
    int add(int64_t rid) {
        if (find(rid)) return fail(ERR_ACCOUNTING, "request " + std::to_string(rid) + " already holds cache");
        const int slot = slots_.alloc();
        if (slot < 0) return -1;
        RequestCache rc;
        rc.slot = slot;
        rc.tables.resize(groups_.size());
        reqs_.emplace(rid, std::move(rc));
        for (auto& g : groups_) std::fill_n(g.mirror.begin() + (size_t)slot * max_blocks_, max_blocks_, -1);
        return slot;
    }

    // Per group, the pages reserve() would have to take for new_tokens more positions.
    void pages_needed(const RequestCache& rc, int64_t new_tokens, int* out) const {
        const int64_t want = (rc.length + new_tokens + page_size_ - 1) / page_size_;
        for (size_t g = 0; g < groups_.size(); ++g)
            out[g] = (int)std::max<int64_t>(0, want - (int64_t)rc.tables[g].size());
    }
    int can_reserve(int64_t rid, int64_t new_tokens) {
        RequestCache* rc = need(rid);
        if (!rc) return ERR_UNKNOWN_REQUEST;
        std::vector<int> n(groups_.size());
        pages_needed(*rc, new_tokens, n.data());
        for (size_t g = 0; g < groups_.size(); ++g)
            if (n[g] > groups_[g].pool.num_free()) return 0;
        return 1;
    }
    // Takes, in every group, the pages for positions [length, length + new_tokens);
    // all or nothing.  1; 0 if some group has too few free pages.
    int reserve(int64_t rid, int64_t new_tokens) {
        RequestCache* rc = need(rid);
        if (!rc) return ERR_UNKNOWN_REQUEST;
        if (rc->length + new_tokens > (int64_t)max_blocks_ * page_size_)
            return fail(ERR_OUT_OF_PAGES, "request " + std::to_string(rid) + " would reach " +
                                              std::to_string(rc->length + new_tokens) + " positions; block tables hold " +
                                              std::to_string((int64_t)max_blocks_ * page_size_));
        std::vector<int> n(groups_.size());
        pages_needed(*rc, new_tokens, n.data());
        for (size_t g = 0; g < groups_.size(); ++g)
            if (n[g] > groups_[g].pool.num_free()) return 0;
        for (size_t g = 0; g < groups_.size(); ++g) {
            if (!n[g]) continue;
            auto& table = rc->tables[g];
            const size_t at = table.size();
            table.resize(at + n[g]);
            const int r = groups_[g].pool.alloc(n[g], table.data() + at);
            if (r != 1) return r < 0 ? r : fail(ERR_ACCOUNTING, "the free list shrank under a reservation");
            std::copy(table.begin() + at, table.end(), groups_[g].mirror.begin() + (size_t)rc->slot * max_blocks_ + at);
        }
        return 1;
    }
    // The step has written new_tokens positions: advance, and give back pages
    // that every later query's window has passed.
    int commit(int64_t rid, int64_t new_tokens) {
        RequestCache* rc = need(rid);
        if (!rc) return ERR_UNKNOWN_REQUEST;
        rc->length += new_tokens;
        for (size_t g = 0; g < groups_.size(); ++g) {
            auto& table = rc->tables[g];
            if ((int64_t)table.size() * page_size_ < rc->length)
                return fail(ERR_ACCOUNTING, "request " + std::to_string(rid) + " wrote " + std::to_string(rc->length) +
                                                " positions into " + std::to_string(table.size()) + " pages");
            if (groups_[g].window > 0) {
                // the first page that the query at position `length` can still see
                const int64_t first_key = std::max<int64_t>(0, rc->length + 1 - groups_[g].window);
                const int64_t keep_from = std::min<int64_t>(first_key / page_size_, (int64_t)table.size());
                for (int64_t i = 0; i < keep_from; ++i) {
                    if (table[i] < 0) continue;
                    if (int e = groups_[g].pool.free(&table[i], 1)) return e;
                    table[i] = -1;
                    groups_[g].mirror[(size_t)rc->slot * max_blocks_ + i] = -1;
                }
            }
        }
        return OK;
    }
    // Gives back everything the request holds.
    int release(int64_t rid) {
        auto it = reqs_.find(rid);
        if (it == reqs_.end()) return fail(ERR_UNKNOWN_REQUEST, "request " + std::to_string(rid) + " holds no cache");
        RequestCache rc = std::move(it->second);
        reqs_.erase(it);
        for (size_t g = 0; g < groups_.size(); ++g)
            for (int p : rc.tables[g])
                if (p >= 0)
                    if (int e = groups_[g].pool.free(&p, 1)) return e;
        return slots_.free(rc.slot);
    }
    // Positions the request could still take before some group runs dry.
    int64_t room(const RequestCache& rc) const {
        int64_t best = INT64_MAX;
        for (size_t g = 0; g < groups_.size(); ++g)
            best = std::min(best, ((int64_t)rc.tables[g].size() + groups_[g].pool.num_free()) * page_size_ - rc.length);
        return best;
    }
    // Every page is either free or held by exactly as many tables as its count says.
    int check() {
        for (size_t g = 0; g < groups_.size(); ++g) {
            PagePool& pool = groups_[g].pool;
            std::vector<int> held(pool.num_pages(), 0), on_free(pool.num_pages(), 0);
            for (auto& kv : reqs_)
                for (int p : kv.second.tables[g])
                    if (p >= 0) {
                        if (p >= pool.num_pages()) return fail(ERR_ACCOUNTING, "a table holds page id " + std::to_string(p));
                        ++held[p];
                    }
            for (int p : pool.free_list())
                if (++on_free[p] > 1)
                    return fail(ERR_ACCOUNTING, "group " + std::to_string(g) + ": a page is on the free list twice");
            for (int p = 0; p < pool.num_pages(); ++p) {
                const int cnt = pool.refcount(p);
                if ((on_free[p] != 0) != (cnt == 0) || held[p] != cnt)
                    return fail(ERR_ACCOUNTING, "group " + std::to_string(g) + " page " + std::to_string(p) + ": count " +
                                                    std::to_string(cnt) + ", held by " + std::to_string(held[p]) +
                                                    " tables, " + (on_free[p] ? "on" : "not on") + " the free list");
            }
        }
        return OK;
    }
    template <typename F>
    void for_each(F f) {
        for (auto& kv : reqs_) f(kv.first, kv.second);
    }

private:
    int page_size_, max_blocks_, max_requests_;
    std::vector<CacheGroup> groups_;
    SlotPool slots_;
    std::unordered_map<int64_t, RequestCache> reqs_;
};

}  // namespace vxh
