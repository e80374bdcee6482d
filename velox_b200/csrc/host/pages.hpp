// Page ids and state slots: the host-side bookkeeping of the cache.
//
// PagePool follows the reference's free list and reference counts
// (src/paged/pages.rs:113, 173-242): a stack of free ids made so that page 0 is
// handed out first, alloc(n) all or nothing, a count per page that free() lowers
// and that returns the page to the stack at zero.  Where the reference only
// warns about a bad id or a second free (src/paged/pages.rs:205-212), these
// fail: a page freed twice would be handed to two requests.
#pragma once
#include <string>
#include <vector>

#include "status.hpp"

namespace vxh {

class PagePool {
public:
    explicit PagePool(int num_pages) : n_(num_pages), refs_(num_pages, 0) {
        free_.reserve(num_pages);
        for (int p = num_pages - 1; p >= 0; --p) free_.push_back(p);
    }
    int num_pages() const { return n_; }
    int num_free() const { return (int)free_.size(); }
    const std::vector<int>& free_list() const { return free_; }

    // n pages with count 1 into out: 1; 0 (and nothing taken) if fewer are free.
    int alloc(int n, int* out) {
        if (n < 0) return fail(ERR_VALUE, "cannot allocate " + std::to_string(n) + " pages");
        if ((int)free_.size() < n) return 0;
        for (int i = 0; i < n; ++i) {
            const int p = free_.back();
            free_.pop_back();
            if (refs_[p] != 0)
                return fail(ERR_ACCOUNTING, "page " + std::to_string(p) + " was on the free list with count " +
                                                std::to_string(refs_[p]));
            refs_[p] = 1;
            out[i] = p;
        }
        return 1;
    }
    int incref(const int* pages, int n) {
        for (int i = 0; i < n; ++i) {
            const int p = pages[i];
            if (int e = check(p)) return e;
            if (refs_[p] < 1) return fail(ERR_ACCOUNTING, "page " + std::to_string(p) + " is free and cannot be shared");
            ++refs_[p];
        }
        return OK;
    }
    int free(const int* pages, int n) {
        for (int i = 0; i < n; ++i) {
            const int p = pages[i];
            if (int e = check(p)) return e;
            if (refs_[p] < 1) return fail(ERR_ACCOUNTING, "page " + std::to_string(p) + " freed twice");
            if (--refs_[p] == 0) free_.push_back(p);
        }
        return OK;
    }
    int refcount(int p) {
        if (int e = check(p)) return e;
        return refs_[p];
    }

private:
    int check(int p) const {
        if (p < 0 || p >= n_)
            return fail(ERR_ACCOUNTING, "page id " + std::to_string(p) + " is outside the pool of " + std::to_string(n_));
        return OK;
    }
    int n_;
    std::vector<int> free_, refs_;
};

// Slots for per-request state of fixed size; the lowest free slot first.
class SlotPool {
public:
    explicit SlotPool(int num_slots) : n_(num_slots), held_(num_slots, 0) {
        for (int s = num_slots - 1; s >= 0; --s) free_.push_back(s);
    }
    int num_slots() const { return n_; }
    int num_free() const { return (int)free_.size(); }
    int alloc() {  // -1: none free
        if (free_.empty()) return -1;
        const int s = free_.back();
        free_.pop_back();
        held_[s] = 1;
        return s;
    }
    int free(int slot) {
        if (slot < 0 || slot >= n_ || !held_[slot])
            return fail(ERR_ACCOUNTING, "state slot " + std::to_string(slot) + " is not held");
        held_[slot] = 0;
        free_.push_back(slot);
        return OK;
    }

private:
    int n_;
    std::vector<int> free_;
    std::vector<char> held_;
};

}  // namespace vxh
