// The C interface of the host library (loaded with ctypes): page and slot pools,
// the cache manager's books, the step builders and the scheduler.  Functions
// return a value >= 0 or a negative Status; vxh_last_error() gives the message
// of the calling thread's last failure.
#include <cstring>

#include "scheduler.hpp"
#include "step_builder.hpp"

using namespace vxh;

extern "C" {

const char* vxh_last_error(void) { return last_error().c_str(); }

// ---- pools ----
void* vxh_pages_create(int n) { return n > 0 ? new PagePool(n) : nullptr; }
void vxh_pages_destroy(void* p) { delete (PagePool*)p; }
int vxh_pages_num_pages(void* p) { return ((PagePool*)p)->num_pages(); }
int vxh_pages_num_free(void* p) { return ((PagePool*)p)->num_free(); }
int vxh_pages_alloc(void* p, int n, int* out) { return ((PagePool*)p)->alloc(n, out); }
int vxh_pages_incref(void* p, const int* pages, int n) { return ((PagePool*)p)->incref(pages, n); }
int vxh_pages_free(void* p, const int* pages, int n) { return ((PagePool*)p)->free(pages, n); }
int vxh_pages_refcount(void* p, int page) { return ((PagePool*)p)->refcount(page); }
int vxh_pages_free_list(void* p, int* out, int cap) {
    const auto& f = ((PagePool*)p)->free_list();
    const int n = (int)std::min<size_t>(f.size(), (size_t)cap);
    std::memcpy(out, f.data(), sizeof(int) * n);
    return (int)f.size();
}

void* vxh_slots_create(int n) { return n > 0 ? new SlotPool(n) : nullptr; }
void vxh_slots_destroy(void* p) { delete (SlotPool*)p; }
int vxh_slots_num_slots(void* p) { return ((SlotPool*)p)->num_slots(); }
int vxh_slots_num_free(void* p) { return ((SlotPool*)p)->num_free(); }
int vxh_slots_alloc(void* p) { return ((SlotPool*)p)->alloc(); }
int vxh_slots_free(void* p, int slot) { return ((SlotPool*)p)->free(slot); }

// ---- cache book ----
void* vxh_cache_create(int n_groups, const int* windows, int page_size, int num_pages, int max_requests, int max_blocks) {
    if (n_groups < 0 || page_size <= 0 || num_pages <= 0 || max_requests <= 0 || max_blocks <= 0) return nullptr;
    return new CacheBook(n_groups, windows, page_size, num_pages, max_requests, max_blocks);
}
void vxh_cache_destroy(void* c) { delete (CacheBook*)c; }
void* vxh_cache_pool(void* c, int g) { return &((CacheBook*)c)->group(g).pool; }
void* vxh_cache_slots(void* c) { return &((CacheBook*)c)->slots(); }
int vxh_cache_add(void* c, int64_t rid) { return ((CacheBook*)c)->add(rid); }
int vxh_cache_has(void* c, int64_t rid) { return ((CacheBook*)c)->find(rid) != nullptr; }
long long vxh_cache_num_requests(void* c) { return (long long)((CacheBook*)c)->num_requests(); }
long long vxh_cache_request_ids(void* c, int64_t* out, long long cap) {
    long long n = 0;
    ((CacheBook*)c)->for_each([&](int64_t id, RequestCache&) {
        if (n < cap) out[n] = id;
        ++n;
    });
    return n;
}
long long vxh_cache_length(void* c, int64_t rid) {
    RequestCache* rc = ((CacheBook*)c)->need(rid);
    return rc ? (long long)rc->length : (long long)ERR_UNKNOWN_REQUEST;
}
long long vxh_cache_max_length(void* c, int n, const int64_t* rids) {  // the longest of these requests
    long long best = 0;
    for (int i = 0; i < n; ++i) {
        RequestCache* rc = ((CacheBook*)c)->need(rids[i]);
        if (!rc) return ERR_UNKNOWN_REQUEST;
        best = std::max<long long>(best, rc->length);
    }
    return best;
}
int vxh_cache_slot(void* c, int64_t rid) {
    RequestCache* rc = ((CacheBook*)c)->need(rid);
    return rc ? rc->slot : (int)ERR_UNKNOWN_REQUEST;
}
int vxh_cache_table(void* c, int64_t rid, int g, int* out, int cap) {  // the table's length; entries copied up to cap
    RequestCache* rc = ((CacheBook*)c)->need(rid);
    if (!rc) return ERR_UNKNOWN_REQUEST;
    const auto& t = rc->tables[g];
    std::memcpy(out, t.data(), sizeof(int) * std::min<size_t>(t.size(), (size_t)cap));
    return (int)t.size();
}
int vxh_cache_pages_needed(void* c, int64_t rid, long long new_tokens, int* out) {
    CacheBook* b = (CacheBook*)c;
    RequestCache* rc = b->need(rid);
    if (!rc) return ERR_UNKNOWN_REQUEST;
    b->pages_needed(*rc, new_tokens, out);
    return OK;
}
int vxh_cache_can_reserve(void* c, int64_t rid, long long n) { return ((CacheBook*)c)->can_reserve(rid, n); }
int vxh_cache_reserve(void* c, int64_t rid, long long n) { return ((CacheBook*)c)->reserve(rid, n); }
int vxh_cache_commit(void* c, int64_t rid, long long n) { return ((CacheBook*)c)->commit(rid, n); }
int vxh_cache_release(void* c, int64_t rid) { return ((CacheBook*)c)->release(rid); }
int vxh_cache_check(void* c) { return ((CacheBook*)c)->check(); }
// reserve (or commit) for every entry of a step; the index of the first entry that found no pages, or n
int vxh_cache_reserve_many(void* c, int n, const int64_t* rids, const int* counts) {
    for (int i = 0; i < n; ++i) {
        const int r = ((CacheBook*)c)->reserve(rids[i], counts[i]);
        if (r < 0) return r;
        if (r == 0) return i;
    }
    return n;
}
int vxh_cache_commit_many(void* c, int n, const int64_t* rids, const int* counts) {
    for (int i = 0; i < n; ++i)
        if (int e = ((CacheBook*)c)->commit(rids[i], counts[i])) return e;
    return OK;
}

// ---- step builders ----
int vxh_build_step(void* c, int n, const int64_t* rids, const int* lens, const int* tokens, const int* want_counts,
                   const int* wants, int vocab, int short_max, int32_t* dst, const int64_t* starts, int64_t* summary) {
    return build_step(*(CacheBook*)c, n, rids, lens, tokens, want_counts, wants, vocab, short_max, dst, starts, summary);
}
int vxh_fill_decode(void* c, int n, int bucket, const int64_t* rids, const int* tokens, int vocab, int32_t* dst,
                    const int64_t* starts, int64_t* max_kv) {
    return fill_decode(*(CacheBook*)c, n, bucket, rids, tokens, vocab, dst, starts, max_kv);
}

// ---- scheduler ----
void* vxh_sched_create(void* cache, int max_running, long long max_batch_tokens, long long chunk_size,
                       long long max_model_len) {
    if (!cache || max_running <= 0 || max_batch_tokens <= 0) return nullptr;
    return new Scheduler((CacheBook*)cache, max_running, max_batch_tokens, chunk_size, max_model_len);
}
void vxh_sched_destroy(void* s) { delete (Scheduler*)s; }
long long vxh_sched_max_model_len(void* s) { return ((Scheduler*)s)->max_model_len(); }
long long vxh_sched_submit(void* s, const int* prompt, long long n, long long max_tokens, int ignore_eos,
                           const int* stop_ids, int n_stop, const int* stop_sequences, const int* seq_lens, int n_seqs) {
    return ((Scheduler*)s)->submit(prompt, n, max_tokens, ignore_eos != 0, stop_ids, n_stop, stop_sequences, seq_lens,
                                   n_seqs);
}
int vxh_sched_has_work(void* s) { return ((Scheduler*)s)->has_work(); }
// Plans a step.  counts: entries, tokens of all entries, ended, admitted.
int vxh_sched_plan(void* s, long long* counts) {
    Scheduler* sc = (Scheduler*)s;
    if (int e = sc->plan()) return e;
    long long tokens = 0;
    for (auto& e : sc->entries()) tokens += e.count;
    counts[0] = (long long)sc->entries().size();
    counts[1] = tokens;
    counts[2] = (long long)sc->ended().size();
    counts[3] = (long long)sc->admitted().size();
    return OK;
}
// The last plan: per entry (id, start, count, wants_last) and its tokens, concatenated.
int vxh_sched_plan_entries(void* s, int64_t* ids, int64_t* starts, int64_t* lens, int* wants, int* tokens) {
    Scheduler* sc = (Scheduler*)s;
    size_t i = 0;
    for (auto& e : sc->entries()) {
        ids[i] = e.id;
        starts[i] = e.start;
        lens[i] = e.count;
        wants[i] = e.wants_last;
        Request* r = sc->find(e.id);
        for (int64_t j = 0; j < e.count; ++j) *tokens++ = r->token_at(e.start + j);
        ++i;
    }
    return OK;
}
int vxh_sched_plan_ended(void* s, int64_t* ids) {
    const auto& v = ((Scheduler*)s)->ended();
    std::copy(v.begin(), v.end(), ids);
    return OK;
}
int vxh_sched_plan_admitted(void* s, int64_t* ids, int* slots) {
    size_t i = 0;
    for (auto& a : ((Scheduler*)s)->admitted()) {
        ids[i] = a.first;
        slots[i++] = a.second;
    }
    return OK;
}
int vxh_sched_update(void* s, int n, const int64_t* ids, const int64_t* counts, const int* wants, const int* sampled,
                     int n_sampled, int64_t* out_ids, int* out_tokens, int* out_finished) {
    return ((Scheduler*)s)->update(n, ids, counts, wants, sampled, n_sampled, out_ids, out_tokens, out_finished);
}
int vxh_sched_finish(void* s, int64_t id, int reason) {
    Scheduler* sc = (Scheduler*)s;
    Request* r = sc->find(id);
    if (!r) return fail(ERR_UNKNOWN_REQUEST, "no request " + std::to_string(id));
    return sc->finish(r, reason);
}
int vxh_sched_cancel(void* s, int64_t id) { return ((Scheduler*)s)->cancel(id); }
void vxh_sched_forget(void* s, int64_t id) { ((Scheduler*)s)->forget(id); }
// which: 0 waiting (queue order), 1 running, 2 finished (by id).  The number of ids; copied up to cap.
long long vxh_sched_list(void* s, int which, int64_t* out, long long cap) {
    Scheduler* sc = (Scheduler*)s;
    long long n = 0;
    auto put = [&](int64_t id) {
        if (n < cap) out[n] = id;
        ++n;
    };
    if (which == 0)
        for (Request* r : sc->waiting()) put(r->id);
    else
        for (auto& kv : (which == 1 ? sc->running() : sc->finished())) put(kv.first);
    return n;
}
int vxh_sched_contains(void* s, int which, int64_t id) {
    Scheduler* sc = (Scheduler*)s;
    if (which == 1) return sc->running().count(id) != 0;
    if (which == 2) return sc->finished().count(id) != 0;
    for (Request* r : sc->waiting())
        if (r->id == id) return 1;
    return 0;
}
// info: prompt tokens, generated tokens, status, finish reason, admitted_at, preemptions, max_tokens
int vxh_sched_request(void* s, int64_t id, int64_t* info) {
    Request* r = ((Scheduler*)s)->find(id);
    if (!r) return fail(ERR_UNKNOWN_REQUEST, "no request " + std::to_string(id));
    info[0] = (int64_t)r->prompt.size();
    info[1] = (int64_t)r->generated.size();
    info[2] = r->status;
    info[3] = r->finish_reason;
    info[4] = r->admitted_at;
    info[5] = r->preemptions;
    info[6] = r->max_tokens;
    return OK;
}
int vxh_sched_request_tokens(void* s, int64_t id, int generated, long long start, long long stop, int* out) {
    Request* r = ((Scheduler*)s)->find(id);
    if (!r) return fail(ERR_UNKNOWN_REQUEST, "no request " + std::to_string(id));
    const auto& v = generated ? r->generated : r->prompt;
    if (start < 0 || stop > (long long)v.size() || start > stop) return fail(ERR_VALUE, "token range outside the request");
    std::copy(v.begin() + start, v.begin() + stop, out);
    return OK;
}
int vxh_sched_stats(void* s, int64_t* out) {
    const SchedulerStats& st = ((Scheduler*)s)->stats();
    const int64_t v[11] = {st.steps, st.tokens_generated, st.prompt_tokens, st.requests_completed,
                           st.requests_refused, st.preemptions, st.last_batch_size, st.last_batch_tokens,
                           st.requests_aborted, st.last_step_us, st.total_step_us};
    std::memcpy(out, v, sizeof(v));
    return OK;
}

}  // extern "C"
