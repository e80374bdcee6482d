// The description of one step that the kernels read, written into one (pinned)
// buffer of 32-bit words whose sections start at the given offsets:
//   0 token_ids [tokens]      1 positions [tokens]     2 seq_of_token [tokens]
//   3 cu_seqlens [requests+1] 4 kv_offsets [requests]  5 state_slots [requests]
//   6 wanted_rows [wanted]    7 single_rows [tokens]    8 portion_seqs [requests]
//   then per group: block_table [requests, max_blocks], slot_mapping [tokens] (page *
//   page_size + offset of each new position).
// single_rows lists the token rows of the requests that bring at most `short_max`
// tokens (1: exactly the decoded tokens), portion_seqs the requests (rows of the
// step) that bring more: a mixed step hands the first, token by token, to the decode
// attention (every token a query of its own over its request's keys, the range of keys
// cut into pieces that many warps share) and the second to the prompt attention.
// The reference rebuilds and uploads block tables and offsets inside every layer
// (src/paged/qwen3.rs:584-627); here the description is built once per step and
// shared by all layers.
#pragma once
#include <cstring>

#include "cache_book.hpp"

namespace vxh {

// A general step: request i brings lens[i] tokens (concatenated in `tokens`) and
// asks for want_counts[i] places among them (concatenated in `wants`).  The pages
// must have been reserved.  summary: total tokens, wanted rows, longest portion,
// largest number of keys any request will have, token rows of short requests, the
// largest number of keys among those requests, requests that bring more than
// `short_max` tokens, the longest short request.
inline int build_step(CacheBook& book, int n, const int64_t* rids, const int* lens, const int* tokens,
                      const int* want_counts, const int* wants, int vocab, int short_max, int32_t* dst,
                      const int64_t* starts, int64_t* summary) {
    const int S = book.page_size(), MB = book.max_blocks(), G = book.num_groups();
    int32_t* token_ids = dst + starts[0];
    int32_t* positions = dst + starts[1];
    int32_t* seq_of_token = dst + starts[2];
    int32_t* cu = dst + starts[3];
    int32_t* offsets = dst + starts[4];
    int32_t* slots = dst + starts[5];
    int32_t* wanted = dst + starts[6];
    int32_t* single_rows = dst + starts[7];
    int32_t* portion_seqs = dst + starts[8];
    int64_t row = 0, nw = 0, max_new = 0, max_kv = 0, n_single = 0, n_portions = 0, max_kv_single = 0, max_short = 0;
    if (short_max < 1) short_max = 1;
    const int* tok = tokens;
    const int* want = wants;
    cu[0] = 0;
    for (int i = 0; i < n; ++i) {
        RequestCache* rc = book.need(rids[i]);
        if (!rc) return ERR_UNKNOWN_REQUEST;
        const int k = lens[i];
        for (int j = 0; j < k; ++j) {
            if (vocab >= 0 && (tok[j] < 0 || tok[j] >= vocab))
                return fail(ERR_VALUE, "entry " + std::to_string(i) + ": token id outside [0, " + std::to_string(vocab) + ")");
            token_ids[row + j] = tok[j];
            positions[row + j] = (int32_t)(rc->length + j);
            seq_of_token[row + j] = i;
        }
        cu[i + 1] = (int32_t)(row + k);
        offsets[i] = (int32_t)rc->length;
        slots[i] = rc->slot;
        for (int w = 0; w < want_counts[i]; ++w) {
            if (want[w] < 0 || want[w] >= k)
                return fail(ERR_VALUE, "entry " + std::to_string(i) + ": wanted place " + std::to_string(want[w]) +
                                           " is not among its " + std::to_string(k) + " tokens");
            wanted[nw++] = (int32_t)(row + want[w]);
        }
        for (int g = 0; g < G; ++g) {
            const auto& table = rc->tables[g];
            if ((int64_t)table.size() * S < rc->length + k)
                return fail(ERR_VALUE, "entry " + std::to_string(i) + ": block table too short (" +
                                           std::to_string(table.size()) + " pages for " + std::to_string(rc->length + k) +
                                           " positions)");
            int32_t* bt = dst + starts[9 + 2 * g] + (int64_t)i * MB;
            int32_t* sm = dst + starts[10 + 2 * g] + row;
            std::memcpy(bt, book.group(g).mirror.data() + (size_t)rc->slot * MB, sizeof(int32_t) * MB);
            for (int j = 0; j < k; ++j) {
                const int64_t pos = rc->length + j;
                const int page = table[pos / S];
                if (page < 0)
                    return fail(ERR_VALUE, "entry " + std::to_string(i) + ": a new position falls into a page that was given back");
                sm[j] = (int32_t)(page * S + pos % S);
            }
        }
        if (k <= short_max) {
            for (int j = 0; j < k; ++j) single_rows[n_single++] = (int32_t)(row + j);
            max_kv_single = std::max<int64_t>(max_kv_single, rc->length + k);
            max_short = std::max<int64_t>(max_short, k);
        } else {
            portion_seqs[n_portions++] = i;
        }
        row += k;
        tok += k;
        want += want_counts[i];
        max_new = std::max<int64_t>(max_new, k);
        max_kv = std::max<int64_t>(max_kv, rc->length + k);
    }
    summary[0] = row;
    summary[1] = nw;
    summary[2] = max_new;
    summary[3] = max_kv;
    summary[4] = n_single;
    summary[5] = max_kv_single;
    summary[6] = n_portions;
    summary[7] = max_short;
    return OK;
}

// A step of decoded tokens only (one per request), padded to `bucket` rows that
// read page 0 at position 0 and write nothing (slot -1).  Only the columns of the
// block tables that these requests can reach are written.  The sections for
// seq_of_token, cu_seqlens, wanted_rows, single_rows and portion_seqs are constant and left alone.
inline int fill_decode(CacheBook& book, int n, int bucket, const int64_t* rids, const int* tokens, int vocab,
                       int32_t* dst, const int64_t* starts, int64_t* max_kv_out) {
    const int S = book.page_size(), MB = book.max_blocks(), G = book.num_groups();
    int32_t* token_ids = dst + starts[0];
    int32_t* positions = dst + starts[1];
    int32_t* offsets = dst + starts[4];
    int32_t* slots = dst + starts[5];
    int64_t max_pos = 0;
    std::vector<RequestCache*> rcs(n);
    for (int i = 0; i < n; ++i) {
        rcs[i] = book.need(rids[i]);
        if (!rcs[i]) return ERR_UNKNOWN_REQUEST;
        if (vocab >= 0 && (tokens[i] < 0 || tokens[i] >= vocab))
            return fail(ERR_VALUE, "entry " + std::to_string(i) + ": token id outside [0, " + std::to_string(vocab) + ")");
        token_ids[i] = tokens[i];
        positions[i] = offsets[i] = (int32_t)rcs[i]->length;
        slots[i] = rcs[i]->slot;
        max_pos = std::max(max_pos, rcs[i]->length);
    }
    for (int i = n; i < bucket; ++i) token_ids[i] = positions[i] = offsets[i] = slots[i] = 0;
    const int cols = (int)std::min<int64_t>(MB, max_pos / S + 1);
    for (int g = 0; g < G; ++g) {
        int32_t* bt = dst + starts[9 + 2 * g];
        int32_t* sm = dst + starts[10 + 2 * g];
        const int32_t* mirror = book.group(g).mirror.data();
        for (int i = 0; i < n; ++i) {
            const int32_t* src = mirror + (size_t)rcs[i]->slot * MB;
            std::memcpy(bt + (size_t)i * MB, src, sizeof(int32_t) * cols);
            const int64_t pos = rcs[i]->length;
            const int page = src[pos / S];
            if (page < 0)
                return fail(ERR_VALUE, "entry " + std::to_string(i) + ": the new position has no page (reserve first)");
            sm[i] = (int32_t)(page * S + pos % S);
        }
        for (int i = n; i < bucket; ++i) {
            sm[i] = -1;
            std::memset(bt + (size_t)i * MB, 0, sizeof(int32_t) * cols);
        }
    }
    *max_kv_out = max_pos + 1;
    return OK;
}

}  // namespace vxh
