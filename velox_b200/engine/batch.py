"""One step's batch and the device-side description that kernels read.

A step is a list of `StepEntry`: a request, its next tokens (a portion of its
prompt, or one decoded token), and the places among them whose logits are
wanted.  The reference's counterpart is `BatchStep`/`SeqSlice`
(src/paged/qwen3.rs:245-269), which rebuilds and uploads block tables and
offsets inside every layer (src/paged/qwen3.rs:584-627); here the description is
built once per step on the host, sent in one copy, and shared by all layers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = ()  # indices into `tokens`


@dataclass
class GroupContext:
    block_table: torch.Tensor   # int32 [requests, max_blocks]; -1 where no page is held
    slot_mapping: torch.Tensor  # int32 [tokens]: page * page_size + offset of each new position


@dataclass
class StepContext:
    n_tokens: int
    n_seqs: int
    token_ids: torch.Tensor      # int32 [tokens]
    positions: torch.Tensor      # int32 [tokens], absolute position in its request
    seq_of_token: torch.Tensor   # int32 [tokens], row of the request in this batch
    cu_seqlens: torch.Tensor     # int32 [requests + 1], first token row of each request
    kv_offsets: torch.Tensor     # int32 [requests], positions already cached before the step
    state_slots: torch.Tensor    # int32 [requests], the request's state slot
    wanted_rows: torch.Tensor    # int32 [wanted], token rows whose logits are asked for
    groups: List[GroupContext]
    # host copies for decisions that need no device round trip
    new_lens: List[int] = field(default_factory=list)
    offsets: List[int] = field(default_factory=list)
    slots: List[int] = field(default_factory=list)
    max_new: int = 0
    max_kv: int = 0

    @property
    def decode_only(self) -> bool:
        return self.max_new == 1


def build_step_arrays(entries: Sequence[StepEntry], cache, vocab_size: Optional[int] = None):
    """Host arrays of a step (numpy int32), after the cache has reserved the
    pages: a dict of named arrays and the list of per-group (block_table, slot_mapping)."""
    S, MB = cache.page_size, cache.max_blocks
    n = len(entries)
    lens = [len(e.tokens) for e in entries]
    total = sum(lens)
    token_ids = np.empty(total, np.int32)
    positions = np.empty(total, np.int32)
    seq_of_token = np.empty(total, np.int32)
    cu = np.zeros(n + 1, np.int32)
    offsets = np.empty(n, np.int32)
    slots = np.empty(n, np.int32)
    wanted: List[int] = []
    groups = [(np.full((n, MB), -1, np.int32), np.empty(total, np.int32)) for _ in cache.groups]
    row = 0
    for i, e in enumerate(entries):
        rc = cache.requests[e.request_id]
        k = lens[i]
        toks = np.asarray(e.tokens, dtype=np.int64)
        if vocab_size is not None and k and (toks.min() < 0 or toks.max() >= vocab_size):
            raise ValueError("request %r: token id outside [0, %d)" % (e.request_id, vocab_size))
        token_ids[row:row + k] = toks
        pos = np.arange(rc.length, rc.length + k, dtype=np.int32)
        positions[row:row + k] = pos
        seq_of_token[row:row + k] = i
        cu[i + 1] = row + k
        offsets[i] = rc.length
        slots[i] = rc.slot
        for w in e.want:
            if not 0 <= w < k:
                raise ValueError("request %r: wanted place %r is not among its %d tokens" % (e.request_id, w, k))
            wanted.append(row + int(w))
        for (bt, sm), table in zip(groups, rc.tables):
            if len(table) * S < rc.length + k:
                raise ValueError("request %r: block table too short (%d pages for %d positions)"
                                 % (e.request_id, len(table), rc.length + k))
            bt[i, :len(table)] = table
            pages = np.asarray(table, np.int32)[pos // S]
            if k and pages.min() < 0:
                raise ValueError("request %r: a new position falls into a page that was given back" % (e.request_id,))
            sm[row:row + k] = pages * S + pos % S
        row += k
    arrays = dict(token_ids=token_ids, positions=positions, seq_of_token=seq_of_token, cu_seqlens=cu,
                  kv_offsets=offsets, state_slots=slots, wanted_rows=np.asarray(wanted, np.int32))
    return arrays, groups, lens


def build_step_context(entries: Sequence[StepEntry], cache, device, vocab_size: Optional[int] = None) -> StepContext:
    """Packs the step's description into one pinned buffer and copies it once."""
    arrays, groups, lens = build_step_arrays(entries, cache, vocab_size)
    parts = list(arrays.values())
    for bt, sm in groups:
        parts += [bt.reshape(-1), sm]
    sizes = [p.size for p in parts]
    # every section starts on a 16-byte boundary
    starts, cur = [], 0
    for s in sizes:
        starts.append(cur)
        cur += (s + 3) // 4 * 4
    host = torch.empty(max(cur, 4), dtype=torch.int32, pin_memory=(torch.device(device).type == "cuda"))
    hv = host.numpy()
    for p, st, s in zip(parts, starts, sizes):
        hv[st:st + s] = p
    dev = host.to(device, non_blocking=True)
    views = [dev[st:st + s] for st, s in zip(starts, sizes)]
    named = dict(zip(arrays.keys(), views[:len(arrays)]))
    gviews = views[len(arrays):]
    n, MB = len(entries), cache.max_blocks
    gctx = [GroupContext(gviews[2 * i].view(n, MB), gviews[2 * i + 1]) for i in range(len(groups))]
    offs = [int(x) for x in arrays["kv_offsets"]]
    return StepContext(
        n_tokens=int(sum(lens)), n_seqs=n, groups=gctx, new_lens=lens, offsets=offs,
        slots=[int(x) for x in arrays["state_slots"]], max_new=max(lens) if lens else 0,
        max_kv=max((o + l for o, l in zip(offs, lens)), default=0), **named)
