"""One step's batch and the device-side description that kernels read.

A step is a list of `StepEntry`: a request, its next tokens (a portion of its
prompt, or one decoded token), and the places among them whose logits are
wanted.  The reference's counterpart is `BatchStep`/`SeqSlice`
(src/paged/qwen3.rs:245-269), which rebuilds and uploads block tables and
offsets inside every layer (src/paged/qwen3.rs:584-627); here the description is
built once per step on the host (by the host library, `csrc/host/step_builder.hpp`,
straight from the cache manager's books), sent in one copy, and shared by all
layers.
"""
from __future__ import annotations

import ctypes
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
    single_rows: torch.Tensor    # int32 [tokens]: token rows of the requests that bring few tokens (first n_single)
    portion_seqs: torch.Tensor   # int32 [requests]: the requests that bring more than one (first n_portions)
    groups: List[GroupContext]
    # host copies for decisions that need no device round trip
    new_lens: List[int] = field(default_factory=list)
    offsets: List[int] = field(default_factory=list)
    slots: List[int] = field(default_factory=list)
    max_new: int = 0
    max_kv: int = 0
    n_single: int = 0        # token rows of the requests that bring at most `short_max` tokens (1: decoded tokens)
    max_kv_single: int = 0   # most keys of any of those requests after the step
    n_portions: int = 0      # requests that bring more
    max_short: int = 0       # the longest of the short requests (1: every row of `single_rows` is its request's only one)

    @property
    def decode_only(self) -> bool:
        return self.max_new == 1


SECTION_NAMES = ["token_ids", "positions", "seq_of_token", "cu_seqlens", "kv_offsets", "state_slots", "wanted_rows",
                 "single_rows", "portion_seqs"]


def _sections(n: int, total: int, wanted: int, n_groups: int, max_blocks: int):
    """Sizes and starts (in 32-bit words, every section on a 16-byte boundary) of the
    sections of a step's description, in the host library's order."""
    sizes = [total, total, total, n + 1, n, n, wanted, total, n]
    for _ in range(n_groups):
        sizes += [n * max_blocks, total]
    starts, cur = [], 0
    for s in sizes:
        starts.append(cur)
        cur += (s + 3) // 4 * 4
    return sizes, starts, cur


def build_step_arrays(entries: Sequence[StepEntry], cache, vocab_size: Optional[int] = None, out=None,
                      short_max: int = 1):
    """The step's description after the cache has reserved the pages, written by the
    host library into `out` (a writable int32 numpy array, made if not given).
    Returns (out, sizes, starts, summary) with summary = (tokens, wanted rows,
    longest portion, most keys of any request after the step, token rows of the
    requests that bring at most `short_max` tokens, most keys among those requests,
    requests that bring more, the longest short request)."""
    from .. import native

    n = len(entries)
    lens = [len(e.tokens) for e in entries]
    total, wanted = sum(lens), sum(len(e.want) for e in entries)
    sizes, starts, words = _sections(n, total, wanted, len(cache.groups), cache.max_blocks)
    if out is None:
        out = np.empty(max(words, 4), np.int32)
    try:
        rids = cache.handles(e.request_id for e in entries)
    except KeyError as e:
        raise KeyError("request %r holds no cache; add it first" % (e.args[0],))
    tokens = np.fromiter((t for e in entries for t in e.tokens), np.int64, total)
    if vocab_size is not None and total and (tokens.min() < 0 or tokens.max() >= vocab_size):
        bad = next(e.request_id for e in entries if any(not 0 <= int(t) < vocab_size for t in e.tokens))
        raise ValueError("request %r: token id outside [0, %d)" % (bad, vocab_size))
    tokens = tokens.astype(np.int32)
    for e, k in zip(entries, lens):
        for w in e.want:
            if not 0 <= w < k:
                raise ValueError("request %r: wanted place %r is not among its %d tokens" % (e.request_id, w, k))
    summary = (ctypes.c_int64 * 8)()
    native.check(cache._lib.vxh_build_step(
        cache._book, n, rids, native.int_array(lens), tokens.ctypes.data_as(ctypes.POINTER(ctypes.c_int)),
        native.int_array(len(e.want) for e in entries), native.int_array(w for e in entries for w in e.want),
        -1 if vocab_size is None else int(vocab_size), int(short_max), out.ctypes.data_as(ctypes.c_void_p),
        native.int64_array(starts), summary))
    return out, sizes, starts, [int(x) for x in summary]


def build_step_context(entries: Sequence[StepEntry], cache, device, vocab_size: Optional[int] = None,
                       short_max: int = 1) -> StepContext:
    """Has the step's description written into one pinned buffer and copies it once."""
    n = len(entries)
    lens = [len(e.tokens) for e in entries]
    _, _, words = _sections(n, sum(lens), sum(len(e.want) for e in entries), len(cache.groups), cache.max_blocks)
    host = torch.empty(max(words, 4), dtype=torch.int32, pin_memory=(torch.device(device).type == "cuda"))
    hv, sizes, starts, summary = build_step_arrays(entries, cache, vocab_size, out=host.numpy(), short_max=short_max)
    dev = host.to(device, non_blocking=True)
    views = [dev[st:st + s] for st, s in zip(starts, sizes)]
    named = dict(zip(SECTION_NAMES, views[:len(SECTION_NAMES)]))
    gviews = views[len(SECTION_NAMES):]
    MB = cache.max_blocks
    gctx = [GroupContext(gviews[2 * i].view(n, MB), gviews[2 * i + 1]) for i in range(len(cache.groups))]
    offs = [int(x) for x in hv[starts[4]:starts[4] + n]]
    return StepContext(
        n_tokens=summary[0], n_seqs=n, groups=gctx, new_lens=lens, offsets=offs,
        slots=[int(x) for x in hv[starts[5]:starts[5] + n]], max_new=summary[2], max_kv=summary[3],
        n_single=summary[4], max_kv_single=summary[5], n_portions=summary[6], max_short=summary[7], **named)
