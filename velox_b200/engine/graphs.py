"""Decode steps as CUDA graphs.

A step in which every request brings exactly one token has the same shape of
work every time, so its ~400 kernel launches are captured once per (batch size,
key-range bucket) and replayed: the host fills one pinned buffer with the step's
description (token ids, positions, block tables, slot mapping, sampling
parameters), copies it into the graph's fixed device buffer, and launches the
graph; embedding, all layers, the head and the sampling kernel run from there.

Small mixed steps (a short prompt portion beside decoded tokens, as a fixed chunk size
and continuous batching produce them) are bound by the host, not the device: some ten
launches a layer from Python take longer than their kernels run.  A step whose shape
(tokens, requests, wanted rows, how many rows go to which attention kernel, longest
portion, key-range buckets) has come up a few times is therefore captured too, at its
exact shape, and replayed when that shape comes again (`MIXED_*` below).

Padding: a batch is padded up to its bucket with rows that read page 0 at
position 0 and write nothing (slot -1); their tokens are dropped.  Models with
per-request state are never padded (a padded row would touch a real slot) and
capture a graph in the step that first needs it (that step runs eagerly, once), and
models with a part that is not marked `cuda_graph_safe` (it reads host-side
fields of the step) do not use graphs at all.
"""
from __future__ import annotations

import ctypes
import gc
import os
import weakref
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import native
from ..csrc import ops
from .batch import SECTION_NAMES, GroupContext, StepContext, StepEntry, _sections, build_step_arrays

SPLIT_KEYS = ops.DECODE_CHUNK_TILES * 16


def batch_bucket(n: int, exact: bool, cap: int) -> int:
    if exact or n <= 8:
        return n
    return min(cap, -(-n // 8) * 8) if cap >= n else n


def keys_bucket(max_kv: int) -> int:
    """Key-range bucket: the next power of two of the number of 256-key pieces."""
    pieces = max(1, -(-max_kv // SPLIT_KEYS))
    b = 1
    while b < pieces:
        b *= 2
    return b * SPLIT_KEYS


def all_buckets(max_batch: int, cap: int, max_kv: int) -> List[Tuple[int, int]]:
    """Every (batch bucket, key-range bucket) that a padded decode step of 1 to
    `max_batch` requests (at most `cap`, the number of slots) with up to `max_kv` keys
    can ask for."""
    batches = sorted({batch_bucket(n, False, cap) for n in range(1, min(max_batch, cap) + 1)})
    keys, k = [], SPLIT_KEYS
    while True:
        keys.append(k)
        if k >= keys_bucket(max_kv):
            break
        k *= 2
    return [(b, kv) for b in batches for kv in keys]


class _Graph:
    def __init__(self, runner, bucket: int, max_kv: int):
        cache, device = runner.cache, runner.device
        self.bucket, self.max_kv = bucket, max_kv
        MB, G = cache.max_blocks, len(cache.groups)
        B = bucket
        names, F = SECTION_NAMES, len(SECTION_NAMES)
        sizes = [B, B, B, B + 1, B, B, B, B, B]
        for _ in range(G):
            sizes += [B * MB, B]
        sizes += [B, B, B]  # temperature, top_p, uniform (float32 bit patterns)
        self.starts, cur = [], 0
        for s in sizes:
            self.starts.append(cur)
            cur += (s + 3) // 4 * 4
        self.sizes = sizes
        self.host = torch.zeros(cur, dtype=torch.int32, pin_memory=True)
        self.hv = self.host.numpy()
        self.host_ptr = ctypes.c_void_p(self.host.data_ptr())
        self.starts_c = (ctypes.c_int64 * len(self.starts))(*self.starts)
        self.dev = torch.zeros(cur, dtype=torch.int32, device=device)
        v = [self.dev[st:st + s] for st, s in zip(self.starts, sizes)]
        hvv = [self.hv[st:st + s] for st, s in zip(self.starts, sizes)]
        self.h = dict(zip(names, hvv[:F]))
        self.h_groups = [(hvv[F + 2 * g].reshape(B, MB), hvv[F + 1 + 2 * g]) for g in range(G)]
        self.h_temp, self.h_top_p, self.h_uniform = (x.view(np.float32) for x in hvv[F + 2 * G:])
        groups = [GroupContext(v[F + 2 * g].view(B, MB), v[F + 1 + 2 * g]) for g in range(G)]
        f = [x.view(torch.float32) for x in v[F + 2 * G:]]
        self.d_temp, self.d_top_p, self.d_uniform = f
        self.ctx = StepContext(n_tokens=B, n_seqs=B, groups=groups, new_lens=[1] * B, offsets=[0] * B,
                               slots=[0] * B, max_new=1, max_kv=max_kv, n_single=B, max_kv_single=max_kv,
                               n_portions=0, max_short=1, **dict(zip(names, v[:F])))
        # constant sections
        self.h["seq_of_token"][:] = np.arange(B)
        self.h["cu_seqlens"][:] = np.arange(B + 1)
        self.h["wanted_rows"][:] = np.arange(B)
        self.h["single_rows"][:] = np.arange(B)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits = self.ids = None
        self.launches = 0
        self.bounded_wait_launches = 0  # of those, kernels whose waits are bounded
        self.copied: Optional[torch.cuda.Event] = None  # the last copy out of the pinned buffer

    def fill(self, entries: Sequence[StepEntry], rids, cache, sampling, vocab_size: int = -1) -> None:
        if self.copied is not None:
            self.copied.synchronize()  # the pinned buffer is free once its last copy has run
        n = len(entries)
        max_kv = ctypes.c_int64(0)
        native.check(cache._lib.vxh_fill_decode(
            cache._book, n, self.bucket, rids,
            native.int_array(int(e.tokens[0]) for e in entries), int(vocab_size), self.host_ptr, self.starts_c,
            ctypes.byref(max_kv)))
        if sampling is None:
            self.h_temp[:] = 0.0
        else:
            temps, tops, us = sampling
            self.h_temp[:n], self.h_top_p[:n], self.h_uniform[:n] = temps, tops, us
            self.h_temp[n:] = 0.0
        self.dev.copy_(self.host, non_blocking=True)
        if self.copied is None:
            self.copied = torch.cuda.Event()
        self.copied.record()

    def run_model(self, runner) -> None:
        residual, delta = runner.model.forward_hidden(self.ctx, runner.cache)
        self.logits = runner.model.logits(residual, delta, self.ctx.wanted_rows)
        self.ids = ops.sample(self.logits, self.d_temp, self.d_top_p, self.d_uniform)


# Larger steps keep the device busy longer than the host needs to launch them, and recording a graph costs tens of
# milliseconds: with 256 here a stream under a budget of 256 tokens a step recorded its 64 graphs and lost a quarter
# of its throughput (Qwen3-14B shape 1,282 against 1,793 tokens a second; with 96 1,781).
# VELOX_B200_MIXED_GRAPH_TOKENS sets it; 0: never.
MIXED_MAX_TOKENS = int(os.environ.get("VELOX_B200_MIXED_GRAPH_TOKENS", "96"))
MIXED_SEEN_BEFORE = 2    # a shape is captured when it comes up for the third time
MIXED_MAX_GRAPHS = 64    # (each holds its activations: tens of MB at the real widths)


class _MixedGraph:
    """A captured step of one exact shape.  Its description lives in a fixed device buffer
    that every replay fills; sampling stays outside (it takes host-made parameters)."""

    def __init__(self, runner, sig):
        cache, device = runner.cache, runner.device
        (total, n, wanted, n_single, n_portions, max_new, max_short, max_kv, max_kv_single) = sig
        self.sig = sig
        MB, G = cache.max_blocks, len(cache.groups)
        self.sizes, self.starts, words = _sections(n, total, wanted, G, MB)
        self.host = torch.zeros(max(words, 4), dtype=torch.int32, pin_memory=True)
        self.dev = torch.zeros(max(words, 4), dtype=torch.int32, device=device)
        v = [self.dev[st:st + sz] for st, sz in zip(self.starts, self.sizes)]
        F = len(SECTION_NAMES)
        groups = [GroupContext(v[F + 2 * g].view(n, MB), v[F + 1 + 2 * g]) for g in range(G)]
        # (the host-side lists are left empty: parts that read them are not graph-safe and never get here)
        self.ctx = StepContext(n_tokens=total, n_seqs=n, groups=groups, max_new=max_new, max_kv=max_kv,
                               n_single=n_single, max_kv_single=max_kv_single, n_portions=n_portions,
                               max_short=max_short, **dict(zip(SECTION_NAMES, v[:F])))
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits = self.ids = None
        self.launches = self.bounded_wait_launches = 0
        self.copied: Optional[torch.cuda.Event] = None

    def fill(self, entries, cache, vocab_size, short_max) -> List[int]:
        if self.copied is not None:
            self.copied.synchronize()
        _, _, _, summary = build_step_arrays(entries, cache, vocab_size, out=self.host.numpy(), short_max=short_max)
        self.dev.copy_(self.host, non_blocking=True)
        if self.copied is None:
            self.copied = torch.cuda.Event()
        self.copied.record()
        return summary

    def run_model(self, runner) -> None:
        self.logits = runner.run(self.ctx)
        if self.logits is None:   # (nothing wanted: the capture still needs a tensor to hand around)
            self.logits = torch.empty((0, runner.vocab_size), dtype=torch.float32, device=runner.device)
        self.ids = self.logits   # (no sampling inside; `_capture` copies both)


class DecodeGraphs:
    def __init__(self, runner):
        self.runner = weakref.proxy(runner)  # (the runner holds these graphs: no cycle, they end with it)
        self.graphs: Dict[Tuple[int, int], _Graph] = {}
        self.pool = None
        cache = runner.cache
        self.has_state = bool(cache._state_layers)
        self.usable = all(getattr(p, "cuda_graph_safe", False) for p in runner.model.parts())
        self.cap = cache.slots.num_slots
        self._collected = False
        self.mixed: Dict[Tuple, _MixedGraph] = {}
        self._mixed_seen: Dict[Tuple, int] = {}

    def capture_all(self, max_batch: int, max_kv: int) -> int:
        """Captures, ahead of the first request, the graph of every (batch bucket,
        key-range bucket) that decode steps of up to `max_batch` requests with up to
        `max_kv` keys can ask for, so that no step has to wait for a capture (some
        tens of milliseconds each).  The captured steps run on padding rows only.
        Returns how many graphs were captured.  Nothing is captured for a model
        with per-request state (its steps are never padded)."""
        if not self.usable or self.has_state:
            return 0
        cache = self.runner.cache
        done = 0
        for b, kv in all_buckets(max_batch, self.cap, max_kv):
            if (b, kv) in self.graphs:
                continue
            g = self.graphs[(b, kv)] = _Graph(self.runner, b, kv)
            g.fill([], cache.handles([]), cache, None, self.runner.vocab_size)
            self._capture(g)
            done += 1
        return done

    def eligible(self, entries: Sequence[StepEntry]) -> bool:
        return self.usable and len(entries) > 0 and all(len(e.tokens) == 1 for e in entries)

    def step(self, entries: Sequence[StepEntry], rids, sampling=None):
        """Runs a decode-only step (`rids`: the entries' ids in the host library, a C
        array).  Returns (logits [bucket, vocab], ids [bucket]): the first
        len(entries) rows are the entries'."""
        cache = self.runner.cache
        n = len(entries)
        max_kv = int(native.check(cache._lib.vxh_cache_max_length(cache._book, n, rids))) + 1
        key = (batch_bucket(n, self.has_state, self.cap), keys_bucket(max_kv))
        g = self.graphs.get(key)
        if g is None:
            g = self.graphs[key] = _Graph(self.runner, *key)
        g.fill(entries, rids, cache, sampling, self.runner.vocab_size)
        if g.graph is None:
            # The capture runs the step once, eagerly, on this step's real rows (a recording
            # runs nothing).  That run IS this step: its results are handed out and the graph
            # is replayed from the next step on.  Replaying it now as well would only write
            # the same keys and values again, but it would advance a mixer's per-request
            # state a second time.
            self._capture(g)
            return g.logits, g.ids
        g.graph.replay()
        ops.add_launches(g.launches)
        if g.bounded_wait_launches:
            ops.note_bounded_wait(g.bounded_wait_launches)
        return g.logits, g.ids

    # -- small mixed steps ---------------------------------------------------------
    def mixed_signature(self, entries: Sequence[StepEntry], rids, short_max: int) -> Optional[Tuple]:
        """The shape of a step that is no pure decode step, if it is small enough to be worth a graph
        (else None): everything a part's choice of kernels and their grids may depend on."""
        if not self.usable or self.has_state:
            return None
        lens = [len(e.tokens) for e in entries]
        total = sum(lens)
        if total > MIXED_MAX_TOKENS or not entries:
            return None
        cache, n = self.runner.cache, len(entries)
        short = [i for i, k in enumerate(lens) if k <= short_max]
        max_new = max(lens)
        longest = int(native.check(cache._lib.vxh_cache_max_length(cache._book, n, rids)))
        max_kv = keys_bucket(longest + max_new)
        max_kv_single = 0
        if short:
            sub = native.int64_array(rids[i] for i in short)
            max_kv_single = keys_bucket(int(native.check(cache._lib.vxh_cache_max_length(cache._book, len(short), sub)))
                                        + max(lens[i] for i in short))
        return (total, n, sum(len(e.want) for e in entries), sum(lens[i] for i in short), n - len(short), max_new,
                max(lens[i] for i in short) if short else 0, max_kv, max_kv_single)

    def mixed_step(self, sig: Tuple, entries: Sequence[StepEntry], short_max: int):
        """Runs a step of shape `sig` from its graph if it has one; captures one if the shape has come up
        often enough; returns the logits at the wanted rows, or NotImplemented for the eager path."""
        g = self.mixed.get(sig)
        if g is None:
            seen = self._mixed_seen.get(sig, 0)
            if seen < MIXED_SEEN_BEFORE or len(self.mixed) >= MIXED_MAX_GRAPHS:
                self._mixed_seen[sig] = seen + 1
                return NotImplemented
            g = self.mixed[sig] = _MixedGraph(self.runner, sig)
        g.fill(entries, self.runner.cache, self.runner.vocab_size, short_max)
        if g.graph is None:
            self._capture(g)   # (its eager run is this step)
        else:
            g.graph.replay()
            ops.add_launches(g.launches)
            if g.bounded_wait_launches:
                ops.note_bounded_wait(g.bounded_wait_launches)
        return g.logits if sig[2] else None

    def _capture(self, g) -> None:
        # once eagerly (first-use set-up of kernels and libraries happens outside the capture) ...
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            g.run_model(self.runner)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        eager_logits, eager_ids = g.logits, g.ids
        # ... then recorded (nothing runs while recording).
        # Garbage is collected before, not during, the recording: an older engine's
        # graphs that happened to be destroyed in the middle of it would invalidate it.
        # A full collection (tens of milliseconds) is made before this engine's first
        # recording only: what was garbage before the engine's time is gone then, and
        # engines themselves are freed by their reference counts, without the collector.
        graph = torch.cuda.CUDAGraph()
        n0, b0 = ops.launch_count(), ops.bounded_wait_launches()
        if not self._collected:
            gc.collect()
            self._collected = True
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph, pool=self.pool):
                g.run_model(self.runner)
        finally:
            if gc_was_on:
                gc.enable()
        g.launches = ops.launch_count() - n0
        ops.add_launches(-g.launches)  # (recorded, not run)
        g.bounded_wait_launches = ops.bounded_wait_launches() - b0
        if self.pool is None:
            self.pool = graph.pool()
        g.graph = graph
        # the eager run's results, in the buffers that the graph's replays will fill
        g.logits.copy_(eager_logits)
        g.ids.copy_(eager_ids)
