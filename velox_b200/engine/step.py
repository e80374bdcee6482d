"""The step function: a batch of (request, its next tokens) in, logits at the
wanted places out.

It runs only the tokens it is given, as one batch, against the cache that earlier
steps left: portions of prompts beside single decoded tokens, cut anywhere.  The
reference's counterpart is `PagedQwen3::forward` under `BatchScheduler::step`
(src/paged/qwen3.rs:994-1017; src/paged/scheduler.rs:299-375), which returns the
last row of every request; here the caller names the rows, and a portion that
does not end a prompt asks for none (the reference computes and discards them,
src/paged/scheduler.rs:416-418).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import native
from ..cache.manager import CacheManager, OutOfPages
from ..csrc import ops
from .batch import StepContext, StepEntry, build_step_context


class ModelRunner:
    """Owns a model and its cache on one device and steps them."""

    def __init__(self, model, cache: CacheManager, device, vocab_size: int, cuda_graphs: bool = False):
        self.model, self.cache, self.device, self.vocab_size = model, cache, torch.device(device), int(vocab_size)
        self.steps = 0
        # requests that bring at most so many tokens are listed token by token for the mixers (a mixer
        # may then treat each token as a decoded one): the largest wish among the model's parts
        self.short_max = max([1] + [int(getattr(p, "short_rows_up_to", 1)) for p in model.parts()])
        self.graphs = None
        if cuda_graphs:
            from .graphs import DecodeGraphs
            self.graphs = DecodeGraphs(self)

    def validate(self, entries: Sequence[StepEntry]) -> None:
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise ValueError("request %r appears twice in one step" % (e.request_id,))
            seen.add(e.request_id)
            if len(e.tokens) == 0:
                raise ValueError("request %r brings no tokens" % (e.request_id,))

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs one batch.  Returns float32 logits [wanted, vocab] on the device
        in the order of the entries and of their `want`, or None if nothing is
        wanted.  Raises `OutOfPages` if the cache cannot hold the new positions:
        nothing is run or written then, and the pages that the step's earlier
        entries had taken already stay with their requests, to be used by their
        next step or given back with them."""
        logits, _ = self._step(entries, None, False)
        return logits

    def step_and_sample(self, entries: Sequence[StepEntry], temperature, top_p, uniform):
        """Runs one batch and samples a token at every wanted place (per-row
        float lists).  Returns (logits [wanted, vocab], int32 ids [wanted]) on
        the device, or (None, None)."""
        return self._step(entries, (temperature, top_p, uniform), True)

    def _step(self, entries, sampling, sample: bool):
        self.validate(entries)
        cache = self.cache
        n = len(entries)
        try:
            rids = cache.handles(e.request_id for e in entries)
            counts = native.int_array(len(e.tokens) for e in entries)
            got = native.check(cache._lib.vxh_cache_reserve_many(cache._book, n, rids, counts))
        except KeyError:
            missing = next(e.request_id for e in entries if not cache.has_request(e.request_id))
            raise KeyError("request %r holds no cache; add it first" % (missing,))
        if got < n:
            # give back nothing: pages already reserved stay with their
            # requests (they are theirs to use in a later step)
            e = entries[got]
            raise OutOfPages("no pages left for request %r (%d new tokens); free pages per group: %s"
                             % (e.request_id, len(e.tokens), cache.free_pages()))
        ids = None
        if self.graphs is not None and self.graphs.eligible(entries):
            for e in entries:
                if not 0 <= int(e.tokens[0]) < self.vocab_size:
                    raise ValueError("request %r: token id outside [0, %d)" % (e.request_id, self.vocab_size))
                if any(w != 0 for w in e.want):
                    raise ValueError("request %r: wanted place is not among its 1 tokens" % (e.request_id,))
            per_entry = None
            if sample:
                # the sampling lists have one value per wanted place; the captured step
                # samples every row (a row nobody wants is sampled greedily and dropped)
                per_entry, k = ([], [], []), 0
                for e in entries:
                    for lst, src, default in zip(per_entry, sampling, (0.0, 1.0, 0.0)):
                        lst.append(src[k] if e.want else default)
                    k += 1 if e.want else 0
            all_logits, all_ids = self.graphs.step(entries, rids, per_entry)
            rows = [i for i, e in enumerate(entries) for _ in e.want]
            if not rows:
                logits = None
            elif rows == list(range(len(entries))):
                logits, ids = all_logits[:len(rows)], all_ids[:len(rows)]
            else:
                idx = torch.tensor(rows, dtype=torch.long, device=self.device)
                logits, ids = all_logits[idx], all_ids[idx]
        else:
            logits, sig = NotImplemented, None
            if self.graphs is not None:
                sig = self.graphs.mixed_signature(entries, rids, self.short_max)
            if sig is not None:
                # a small mixed step: from its graph, if this shape has one by now (the step's
                # description is checked by the host library as it is written, as in the eager path)
                logits = self.graphs.mixed_step(sig, entries, self.short_max)
            if logits is NotImplemented:
                ctx = build_step_context(entries, self.cache, self.device, self.vocab_size, self.short_max)
                logits = self.run(ctx)
            if sample and logits is not None:
                t = torch.tensor([sampling[0], sampling[1], sampling[2]], dtype=torch.float32).to(self.device, non_blocking=True)
                ids = ops.sample(logits, t[0], t[1], t[2]) if any(x > 0 for x in sampling[0]) else ops.sample(logits)
        native.check(cache._lib.vxh_cache_commit_many(cache._book, n, rids, counts))
        self.steps += 1
        return logits, (ids if sample else None)

    @property
    def pending_error_check(self) -> bool:
        """True if a kernel whose waits are bounded has run since the error word was last
        read: a wait that ran out must not pass for a result, so whoever hands out a
        step's results calls `check_errors()` first.  Which kernels those are is the
        kernel library's knowledge (`ops.note_bounded_wait`), not the step's."""
        return ops.bounded_wait_pending()

    def check_errors(self) -> None:
        ops.check_pending_device_errors()

    def run(self, ctx: StepContext) -> Optional[torch.Tensor]:
        residual, delta = self.model.forward_hidden(ctx, self.cache)
        if ctx.wanted_rows.numel() == 0:
            return None
        return self.model.logits(residual, delta, ctx.wanted_rows)
