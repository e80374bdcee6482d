"""Continuous batching above the step function: admit, cut prompts into portions
under a token budget, decode, finish and free.

What is kept of the reference's `BatchScheduler` (src/paged/scheduler.rs:75-535):
first come first served from a queue (:220-295), at most `max_running_requests`
holding cache (:239), requests in a step ordered by id (:311-312), one new token
per decoding request per step (:337-343), the first token sampled from the step
that completes the prompt (:407-421), an end-of-sequence token kept and counted
(:426), finish reasons "stop" and "length" (:465-484), and its counters (:95-105).

What differs, on purpose:
  * Prompts are really cut.  The reference offers a request's whole remaining
    prompt or defers it (src/paged/scheduler.rs:322-330), so one long prompt
    still runs whole.  Here decoding requests go first (one token each), then
    the budget `max_batch_tokens` is filled with portions of prompts in arrival
    order, each at most `chunk_size` if that is set.
  * Pages are taken step by step, not for prompt + max_tokens at admission
    (src/paged/scheduler.rs:255).  So they can run out in mid-flight: then the
    running request that was admitted last is preempted: its pages and slot
    are given back, its tokens are kept, and it returns to the FRONT of the
    queue to be recomputed (prompt and generated tokens as one prompt).  A
    request that is alone and still cannot grow ends with reason "length".
  * A request that could never fit (longer than the pool or than
    `max_model_len`) is refused at submit; the reference would queue it forever
    (src/paged/scheduler.rs:284-292).

The scheduler decides and keeps books; it runs nothing on the device.  `plan()`
reserves the pages of the step it returns; `update()` takes the sampled tokens.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams
from .batch import StepEntry

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Request:
    request_id: int
    prompt: List[int]
    params: SamplingParams
    generated: List[int] = field(default_factory=list)
    status: str = WAITING
    finish_reason: Optional[str] = None
    admitted_at: int = -1  # admission counter: the latest is preempted first
    preemptions: int = 0

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.generated

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.generated)

    def token_slice(self, start: int, stop: int) -> List[int]:
        """tokens[start:stop] without building the whole list."""
        n = len(self.prompt)
        if stop <= n:
            return self.prompt[start:stop]
        if start >= n:
            return self.generated[start - n:stop - n]
        return self.prompt[start:] + self.generated[:stop - n]


@dataclass
class SchedulerStats:
    steps: int = 0
    tokens_generated: int = 0
    prompt_tokens: int = 0
    requests_completed: int = 0
    requests_refused: int = 0
    preemptions: int = 0
    last_batch_size: int = 0
    last_batch_tokens: int = 0


class RequestRefused(ValueError):
    pass


class Scheduler:
    def __init__(self, cache: CacheManager, max_running_requests: int = 64, max_batch_tokens: int = 2048,
                 chunk_size: Optional[int] = None, max_model_len: Optional[int] = None):
        self.cache = cache
        self.max_running_requests = int(max_running_requests)
        self.max_batch_tokens = int(max_batch_tokens)
        self.chunk_size = chunk_size
        limit = cache.max_blocks * cache.page_size
        self.max_model_len = min(int(max_model_len), limit) if max_model_len else limit
        self.waiting: Deque[Request] = deque()
        self.running: Dict[int, Request] = {}
        self.finished: Dict[int, Request] = {}
        self.stats = SchedulerStats()
        self._next_id = 0
        self._admissions = 0

    # -- submit ---------------------------------------------------------------
    def submit(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        params = params or SamplingParams()
        prompt = [int(t) for t in prompt]
        if not prompt:  # the reference rejects an empty prompt too (src/paged/scheduler.rs:165-167)
            self.stats.requests_refused += 1
            raise RequestRefused("empty prompt")
        total = len(prompt) + params.max_tokens
        if total > self.max_model_len:
            self.stats.requests_refused += 1
            raise RequestRefused("prompt (%d) + max_tokens (%d) exceeds the longest sequence %d"
                                 % (len(prompt), params.max_tokens, self.max_model_len))
        pages = -(-total // self.cache.page_size)
        for g in self.cache.groups:
            need = pages if g.window <= 0 else min(pages, -(-(g.window + min(self._portion_cap(), total))
                                                           // self.cache.page_size) + 1)
            if need > g.allocator.num_pages:
                self.stats.requests_refused += 1
                raise RequestRefused("the request needs %d pages of a pool of %d and could never run"
                                     % (need, g.allocator.num_pages))
        rid = self._next_id
        self._next_id += 1
        self.waiting.append(Request(rid, prompt, params))
        return rid

    def _portion_cap(self) -> int:
        return min(self.max_batch_tokens, self.chunk_size) if self.chunk_size else self.max_batch_tokens

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # -- one step's plan ------------------------------------------------------
    def _remaining(self, r: Request) -> int:
        return len(r.prompt) + len(r.generated) - self.cache.length(r.request_id)

    def _preempt(self, victim: Request) -> None:
        self.cache.release(victim.request_id)
        del self.running[victim.request_id]
        victim.status = WAITING
        victim.preemptions += 1
        self.stats.preemptions += 1
        self.waiting.appendleft(victim)

    def _finish(self, r: Request, reason: str) -> None:
        if self.cache.has_request(r.request_id):
            self.cache.release(r.request_id)
        self.running.pop(r.request_id, None)
        r.status, r.finish_reason = FINISHED, reason
        self.finished[r.request_id] = r
        self.stats.requests_completed += 1

    def plan(self) -> Tuple[List[StepEntry], List[Request]]:
        """The next step: its entries (pages already reserved) and the requests
        that were ended while planning (alone and out of pages)."""
        ended: List[Request] = []
        while True:
            entries = self._plan_once(ended)
            if entries or not self.running:
                return entries, ended
            # Requests hold cache but none can move (every one waits for pages
            # the others hold): the one admitted last makes room.
            victim = max(self.running.values(), key=lambda q: q.admitted_at)
            if len(self.running) == 1:
                self._finish(victim, "length")
                ended.append(victim)
            else:
                self._preempt(victim)

    def _plan_once(self, ended: List[Request]) -> List[StepEntry]:
        budget = self.max_batch_tokens
        chosen: Dict[int, int] = {}
        preempted = False

        # 1. requests that decode: one token each, oldest id first
        for rid in sorted(self.running):
            r = self.running.get(rid)
            if r is None or self._remaining(r) != 1 or not r.generated:
                continue
            if budget <= 0:
                break
            while not self.cache.reserve(rid, 1):
                victim = max(self.running.values(), key=lambda q: q.admitted_at)
                if victim is r and len(self.running) == 1:
                    self._finish(r, "length")
                    ended.append(r)
                    break
                chosen.pop(victim.request_id, None)
                self._preempt(victim)
                preempted = True
                if victim is r:
                    break
            else:
                chosen[rid] = 1
                budget -= 1

        # 2. prompts under way (and recomputations), oldest id first
        for rid in sorted(self.running):
            r = self.running[rid]
            if rid in chosen or budget <= 0:
                continue
            rem = self._remaining(r)
            if rem == 1 and r.generated and rid not in chosen:
                continue  # a decode that found no budget
            k = min(rem, budget, self._portion_cap())
            k = self._fit(rid, k)
            if k > 0:
                chosen[rid] = k
                budget -= k

        # 3. admissions, first come first served; none in a step that had to
        # preempt (the pages just freed are for those that stayed)
        while (not preempted and self.waiting and budget > 0
               and len(self.running) < self.max_running_requests):
            r = self.waiting[0]
            if self.cache.add_request(r.request_id) is None:
                break
            k = self._fit(r.request_id, min(r.num_tokens, budget, self._portion_cap()))
            if k <= 0:
                self.cache.release(r.request_id)
                if not self.running:  # nothing will ever free a page for it
                    self.waiting.popleft()
                    self._finish(r, "length")
                    ended.append(r)
                    continue
                break  # head of the line waits; nobody overtakes it
            self.waiting.popleft()
            r.status = RUNNING
            r.admitted_at = self._admissions
            self._admissions += 1
            self.running[r.request_id] = r
            chosen[r.request_id] = k
            budget -= k

        entries: List[StepEntry] = []
        for rid in sorted(chosen):
            r = self.running[rid]
            done = self.cache.length(rid)
            toks = r.token_slice(done, done + chosen[rid])
            last = done + chosen[rid] == r.num_tokens
            entries.append(StepEntry(rid, toks, [len(toks) - 1] if last else []))
        return entries

    def _fit(self, rid: int, k: int) -> int:
        """The largest portion <= k whose pages can be reserved now (reserves it)."""
        while k > 0:
            if self.cache.reserve(rid, k):
                return k
            # fewer pages: shrink to what the scarcest group can still hold
            rc = self.cache.requests[rid]
            room = min((len(t) + g.allocator.num_free) * self.cache.page_size - rc.length
                       for t, g in zip(rc.tables, self.cache.groups))
            k = min(k - 1, room)
        return 0

    # -- after the step -------------------------------------------------------
    def update(self, entries: Sequence[StepEntry], sampled: Sequence[int]) -> List[Tuple[int, int, bool]]:
        """Takes the tokens sampled for the entries that wanted one (in order).
        Returns (request id, token, finished) for each."""
        out: List[Tuple[int, int, bool]] = []
        it = iter(sampled)
        self.stats.steps += 1
        self.stats.last_batch_size = len(entries)
        self.stats.last_batch_tokens = sum(len(e.tokens) for e in entries)
        for e in entries:
            r = self.running[e.request_id]
            if not e.want:
                self.stats.prompt_tokens += len(e.tokens)
                continue
            tok = int(next(it))
            if len(e.tokens) > 1 or not r.generated:
                self.stats.prompt_tokens += len(e.tokens)
            r.generated.append(tok)
            self.stats.tokens_generated += 1
            p = r.params
            reason = None
            if not p.ignore_eos and (tok in p.eos_token_ids or tok in p.stop_token_ids):
                reason = "stop"
            elif len(r.generated) >= p.max_tokens:
                reason = "length"
            elif len(r.prompt) + len(r.generated) >= self.max_model_len:
                reason = "length"
            if reason:
                self._finish(r, reason)
            out.append((r.request_id, tok, reason is not None))
        return out
