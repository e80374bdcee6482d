"""Continuous batching above the step function: admit, cut prompts into portions
under a token budget, decode, finish and free.

What is kept of the reference's `BatchScheduler` (src/paged/scheduler.rs:75-535):
first come first served from a queue (:220-295), at most `max_running_requests`
holding cache (:239), requests in a step ordered by id (:311-312), one new token
per decoding request per step (:337-343), the first token sampled from the step
that completes the prompt (:407-421), an end-of-sequence token kept and counted
(:426), finish reasons "stop", "length" and "cancelled" (:440-452, :465-484), and
its counters with the last step's wall time (:95-105, :528-532).

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

The decisions are made by the host library (`csrc/host/scheduler.hpp`), next to
the cache manager's books that they read and change.  This module is its Python
face: it keeps what only Python needs (the sampling parameters of a request) and
shows requests and queues as views that ask the library when they are read.
"""
from __future__ import annotations

import ctypes
import weakref
from dataclasses import dataclass
from typing import Dict, Iterator, List, Mapping, Optional, Sequence, Tuple

from .. import native
from ..cache.manager import CacheManager
from ..native import RequestRefused  # noqa: F401  (part of this module's interface)
from ..sampling.params import SamplingParams
from .batch import StepEntry

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
_STATUS = (WAITING, RUNNING, FINISHED)
_REASON = (None, "stop", "length", "cancelled")


class Request:
    """A request as the library holds it; every attribute is read there."""

    def __init__(self, scheduler: "Scheduler", request_id: int):
        self._s, self.request_id = scheduler, int(request_id)

    def _info(self) -> List[int]:
        info = (ctypes.c_int64 * 8)()
        native.check(self._s._lib.vxh_sched_request(self._s._sched, self.request_id, info))
        return list(info)

    def _tokens(self, generated: int, start: int, stop: int) -> List[int]:
        out = (ctypes.c_int * max(stop - start, 1))()
        native.check(self._s._lib.vxh_sched_request_tokens(self._s._sched, self.request_id, generated, start, stop, out))
        return list(out[:stop - start])

    @property
    def params(self) -> SamplingParams:
        return self._s._params[self.request_id]

    @property
    def prompt(self) -> List[int]:
        return self._tokens(0, 0, self._info()[0])

    @property
    def generated(self) -> List[int]:
        return self._tokens(1, 0, self._info()[1])

    @property
    def num_generated(self) -> int:
        return self._info()[1]

    @property
    def last_token(self) -> int:
        n = self._info()[1]
        return self._tokens(1, n - 1, n)[0]

    @property
    def status(self) -> str:
        return _STATUS[self._info()[2]]

    @property
    def finish_reason(self) -> Optional[str]:
        return _REASON[self._info()[3]]

    @property
    def admitted_at(self) -> int:
        return self._info()[4]

    @property
    def preemptions(self) -> int:
        return self._info()[5]

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.generated

    @property
    def num_tokens(self) -> int:
        info = self._info()
        return info[0] + info[1]

    def __eq__(self, other) -> bool:
        return (isinstance(other, Request) and other.request_id == self.request_id
                and other._s._sched.value == self._s._sched.value)

    def __hash__(self) -> int:
        return hash(self.request_id)

    def __repr__(self) -> str:
        return "Request(%d, %s)" % (self.request_id, self.status)


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
    requests_aborted: int = 0   # withdrawn with `cancel`; not among the completed
    last_step_us: int = 0       # wall time of the last step, from its planning to its tokens
    total_step_us: int = 0

    @property
    def mean_step_us(self) -> float:
        return self.total_step_us / self.steps if self.steps else 0.0


class _Queue(Mapping):
    """`scheduler.running` / `scheduler.finished`: request id -> `Request`, by id."""

    def __init__(self, scheduler: "Scheduler", which: int):
        self._s, self._which = weakref.proxy(scheduler), which  # (the scheduler holds this view: no cycle)

    def _ids(self) -> List[int]:
        s = self._s
        n = s._lib.vxh_sched_list(s._sched, self._which, None, 0)
        out = (ctypes.c_int64 * max(n, 1))()
        s._lib.vxh_sched_list(s._sched, self._which, out, n)
        return list(out[:n])

    def __getitem__(self, request_id) -> Request:
        if not isinstance(request_id, int) or not self._s._lib.vxh_sched_contains(self._s._sched, self._which, request_id):
            raise KeyError(request_id)
        return Request(self._s, request_id)

    def __iter__(self) -> Iterator[int]:
        return iter(self._ids())

    def __len__(self) -> int:
        return int(self._s._lib.vxh_sched_list(self._s._sched, self._which, None, 0))


class _Waiting(Sequence):
    """`scheduler.waiting`: the queue, its head first."""

    def __init__(self, scheduler: "Scheduler"):
        self._q = _Queue(scheduler, 0)

    def __getitem__(self, i):
        ids = self._q._ids()
        if isinstance(i, slice):
            return [Request(self._q._s, r) for r in ids[i]]
        return Request(self._q._s, ids[i])

    def __len__(self) -> int:
        return len(self._q)


class Scheduler:
    def __init__(self, cache: CacheManager, max_running_requests: int = 64, max_batch_tokens: int = 2048,
                 chunk_size: Optional[int] = None, max_model_len: Optional[int] = None):
        self.cache = cache
        self.max_running_requests = int(max_running_requests)
        self.max_batch_tokens = int(max_batch_tokens)
        self.chunk_size = chunk_size
        self._lib = native.library()
        self._sched = ctypes.c_void_p(self._lib.vxh_sched_create(
            cache._book, self.max_running_requests, self.max_batch_tokens, int(chunk_size or 0), int(max_model_len or 0)))
        if not self._sched:
            raise ValueError("max_running_requests and max_batch_tokens must be positive")
        self.max_model_len = int(self._lib.vxh_sched_max_model_len(self._sched))
        self._params: Dict[int, SamplingParams] = {}
        self.waiting = _Waiting(self)
        self.running = _Queue(self, 1)
        self.finished = _Queue(self, 2)

    def __del__(self):
        if getattr(self, "_sched", None):
            self._lib.vxh_sched_destroy(self._sched)
            self._sched = None

    @property
    def stats(self) -> SchedulerStats:
        out = (ctypes.c_int64 * 11)()
        self._lib.vxh_sched_stats(self._sched, out)
        return SchedulerStats(*[int(x) for x in out])

    def params_of(self, request_id: int) -> SamplingParams:
        return self._params[request_id]

    def request(self, request_id: int) -> Request:
        """The request with that id, wherever it is (KeyError if there is none)."""
        r = Request(self, request_id)
        r._info()
        return r

    # -- submit ---------------------------------------------------------------
    def submit(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        params = params or SamplingParams()
        toks = native.int_array(int(t) for t in prompt)
        stops = native.int_array(list(params.eos_token_ids) + list(params.stop_token_ids))
        seqs = [[int(t) for t in q] for q in params.stop_sequences if len(q)]
        flat, lens = native.int_array(t for q in seqs for t in q), native.int_array(len(q) for q in seqs)
        rid = native.check(self._lib.vxh_sched_submit(self._sched, toks, len(toks), int(params.max_tokens),
                                                      1 if params.ignore_eos else 0, stops, len(stops),
                                                      flat, lens, len(seqs)))
        self._params[rid] = params
        return rid

    def has_work(self) -> bool:
        return bool(self._lib.vxh_sched_has_work(self._sched))

    # -- one step's plan ------------------------------------------------------
    def plan(self) -> Tuple[List[StepEntry], List[Request]]:
        """The next step: its entries (pages already reserved) and the requests
        that were ended while planning (alone and out of pages)."""
        counts = (ctypes.c_longlong * 4)()
        native.check(self._lib.vxh_sched_plan(self._sched, counts))
        n, total, n_ended, n_admitted = (int(x) for x in counts)
        entries: List[StepEntry] = []
        if n:
            ids, starts, lens = (ctypes.c_int64 * n)(), (ctypes.c_int64 * n)(), (ctypes.c_int64 * n)()
            wants, tokens = (ctypes.c_int * n)(), (ctypes.c_int * max(total, 1))()
            self._lib.vxh_sched_plan_entries(self._sched, ids, starts, lens, wants, tokens)
            at = 0
            for i in range(n):
                k = int(lens[i])
                entries.append(StepEntry(int(ids[i]), tokens[at:at + k], [k - 1] if wants[i] else []))
                at += k
        ended: List[Request] = []
        if n_ended:
            ids = (ctypes.c_int64 * n_ended)()
            self._lib.vxh_sched_plan_ended(self._sched, ids)
            ended = [Request(self, int(r)) for r in ids]
        if n_admitted and self.cache._state_layers:
            ids, slots = (ctypes.c_int64 * n_admitted)(), (ctypes.c_int * n_admitted)()
            self._lib.vxh_sched_plan_admitted(self._sched, ids, slots)
            for slot in slots:  # a state slot starts from zero
                self.cache.zero_state(int(slot))
        return entries, ended

    # -- after the step -------------------------------------------------------
    def update(self, entries: Sequence[StepEntry], sampled: Sequence[int]) -> List[Tuple[int, int, bool]]:
        """Takes the tokens sampled for the entries that wanted one (in order).
        Returns (request id, token, finished) for each."""
        n = len(entries)
        ids = native.int64_array(e.request_id for e in entries)
        lens = native.int64_array(len(e.tokens) for e in entries)
        wants = native.int_array(1 if e.want else 0 for e in entries)
        toks = native.int_array(int(t) for t in sampled)
        m = max(len(toks), 1)
        out_ids, out_tok, out_fin = (ctypes.c_int64 * m)(), (ctypes.c_int * m)(), (ctypes.c_int * m)()
        k = native.check(self._lib.vxh_sched_update(self._sched, n, ids, lens, wants, toks, len(toks),
                                                    out_ids, out_tok, out_fin))
        return [(int(out_ids[i]), int(out_tok[i]), bool(out_fin[i])) for i in range(k)]

    def _finish(self, request, reason: str) -> None:
        """Ends a request from outside (its cache is given back)."""
        rid = request.request_id if isinstance(request, Request) else int(request)
        native.check(self._lib.vxh_sched_finish(self._sched, rid, _REASON.index(reason)))

    def cancel(self, request_id: int) -> bool:
        """Withdraws a waiting or running request between two steps: its pages and
        slot are given back at once, its tokens so far stay readable, its finish
        reason is "cancelled" (src/paged/scheduler.rs:440-452).  False if it had
        finished already; KeyError if there is no such request."""
        return bool(native.check(self._lib.vxh_sched_cancel(self._sched, int(request_id))))

    def forget(self, request_id: int) -> None:
        """Drops the record of a finished request whose tokens have been read."""
        self._lib.vxh_sched_forget(self._sched, int(request_id))
        self._params.pop(int(request_id), None)
