"""The scheduler's decisions (CPU), driven with a stand-in for the device step."""
import hashlib

import pytest

from velox_b200.cache import CacheManager
from velox_b200.engine import RequestRefused, Scheduler
from velox_b200.parts.base import PagedKV
from velox_b200.sampling import SamplingParams


def make(num_pages=64, page=4, window=0, **kw):
    specs = [PagedKV(2, 16, 0), PagedKV(2, 16, window)]
    cache = CacheManager(specs, [None, None], page, num_pages, kw.pop("max_requests", 8), kw.pop("max_blocks", 64))
    return cache, Scheduler(cache, **kw)


def next_token(tokens):
    """A stand-in model: the next token is a hash of everything before it."""
    return int.from_bytes(hashlib.sha256(repr(list(tokens)).encode()).digest()[:2], "little") % 251


class Driver:
    """Plays the device: keeps, per request, the tokens its cache would hold."""

    def __init__(self, cache, sched):
        self.cache, self.s, self.held, self.log = cache, sched, {}, []

    def step(self):
        entries, ended = self.s.plan()
        sampled = []
        for e in entries:
            r = self.s.running[e.request_id]
            # a preempted request lost its cache: it starts again from nothing
            have = self.held.setdefault((e.request_id, r.preemptions), [])
            assert len(have) == self.cache.length(e.request_id)
            assert list(e.tokens) == r.tokens[len(have):len(have) + len(e.tokens)], "the step feeds the wrong tokens"
            have.extend(e.tokens)
            self.cache.commit(e.request_id, len(e.tokens))
            if e.want:
                assert list(e.want) == [len(e.tokens) - 1] and len(have) == len(r.tokens)
                sampled.append(next_token(have))
        self.log.append([(e.request_id, len(e.tokens)) for e in entries])
        out = self.s.update(entries, sampled)
        self.cache.check()
        return entries, out

    def run(self, limit=10000):
        while self.s.has_work():
            self.step()
            limit -= 1
            assert limit > 0, "the scheduler does not finish"


def expected(prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(next_token(toks))
    return toks[len(prompt):]


def test_budget_portions_and_order():
    cache, s = make(max_batch_tokens=16)
    d = Driver(cache, s)
    a = s.submit(list(range(40)), SamplingParams(max_tokens=3))
    b = s.submit(list(range(5)), SamplingParams(max_tokens=3))
    d.run()
    assert all(sum(k for _, k in step) <= 16 for step in d.log)
    # first come first served: a's prompt fills the first steps, b starts when budget is left
    assert d.log[0] == [(a, 16)] and d.log[1] == [(a, 16)] and d.log[2] == [(a, 8), (b, 5)]
    # afterwards both decode, one token each, ordered by id
    assert d.log[3] == [(a, 1), (b, 1)]
    assert s.finished[a].generated == expected(range(40), 3) and s.finished[b].generated == expected(range(5), 3)
    assert cache.free_pages() == [64] and not cache.requests


def test_decodes_go_before_prompt_portions():
    cache, s = make(max_batch_tokens=8)
    d = Driver(cache, s)
    a = s.submit([1, 2, 3], SamplingParams(max_tokens=10))
    d.step()
    b = s.submit(list(range(30)), SamplingParams(max_tokens=2))
    entries, _ = d.step()
    assert [(e.request_id, len(e.tokens)) for e in entries] == [(a, 1), (b, 7)]  # 1 decode + 7 of the prompt


def test_fixed_chunk_size():
    cache, s = make(max_batch_tokens=64, chunk_size=7)
    d = Driver(cache, s)
    ids = [s.submit(list(range(n)), SamplingParams(max_tokens=6)) for n in (1, 9, 23, 40)]
    d.run()
    for step in d.log:
        assert all(k <= 7 for _, k in step)
    for rid, n in zip(ids, (1, 9, 23, 40)):
        assert s.finished[rid].generated == expected(range(n), 6)
        assert s.finished[rid].finish_reason == "length"


def test_finish_reasons():
    cache, s = make()
    d = Driver(cache, s)
    prompt = [5, 6, 7]
    want = expected(prompt, 4)
    stop = s.submit(prompt, SamplingParams(max_tokens=10, eos_token_ids=[want[1]]))
    ignore = s.submit(prompt, SamplingParams(max_tokens=4, eos_token_ids=[want[1]], ignore_eos=True))
    d.run()
    assert s.finished[stop].generated == want[:2] and s.finished[stop].finish_reason == "stop"  # the token is kept
    assert s.finished[ignore].generated == want and s.finished[ignore].finish_reason == "length"
    assert s.stats.requests_completed == 2 and s.stats.tokens_generated == 6


def test_refusals():
    cache, s = make(num_pages=8, page=4, max_blocks=16)
    with pytest.raises(RequestRefused, match="empty"):
        s.submit([])
    with pytest.raises(RequestRefused, match="longest"):
        s.submit([1] * 60, SamplingParams(max_tokens=10))  # 70 > 16 * 4
    with pytest.raises(RequestRefused, match="never"):
        s.submit([1] * 30, SamplingParams(max_tokens=10))  # 10 pages > pool of 8
    assert s.stats.requests_refused == 3 and not s.has_work()


def test_max_running_requests():
    cache, s = make(max_running_requests=2)
    d = Driver(cache, s)
    ids = [s.submit([1, 2, i], SamplingParams(max_tokens=3)) for i in range(5)]
    while s.has_work():
        d.step()
        assert len(s.running) <= 2
    assert [s.finished[i].generated for i in ids] == [expected([1, 2, i], 3) for i in range(5)]


def test_pages_run_out_latest_admitted_is_preempted_and_recomputed():
    # 3 requests of 8 prompt tokens that each want to grow to 24 positions (6 pages); pool of 12 pages
    cache, s = make(num_pages=12, page=4)
    d = Driver(cache, s)
    ids = [s.submit([i] * 8, SamplingParams(max_tokens=16)) for i in range(3)]
    d.run()
    assert s.stats.preemptions > 0
    assert s.finished[ids[2]].preemptions > 0 and s.finished[ids[0]].preemptions == 0  # the oldest is never the victim
    for i, rid in enumerate(ids):
        assert s.finished[rid].generated == expected([i] * 8, 16)  # same tokens as without preemption
        assert s.finished[rid].finish_reason == "length"
    assert cache.free_pages() == [12] and cache.slots.num_free == 8


def test_preempted_request_returns_to_the_front():
    # a and b fill the first step's budget, so c still waits when b has to go
    cache, s = make(num_pages=5, page=4, max_batch_tokens=16)
    d = Driver(cache, s)
    a = s.submit([1] * 8, SamplingParams(max_tokens=12))
    b = s.submit([2] * 8, SamplingParams(max_tokens=12))
    c = s.submit([3] * 4, SamplingParams(max_tokens=2))
    saw_preempt = False
    while s.has_work():
        d.step()
        if s.stats.preemptions and not saw_preempt:
            saw_preempt = True
            assert s.waiting[0].request_id == b  # ahead of c, which arrived later
    assert saw_preempt
    for rid, p, n in ((a, [1] * 8, 12), (b, [2] * 8, 12), (c, [3] * 4, 2)):
        assert s.finished[rid].generated == expected(p, n)


def test_a_request_alone_that_cannot_grow_ends_with_length():
    cache, s = make(num_pages=3, page=4, max_blocks=3)
    d = Driver(cache, s)
    # fits at submit (12 positions = 3 pages) ...
    rid = s.submit([7] * 6, SamplingParams(max_tokens=6))
    # ... but somebody else holds a page for good
    cache.add_request("squatter")
    assert cache.reserve("squatter", 1)
    d.run()
    r = s.finished[rid]
    assert r.finish_reason == "length" and 0 < len(r.generated) < 6
    assert r.generated == expected([7] * 6, len(r.generated))


def test_window_group_frees_pages_during_generation():
    cache, s = make(num_pages=16, page=4, window=6)
    d = Driver(cache, s)
    rid = s.submit([1] * 10, SamplingParams(max_tokens=40))
    least_free_windowed = 16
    while s.has_work():
        d.step()
        least_free_windowed = min(least_free_windowed, cache.free_pages()[1])
    assert least_free_windowed >= 16 - 4  # never more than prompt-portion + window pages
    assert s.finished[rid].generated == expected([1] * 10, 40)
    assert cache.free_pages() == [16, 16]


def test_random_workloads_finish_and_free_everything():
    import random
    rng = random.Random(3)
    for trial in range(10):
        cache, s = make(num_pages=rng.randint(10, 30), page=rng.choice([2, 4, 8]), window=rng.choice([0, 7]),
                        max_batch_tokens=rng.choice([4, 16, 64]), chunk_size=rng.choice([None, 3, 7]),
                        max_running_requests=rng.choice([2, 4, 8]))
        d = Driver(cache, s)
        total = cache.free_pages()
        want = {}
        for i in range(rng.randint(3, 10)):
            p = [rng.randrange(250) for _ in range(rng.randint(1, 20))]
            n = rng.randint(1, 12)
            try:
                want[s.submit(p, SamplingParams(max_tokens=n))] = (p, n)
            except RequestRefused:
                pass
            if rng.random() < 0.5 and s.has_work():
                d.step()
        d.run()
        for rid, (p, n) in want.items():
            r = s.finished[rid]
            assert r.generated == expected(p, len(r.generated))
            assert len(r.generated) == n or r.finish_reason == "length"
        assert cache.free_pages() == total and cache.slots.num_free == 8


def test_a_run_of_generated_tokens_can_end_a_request():
    cache, s = make()
    prompt = [3, 1, 4, 1, 5]
    full = expected(prompt, 12)
    stop = full[4:7]                                   # tokens 5 to 7 of what will be generated
    rid = s.submit(prompt, SamplingParams(max_tokens=12, stop_sequences=[[250, 250], stop]))
    other = s.submit(prompt, SamplingParams(max_tokens=12, stop_sequences=[stop[1:] + [stop[0]]]))  # never matches
    Driver(cache, s).run()
    assert s.finished[rid].generated == full[:7] and s.finished[rid].finish_reason == "stop"
    assert s.finished[other].generated == full and s.finished[other].finish_reason == "length"


def test_cancel_while_waiting_in_prompt_in_decode_and_after_preemption():
    # (src/paged/scheduler.rs:440-452: a request whose caller is gone ends with "cancelled" and frees its pages)
    cache, s = make(num_pages=12, page=4, max_batch_tokens=8, max_running_requests=2)
    d = Driver(cache, s)
    a = s.submit([1] * 20, SamplingParams(max_tokens=8))   # its prompt takes three steps
    b = s.submit([2] * 3, SamplingParams(max_tokens=30))
    c = s.submit([3] * 5, SamplingParams(max_tokens=4))    # waits: two requests run at most
    d.step()
    assert s.running[a].status == "running" and cache.length(a) == 8   # in the middle of its prompt
    assert s.cancel(c) is True                                          # while it waits
    assert s.finished[c].finish_reason == "cancelled" and s.finished[c].generated == []
    assert [r.request_id for r in s.waiting] == [b]
    held = 12 - cache.free_pages()[0]
    assert held == 2
    assert s.cancel(a) is True                                          # in the middle of its prompt
    assert cache.free_pages() == [12] and not cache.has_request(a)
    cache.check()
    assert s.finished[a].finish_reason == "cancelled" and s.cancel(a) is False
    for _ in range(4):
        d.step()
    got = list(s.running[b].generated)
    assert len(got) >= 2                                                # b decodes
    assert s.cancel(b) is True
    assert s.finished[b].generated == got == expected([2] * 3, len(got))  # what it had stays readable
    assert not s.has_work() and cache.free_pages() == [12] and cache.slots.num_free == 8
    cache.check()
    st = s.stats
    assert st.requests_aborted == 3 and st.requests_completed == 0
    with pytest.raises(KeyError):
        s.cancel(12345)
    # after a preemption: the victim waits at the front without cache; cancelling it leaves the others as they were
    cache, s = make(num_pages=12, page=4)
    d = Driver(cache, s)
    ids = [s.submit([i] * 8, SamplingParams(max_tokens=16)) for i in range(3)]
    while not s.stats.preemptions:
        d.step()
    victim = s.waiting[0].request_id
    assert s.waiting[0].preemptions == 1 and s.cancel(victim)
    d.run()
    for i, rid in enumerate(ids):
        r = s.finished[rid]
        if rid == victim:
            assert r.finish_reason == "cancelled" and r.generated == expected([i] * 8, len(r.generated))
        else:
            assert r.finish_reason == "length" and r.generated == expected([i] * 8, 16)
    assert cache.free_pages() == [12] and cache.slots.num_free == 8
    assert s.stats.requests_aborted == 1 and s.stats.requests_completed == 2


def test_cancel_in_random_workloads_loses_no_page():
    import random
    rng = random.Random(11)
    for trial in range(10):
        cache, s = make(num_pages=rng.randint(10, 30), page=rng.choice([2, 4, 8]), window=rng.choice([0, 7]),
                        max_batch_tokens=rng.choice([4, 16, 64]), max_running_requests=rng.choice([2, 4, 8]))
        d = Driver(cache, s)
        total = cache.free_pages()
        want, cancelled = {}, set()
        for i in range(rng.randint(4, 10)):
            p = [rng.randrange(250) for _ in range(rng.randint(1, 20))]
            try:
                want[s.submit(p, SamplingParams(max_tokens=rng.randint(1, 12)))] = p
            except RequestRefused:
                pass
            if rng.random() < 0.6 and s.has_work():
                d.step()
            if want and rng.random() < 0.4:
                rid = rng.choice(sorted(want))
                if s.cancel(rid):
                    cancelled.add(rid)
                cache.check()
        d.run()
        for rid, p in want.items():
            r = s.finished[rid]
            assert r.generated == expected(p, len(r.generated))
            assert (r.finish_reason == "cancelled") == (rid in cancelled)
        assert cache.free_pages() == total and cache.slots.num_free == 8
        assert s.stats.requests_aborted == len(cancelled)


def test_step_time_is_kept():
    import time
    cache, s = make()
    d = Driver(cache, s)
    s.submit([1, 2, 3], SamplingParams(max_tokens=3))
    assert s.stats.last_step_us == 0 and s.stats.mean_step_us == 0.0
    entries, _ = s.plan()
    time.sleep(0.02)   # the device's work would pass here
    for e in entries:
        cache.commit(e.request_id, len(e.tokens))
    s.update(entries, [next_token([1, 2, 3])])
    d.held[(0, 0)] = [1, 2, 3]
    st = s.stats
    assert 20000 <= st.last_step_us < 2000000 and st.total_step_us == st.last_step_us and st.steps == 1
    d.run()
    st = s.stats
    assert st.steps == 3 and st.total_step_us >= 20000 and abs(st.mean_step_us - st.total_step_us / 3) < 1e-9
