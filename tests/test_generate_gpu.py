"""Generation through the Python entry point against the plain implementation."""
import numpy as np
import pytest

import plain_qwen3 as P
from helpers import MAX_SLACK, TINY, random_tokens

pytestmark = pytest.mark.gpu


def engine(folder, name, dtype, **kw):
    from velox_b200 import Engine, EngineConfig
    return Engine(folder, EngineConfig(dtype=dtype, page_size=TINY[name]["page_size"], max_model_len=256, **kw),
                  poison_cache=True)


def check_greedy_path(cfg, w, prompt, generated, dtype):
    """Every generated token is the plain implementation's argmax given the
    engine's own path so far.  In bfloat16 the engine's logits may lie up to MAX_SLACK times
    what rounding costs at that row from the exact ones (helpers.assert_close), so the token
    it picks may be that much below the exact maximum on either side, and no more."""
    rows = list(range(len(prompt) - 1, len(prompt) - 1 + len(generated)))
    logits = P.forward_logits(cfg, w, list(prompt) + list(generated), rows=rows)
    if dtype != "float32":
        rounded = P.forward_logits(cfg, w, list(prompt) + list(generated), store=P.store_bfloat16, rows=rows)
        cost = np.sqrt(np.mean(np.square(rounded - logits), axis=1))
    for n, tok in enumerate(generated):
        row = logits[n]
        best = int(np.argmax(row))
        if dtype == "float32":
            assert tok == best, "token %d: engine %d, plain %d" % (n, tok, best)
        else:
            assert row[best] - row[tok] <= 2 * MAX_SLACK * cost[n], "token %d: engine %d is %.3g below plain's %d (rounding costs %.3g)" % (
                n, tok, row[best] - row[tok], best, cost[n])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_tiny_a(model_folders, dtype):
    from velox_b200 import SamplingParams
    cfg, w = P.load_model_folder(model_folders["tiny_a"])
    prompts = [random_tokens(cfg["vocab_size"], n, 40 + n) for n in (5, 11, 17)]
    e = engine(model_folders["tiny_a"], "tiny_a", dtype, num_pages=64)
    outs = e.generate(prompts, SamplingParams(max_tokens=8))
    assert [len(o) for o in outs] == [8, 8, 8]
    for p, o in zip(prompts, outs):
        check_greedy_path(cfg, w, p, o, dtype)
    if dtype == "float32":
        assert outs == [P.greedy_generate(cfg, w, p, 8) for p in prompts]
    assert e.cache.free_pages() == [64] and e.stats()["requests_completed"] == 3
    e.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_chunked_prefill_mixed_with_decode_and_temperature_tiny_b(model_folders, dtype):
    """Prompts 1, 9, 23, 40 cut into portions of 7 beside decoding requests;
    temperature 0.8 with a fixed seed, 6 new tokens."""
    from velox_b200 import SamplingParams
    from velox_b200.sampling.rng import uniform
    cfg, w = P.load_model_folder(model_folders["tiny_b"])
    prompts = [random_tokens(cfg["vocab_size"], n, 60 + n) for n in (1, 9, 23, 40)]
    e = engine(model_folders["tiny_b"], "tiny_b", dtype, num_pages=40, chunk_size=7, max_batch_tokens=16)
    params = [SamplingParams(max_tokens=6, temperature=0.8, seed=1000 + i) for i in range(4)]
    outs = e.generate(prompts, params)
    assert [len(o) for o in outs] == [6] * 4
    again = engine(model_folders["tiny_b"], "tiny_b", dtype, num_pages=40, chunk_size=3, max_batch_tokens=64)
    assert again.generate(prompts, params) == outs  # the cutting does not change the tokens
    if dtype == "float32":
        for i, (p, o) in enumerate(zip(prompts, outs)):
            logits = P.forward_logits(cfg, w, p + o)
            for n, tok in enumerate(o):
                probs = P.probabilities(logits[len(p) - 1 + n], 0.8)
                assert tok == P.sample_from(probs, uniform(1000 + i, 0, n)), (i, n)
    assert e.stats()["preemptions"] == 0 and e.cache.free_pages() == [40, 40]


def test_pages_run_out_preempted_request_generates_the_same(model_folders):
    from velox_b200 import SamplingParams
    cfg, w = P.load_model_folder(model_folders["tiny_a"])
    prompts = [random_tokens(cfg["vocab_size"], 8, 80 + n) for n in range(3)]
    roomy = engine(model_folders["tiny_a"], "tiny_a", "float32", num_pages=64)
    want = roomy.generate(prompts, SamplingParams(max_tokens=16))
    tight = engine(model_folders["tiny_a"], "tiny_a", "float32", num_pages=12)  # 3 x 24 positions need 18 pages of 4
    got = tight.generate(prompts, SamplingParams(max_tokens=16))
    assert tight.stats()["preemptions"] > 0
    assert got == want
    assert tight.cache.free_pages() == [12]
    tight.cache.check()


def test_eos_and_refusal(model_folders):
    from velox_b200 import SamplingParams
    from velox_b200.engine import RequestRefused
    cfg, w = P.load_model_folder(model_folders["tiny_a"])
    prompt = random_tokens(cfg["vocab_size"], 6, 90)
    e = engine(model_folders["tiny_a"], "tiny_a", "float32", num_pages=64)
    free_run = e.generate([prompt], SamplingParams(max_tokens=8))[0]
    stopped = e.generate([prompt], SamplingParams(max_tokens=8, eos_token_ids=[free_run[2]]))[0]
    assert stopped == free_run[:free_run.index(free_run[2]) + 1]
    with pytest.raises(RequestRefused):
        e.add_request(prompt, SamplingParams(max_tokens=1000))
    with pytest.raises(ValueError):
        e.add_request([cfg["vocab_size"]], SamplingParams(max_tokens=2))


def test_a_single_token_that_wants_nothing_rides_in_a_captured_step(model_folders):
    """A recomputed request may bring one token that is not its last: the step has the
    shape of a decode step (and runs as a captured one), but that row is not sampled."""
    from velox_b200.engine import StepEntry
    cfg, w = P.load_model_folder(model_folders["tiny_a"])
    e = engine(model_folders["tiny_a"], "tiny_a", "float32", num_pages=64)
    a, b = random_tokens(cfg["vocab_size"], 9, 70), random_tokens(cfg["vocab_size"], 6, 71)
    for rid, toks in (("a", a), ("b", b)):
        e.cache.add_request(rid)
        e.run_step([StepEntry(rid, toks[:-1], [])])
    logits, ids = e.runner.step_and_sample([StepEntry("a", [a[-1]], []), StepEntry("b", [b[-1]], [0])], [0.0], [1.0], [0.0])
    assert logits.shape[0] == 1 and ids.tolist() == [int(np.argmax(P.forward_logits(cfg, w, b)[-1]))]
    assert e.cache.length("a") == 9 and e.cache.length("b") == 6
    logits, ids = e.runner.step_and_sample([StepEntry("a", [3], []), StepEntry("b", [4], [])], [], [], [])
    assert logits is None and ids is None


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_graphs_captured_ahead_are_the_ones_the_steps_use(model_folders, dtype):
    """`capture_decode_graphs` records every decode step's graph on padding rows before a
    request exists: it leaves the cache as it found it, generation afterwards gives the
    plain implementation's tokens, and no step has to capture a graph of its own."""
    from velox_b200 import SamplingParams
    cfg, w = P.load_model_folder(model_folders["tiny_b"])
    e = engine(model_folders["tiny_b"], "tiny_b", dtype, num_pages=64, max_running_requests=4)
    n = e.capture_decode_graphs()
    assert n >= 4 and n == len(e.runner.graphs.graphs)
    assert e.capture_decode_graphs() == 0          # all there already
    assert set(e.cache.free_pages()) == {64}       # (every group of layers has its own pages)
    e.cache.check()
    prompts = [random_tokens(cfg["vocab_size"], k, 300 + k) for k in (3, 20, 9, 33)]
    outs = e.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))
    for p, o in zip(prompts, outs):
        check_greedy_path(cfg, w, p, o, dtype)
    assert len(e.runner.graphs.graphs) == n, "a step captured a graph that was not captured ahead"


def test_graphs_of_an_engine_that_is_gone_do_not_disturb_a_capture(model_folders, monkeypatch):
    """Engines come and go in one process.  The graphs of a dead engine are destroyed
    whenever the garbage collector gets to them; if that happened in the middle of
    another engine's capture, the capture would be invalid.  So the collector runs
    before a capture, and here it is also made to run in the middle of one: by then it
    must find nothing of the kind left."""
    import gc
    import torch
    from velox_b200 import SamplingParams
    from velox_b200.engine import graphs
    cfg, w = P.load_model_folder(model_folders["tiny_a"])
    prompt = random_tokens(cfg["vocab_size"], 5, 72)
    want = P.greedy_generate(cfg, w, prompt, 6)
    gc.collect()
    gc.disable()
    try:
        e = engine(model_folders["tiny_a"], "tiny_a", "float32", num_pages=32)
        assert e.generate([prompt], SamplingParams(max_tokens=6)) == [want]
        assert e.runner.graphs.graphs, "the first engine captured no graph"
        ring = [e]
        ring.append(ring)              # only the collector can free this engine and its graphs
        del e, ring
        run_model = graphs._Graph.run_model

        def collecting(self, runner):
            if torch.cuda.is_current_stream_capturing():
                gc.collect()
            return run_model(self, runner)
        monkeypatch.setattr(graphs._Graph, "run_model", collecting)
        e2 = engine(model_folders["tiny_a"], "tiny_a", "float32", num_pages=32)
        assert e2.generate([prompt], SamplingParams(max_tokens=6)) == [want]
    finally:
        gc.enable()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_workloads_generate_what_the_plain_implementation_does(model_folders, dtype):
    """Scheduler, portions, preemption and captured decode steps together: random
    requests, pools from barely enough to ample, budgets from 8 tokens a step."""
    import random
    from velox_b200 import Engine, EngineConfig, SamplingParams
    models = {n: P.load_model_folder(f) for n, f in model_folders.items()}
    preemptions = 0
    for seed in range(24):
        rng = random.Random(seed)
        name = rng.choice(sorted(model_folders))
        cfg, w = models[name]
        page = TINY[name]["page_size"]
        prompts = [random_tokens(cfg["vocab_size"], rng.choice([1, 2, 5, 17, 40, 77, 130]), 1000 * seed + i)
                   for i in range(rng.randint(1, 7))]
        new = [rng.choice([1, 3, 9, 20]) for _ in prompts]
        longest = max(len(p) + n for p, n in zip(prompts, new))
        total = sum(len(p) + n for p, n in zip(prompts, new))
        pool = rng.choice([longest + page, max(longest + page, total // 2), total + 64])
        e = Engine(model_folders[name], EngineConfig(
            dtype=dtype, page_size=page, num_pages=-(-pool // page), max_running_requests=rng.choice([2, 4, 8]),
            max_batch_tokens=rng.choice([8, 32, 64, 256]), chunk_size=rng.choice([None, 3, 16, 50]),
            max_model_len=longest + page))
        outs = e.generate(prompts, [SamplingParams(max_tokens=n, ignore_eos=True) for n in new])
        for p, n, o in zip(prompts, new, outs):
            assert len(o) == n
            check_greedy_path(cfg, w, p, o, dtype)
        e.cache.check()
        assert e.cache.free_pages() == [g.allocator.num_pages for g in e.cache.groups]
        preemptions += e.stats()["preemptions"]
    assert preemptions > 0, "no workload ran out of pages: the test lost its point"


def test_an_engine_ends_when_it_is_dropped(model_folders):
    """No reference cycle holds an engine: its cache pool, graphs and host-side books
    are gone when the last reference is, without waiting for the garbage collector."""
    import gc
    import weakref
    import torch
    from velox_b200 import SamplingParams
    gc.collect()
    gc.disable()
    try:
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        e = engine(model_folders["tiny_a"], "tiny_a", "bfloat16", num_pages=4096)
        e.generate([[1, 2, 3]], SamplingParams(max_tokens=4))
        assert torch.cuda.memory_allocated() > before
        alive = [weakref.ref(e), weakref.ref(e.cache), weakref.ref(e.scheduler), weakref.ref(e.runner)]
        pool = e.cache.groups[0].allocator
        del e
        assert [r() for r in alive] == [None] * 4
        with pytest.raises(ReferenceError):
            pool.num_free                      # a pool of a manager that is gone says so
        assert torch.cuda.memory_allocated() <= before
    finally:
        gc.enable()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("count", [9, 17, 24, 33, 64])
def test_decode_steps_of_more_than_eight_requests(model_folders, dtype, count):
    """Decode steps of 9 to 64 requests run as captured graphs padded to multiples of 8
    rows.  Prompts of mixed lengths (some past 256 and 512 keys, so requests of one step
    have different numbers of 256-key pieces) and different numbers of new tokens, so
    that requests finish at different steps and the batch shrinks through every bucket
    below its first.  The pool is filled with NaN first."""
    from velox_b200 import Engine, EngineConfig, SamplingParams
    name = "tiny_d"
    cfg, w = P.load_model_folder(model_folders[name])
    lens = [(3, 40, 100, 260, 17, 300, 520, 64, 600, 1, 33)[i % 11] for i in range(count)]
    new = [6 + (7 * i) % 13 for i in range(count)]
    prompts = [random_tokens(cfg["vocab_size"], n, 9000 + 100 * count + i) for i, n in enumerate(lens)]
    pages = sum(-(-(n + k) // 16) for n, k in zip(lens, new)) + 4
    e = Engine(model_folders[name], EngineConfig(dtype=dtype, page_size=16, num_pages=pages, max_model_len=640,
                                                 max_running_requests=64, max_batch_tokens=4096), poison_cache=True)
    outs = e.generate(prompts, [SamplingParams(max_tokens=k, ignore_eos=True) for k in new])
    assert [len(o) for o in outs] == new
    for p, o in zip(prompts, outs):
        check_greedy_path(cfg, w, p, o, dtype)
    buckets = sorted({b for b, _ in e.runner.graphs.graphs})
    padded = -(-count // 8) * 8
    assert padded in buckets and all(b <= 8 or b % 8 == 0 for b in buckets), buckets
    assert len([b for b in buckets if b > 8]) >= max(1, (padded // 8 - 1) // 2), buckets   # and buckets on the way down
    e.cache.check()
    assert e.cache.free_pages() == [pages, pages] and e.stats()["preemptions"] == 0


def test_cancelling_a_request_leaves_the_others_tokens_as_they_were(model_folders):
    """A request withdrawn between two steps gives its pages back at once; what the
    others generate does not change (src/paged/scheduler.rs:440-452)."""
    from velox_b200 import SamplingParams
    cfg, w = P.load_model_folder(model_folders["tiny_a"])
    prompts = [random_tokens(cfg["vocab_size"], n, 600 + n) for n in (7, 30, 12, 21)]
    want = [P.greedy_generate(cfg, w, p, 10) for p in prompts]
    e = engine(model_folders["tiny_a"], "tiny_a", "float32", num_pages=48, max_batch_tokens=16, max_running_requests=3)
    ids = [e.add_request(p, SamplingParams(max_tokens=10, ignore_eos=True)) for p in prompts]
    e.step()                                       # 7 + 9 of the 30: request 1 is in the middle of its prompt
    assert e.request(ids[1]).status == "running" and e.request(ids[1]).num_generated == 0
    assert e.cancel(ids[1]) is True
    e.step(); e.step(); e.step()
    assert e.request(ids[3]).status in ("running", "waiting")
    assert e.cancel(ids[3]) is True                # while it waits or has just begun
    held = e.request(ids[0]).num_generated
    assert held >= 3
    while e.scheduler.has_work():
        e.step()
    for i in (0, 2):
        r = e.request(ids[i])
        assert r.generated == want[i] and r.finish_reason == "length"
    for i in (1, 3):
        r = e.request(ids[i])
        assert r.finish_reason == "cancelled" and r.generated == want[i][:len(r.generated)]
    assert e.cancel(ids[0]) is False
    st = e.stats()
    assert st["requests_aborted"] == 2 and st["requests_completed"] == 2 and st["last_step_us"] > 0
    assert e.cache.free_pages() == [48]
    e.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("portion", [40, 16])
def test_small_mixed_steps_of_a_recurring_shape_run_from_a_graph(model_folders, dtype, portion):
    """A long prompt fed in portions of a fixed size beside four decoding requests gives the same
    shape of step again and again: from its third occurrence the step is captured in a CUDA graph
    and replayed.  Logits before, at and after the capture against the plain implementation (a
    portion of 40 goes to the tcgen05 prompt kernel, one of 16 token by token to the decode kernel)."""
    from helpers import Oracle, RoundingJudge, assert_close
    from velox_b200.engine import StepEntry
    name = "tiny_d"
    cfg, w = P.load_model_folder(model_folders[name])
    from velox_b200 import Engine, EngineConfig
    e = Engine(model_folders[name], EngineConfig(dtype=dtype, page_size=16, num_pages=96, max_model_len=512,
                                                 max_running_requests=8), poison_cache=True)
    steps = 9
    long_ = random_tokens(cfg["vocab_size"], 30 + portion * steps, 77)
    shorts = [random_tokens(cfg["vocab_size"], 20 + 13 * i + steps, 78 + i) for i in range(4)]
    oracles = {"L": Oracle(cfg, w, long_)}
    oracles.update({"s%d" % i: Oracle(cfg, w, t) for i, t in enumerate(shorts)})
    judge = RoundingJudge.of(oracles.values(), "mixed steps from a graph (%d)" % portion)
    e.cache.add_request("L")
    e.run_step([StepEntry("L", long_[:30], [])])
    at = {"L": 30}
    for i, t in enumerate(shorts):
        e.cache.add_request("s%d" % i)
        at["s%d" % i] = len(t) - steps
        e.run_step([StepEntry("s%d" % i, t[:at["s%d" % i]], [])])
    for k in range(steps):
        entries, rows, costs = [], [], []
        for i, t in enumerate(shorts):
            rid = "s%d" % i
            entries.append(StepEntry(rid, [t[at[rid]]], [0]))
            rows.append(oracles[rid][at[rid]])
            costs.append(oracles[rid].cost[at[rid]])
            at[rid] += 1
        entries.insert(2, StepEntry("L", long_[at["L"]:at["L"] + portion], [0, portion - 1]))   # (in the middle of the step)
        rows[2:2] = [oracles["L"][at["L"]], oracles["L"][at["L"] + portion - 1]]
        costs[2:2] = [oracles["L"].cost[at["L"]], oracles["L"].cost[at["L"] + portion - 1]]
        at["L"] += portion
        got = e.run_step(entries).cpu().numpy()
        assert_close(got, np.stack(rows), dtype, "step %d (%d graphs)" % (k, len(e.runner.graphs.mixed)),
                     cost=np.array(costs), judge=judge)
    if dtype == "bfloat16":
        judge.finish()
    g = e.runner.graphs
    assert len(g.mixed) >= 1 and any(m.graph is not None for m in g.mixed.values()), "no mixed step was captured"
