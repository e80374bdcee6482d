"""Trace replay through bin/trace_run against the plain implementation: the same
requests whole, with the last 32 tokens one by one, in portions of changing size,
and mixed with other requests in a pool so small that pages are used again; in
32-bit and in bfloat16.  The cache pool is filled with NaN first, so a read of a
slot that was never written (or written by somebody else and not yet
overwritten) cannot pass unnoticed."""
import numpy as np
import pytest

import plain_qwen3 as P
from helpers import TINY, Oracle, RoundingJudge, assert_close, random_tokens, run_trace

pytestmark = pytest.mark.gpu

LENGTHS = {"tiny_a": [70, 45, 33, 90, 1, 2, 3, 64], "tiny_b": [81, 40, 57, 96, 1, 2, 3, 48],
           "tiny_c": [300, 45, 129, 77, 1, 2, 17, 64], "tiny_d": [420, 45, 129, 300, 1, 2, 17, 64]}


class Trace:
    def __init__(self):
        self.steps, self.expect, self.cost = [], {}, {}

    def add(self, entries, end=(), plain=None):
        """entries: [(request id, tokens, want, first position)]"""
        n = len(self.steps)
        self.steps.append({"step": n, "entries": [{"id": i, "tokens": t, "want": w} for i, t, w, _ in entries],
                           "end": list(end)})
        rows = [plain[i][pos + w_] for i, t, w, pos in entries for w_ in w]
        if rows:
            self.expect[n] = np.stack(rows)
            self.cost[n] = np.array([plain[i].cost[pos + w_] for i, t, w, pos in entries for w_ in w])


def cut(tokens, sizes):
    out, at, k = [], 0, 0
    while at < len(tokens):
        s = sizes[k % len(sizes)]
        out.append((at, tokens[at:at + s]))
        at += s
        k += 1
    return out


def build_trace(seqs, plain):
    """seqs: {id: tokens}; plain: {id: logits [T, V]} -> Trace with all four ways of cutting."""
    tr = Trace()
    ids = list(seqs)
    # 1. each request alone and whole
    for i in ids:
        t = seqs[i]
        tr.add([(i, t, list(range(len(t))), 0)], end=[i], plain=plain)
    # 2. most of it in one step, the last 32 tokens one by one
    for i in ids:
        t = seqs[i]
        head = max(len(t) - 32, 0)
        if head:
            tr.add([(i, t[:head], list(range(head)), 0)], plain=plain)
        for p in range(head, len(t)):
            tr.add([(i, [t[p]], [0], p)], end=[i] if p == len(t) - 1 else [], plain=plain)
    # 3. portions of changing size, down to two tokens
    for i in ids:
        t = seqs[i]
        parts = cut(t, [7, 5, 3, 2, 2, 11, 2, 1, 16])
        for n, (at, toks) in enumerate(parts):
            tr.add([(i, toks, list(range(len(toks))), at)], end=[i] if n == len(parts) - 1 else [], plain=plain)
    # 4. mixed: up to four live, portions of some beside decoded tokens of others;
    #    later requests start when earlier ones end, in the pages those gave back
    waiting = list(ids)
    live = {}  # id -> position reached
    sizes = {}
    k = 0
    while waiting or live:
        while waiting and len(live) < 4:
            i = waiting.pop(0)
            live[i] = 0
            # some requests go in portions then token by token, some token by token early
            sizes[i] = [[9, 4, 2], [13], [2, 3], [6, 1, 1]][k % 4]
            k += 1
        entries, end = [], []
        for n, i in enumerate(list(live)):
            t, at = seqs[i], live[i]
            left = len(t) - at
            s = 1 if left <= 12 + 5 * (n % 2) else sizes[i][(at + n) % len(sizes[i])]
            s = min(s, left)
            if (len(tr.steps) + n) % 5 == 4 and len(live) > 1:
                continue  # a request may sit out a step and go on later
            entries.append((i, t[at:at + s], list(range(s)), at))
            live[i] = at + s
            if live[i] == len(t):
                end.append(i)
                del live[i]
        if entries:
            tr.add(entries, end=end, plain=plain)
    return tr


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c", "tiny_d"])
def test_replay_every_way_of_cutting(model_folders, tmp_path, name, dtype):
    folder = model_folders[name]
    cfg, w = P.load_model_folder(folder)
    seqs = {"r%d" % n: random_tokens(cfg["vocab_size"], L, 100 + n) for n, L in enumerate(LENGTHS[name])}
    plain = {i: Oracle(cfg, w, t) for i, t in seqs.items()}
    tr = build_trace(seqs, plain)
    # the four longest live at once, each rounded up to 64: nothing to spare, so pages are used again
    pool = sum(-(-L // 64) * 64 for L in sorted(LENGTHS[name])[-4:])
    got = run_trace(folder, dtype, tr.steps, pool, str(tmp_path / "out"), page_size=TINY[name]["page_size"])
    assert sorted(got) == sorted(tr.expect)
    judge = RoundingJudge.of(plain.values(), "replay %s" % name)
    for n in sorted(tr.expect):
        assert_close(got[n], tr.expect[n], dtype, "%s %s step %d %s" % (name, dtype, n, [
            (e["id"], len(e["tokens"])) for e in tr.steps[n]["entries"]]), cost=tr.cost[n], judge=judge)
    if dtype == "bfloat16":
        judge.finish()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_folders, tmp_path, dtype):
    """Several hundred tokens one by one, two requests side by side."""
    folder = model_folders["tiny_c"]
    cfg, w = P.load_model_folder(folder)
    seqs = {"x": random_tokens(cfg["vocab_size"], 420, 7), "y": random_tokens(cfg["vocab_size"], 333, 8)}
    plain = {i: Oracle(cfg, w, t) for i, t in seqs.items()}
    tr = Trace()
    tr.add([("x", seqs["x"][:20], [19], 0), ("y", seqs["y"][:5], [4], 0)], plain=plain)
    at = {"x": 20, "y": 5}
    while at:
        entries, end = [], []
        for i in list(at):
            entries.append((i, [seqs[i][at[i]]], [0], at[i]))
            at[i] += 1
            if at[i] == len(seqs[i]):
                end.append(i)
                del at[i]
        tr.add(entries, end=end, plain=plain)
    got = run_trace(folder, dtype, tr.steps, 448 + 384, str(tmp_path / "out"), page_size=16)
    judge = RoundingJudge.of(plain.values(), "long decoding")
    for n in sorted(tr.expect):
        assert_close(got[n], tr.expect[n], dtype, "long decode step %d" % n, cost=tr.cost[n], judge=judge)
    if dtype == "bfloat16":
        judge.finish()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_in_one_step_and_in_two(model_folders, tmp_path, dtype):
    """1,100 tokens at once (the step's matrix products and attention take their
    large-shape kernels), then the same prompt as 1,030 + 70 on top of the cache."""
    folder = model_folders["tiny_d"]
    cfg, w = P.load_model_folder(folder)
    toks = random_tokens(cfg["vocab_size"], 1100, 9)
    plain = {"whole": Oracle(cfg, w, toks)}
    plain["cut"] = plain["whole"]
    want = list(range(0, 1100, 37)) + [1099]
    tr = Trace()
    tr.add([("whole", toks, want, 0)], end=["whole"], plain=plain)
    tr.add([("cut", toks[:1030], [w_ for w_ in want if w_ < 1030], 0)], plain=plain)
    tr.add([("cut", toks[1030:], [w_ - 1030 for w_ in want if w_ >= 1030], 1030)], end=["cut"], plain=plain)
    got = run_trace(folder, dtype, tr.steps, 1152, str(tmp_path / "out"), page_size=16)
    judge = RoundingJudge.of(plain.values(), "a long prompt")
    for n in sorted(tr.expect):
        assert_close(got[n], tr.expect[n], dtype, "long prompt step %d" % n, cost=tr.cost[n], judge=judge)
    if dtype == "bfloat16":
        judge.finish()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_context_of_4000_tokens(model_folders, tmp_path, dtype):
    """A prompt of 3,950 tokens in portions of 2,048, 1,802 (on top of 2,048 cached
    positions) and 100 (on top of 3,850: few query tiles and thirty key tiles, which
    the prefill attention cuts into runs, in the windowed layers runs without keys
    among them), then 50 tokens one by one beside a short request: sixteen pieces of
    keys per decoded token, a window of 200 far from the start."""
    folder = model_folders["tiny_d"]
    cfg, w = P.load_model_folder(folder)
    long_, short = random_tokens(cfg["vocab_size"], 4000, 41), random_tokens(cfg["vocab_size"], 60, 42)
    plain = {"L": Oracle(cfg, w, long_), "s": Oracle(cfg, w, short)}
    tr = Trace()
    tr.add([("L", long_[:2048], [0, 1000, 2047], 0)], plain=plain)
    tr.add([("L", long_[2048:3850], [0, 1, 951, 1801], 2048)], plain=plain)
    tr.add([("L", long_[3850:3950], [0, 1, 31, 32, 64, 99], 3850), ("s", short[:10], [9], 0)], plain=plain)
    for k in range(50):
        tr.add([("L", [long_[3950 + k]], [0], 3950 + k), ("s", [short[10 + k]], [0], 10 + k)],
               end=["L", "s"] if k == 49 else [], plain=plain)
    got = run_trace(folder, dtype, tr.steps, 4032 + 64, str(tmp_path / "out"), page_size=16)
    judge = RoundingJudge.of(plain.values(), "a context of 4000")
    for n in sorted(tr.expect):
        assert_close(got[n], tr.expect[n], dtype, "context of 4000, step %d" % n, cost=tr.cost[n], judge=judge)
    if dtype == "bfloat16":
        judge.finish()


ODD = {
    # seven query heads per kv head, head size 112, three layers, a window on the last two
    "odd_a": dict(seed=11, page_size=16, lens=[150, 45, 33, 90, 1, 2, 3, 64],
                  config=dict(vocab_size=1000, hidden_size=200, intermediate_size=100, num_hidden_layers=3,
                              num_attention_heads=14, head_dim=112, attention_bias=False, num_key_value_heads=2,
                              max_position_embeddings=1024, tie_word_embeddings=True, rope_theta=10000.0,
                              rms_norm_eps=1e-5, hidden_act="silu", use_sliding_window=True, sliding_window=150,
                              max_window_layers=1)),
    # head size 256, five query heads per kv head, a width of 50 and a vocabulary of 97, biases, pages of 8
    "odd_b": dict(seed=12, page_size=8, lens=[130, 45, 33, 70, 1, 2, 3, 64],
                  config=dict(vocab_size=97, hidden_size=50, intermediate_size=144, num_hidden_layers=1,
                              num_attention_heads=10, head_dim=256, attention_bias=True, num_key_value_heads=2,
                              max_position_embeddings=1024, tie_word_embeddings=False, rope_theta=500000.0,
                              rms_norm_eps=1e-6, hidden_act="silu", use_sliding_window=True, sliding_window=33,
                              max_window_layers=0)),
    # a head size that is even and no multiple of 16 (40), three query heads per kv head, a width of 72
    "odd_c": dict(seed=13, page_size=4, lens=[90, 45, 33, 70, 1, 2, 3, 64],
                  config=dict(vocab_size=211, hidden_size=72, intermediate_size=104, num_hidden_layers=2,
                              num_attention_heads=6, head_dim=40, attention_bias=False, num_key_value_heads=2,
                              max_position_embeddings=512, tie_word_embeddings=True, rope_theta=10000.0,
                              rms_norm_eps=1e-6, hidden_act="silu", use_sliding_window=True, sliding_window=50,
                              max_window_layers=1)),
    # heads of 128 with five query heads per kv head (the tensor-core prompt attention gives each head 24 rows of a
    # tile and leaves 8 idle), a window, prompts long enough for two query tiles and several key tiles
    "odd_d": dict(seed=14, page_size=16, lens=[300, 45, 150, 70, 1, 2, 33, 64],
                  config=dict(vocab_size=300, hidden_size=160, intermediate_size=208, num_hidden_layers=2,
                              num_attention_heads=10, head_dim=128, attention_bias=False, num_key_value_heads=2,
                              max_position_embeddings=1024, tie_word_embeddings=True, rope_theta=10000.0,
                              rms_norm_eps=1e-6, hidden_act="silu", use_sliding_window=True, sliding_window=170,
                              max_window_layers=1)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ODD))
def test_sizes_that_no_fast_kernel_takes(tmp_path, name, dtype):
    """Head sizes, group sizes and widths outside what the tensor-core kernels take, or at
    the edge of it: the engine has to find another kernel for each, or refuse; never a wrong
    result."""
    from velox_b200.config import Qwen3Config
    from velox_b200.weights import write_random_model

    spec = ODD[name]
    folder = write_random_model(str(tmp_path / "model"), Qwen3Config.from_dict(spec["config"]), seed=spec["seed"],
                                dtype="bfloat16")
    cfg, w = P.load_model_folder(folder)
    seqs = {"r%d" % n: random_tokens(cfg["vocab_size"], L, 300 + n) for n, L in enumerate(spec["lens"])}
    plain = {i: Oracle(cfg, w, t) for i, t in seqs.items()}
    tr = build_trace(seqs, plain)
    pool = sum(-(-L // 64) * 64 for L in sorted(spec["lens"])[-4:])
    got = run_trace(folder, dtype, tr.steps, pool, str(tmp_path / "out"), page_size=spec["page_size"])
    assert sorted(got) == sorted(tr.expect)
    judge = RoundingJudge.of(plain.values(), "sizes no fast kernel takes, %s" % name)
    for n in sorted(tr.expect):
        assert_close(got[n], tr.expect[n], dtype, "%s %s step %d" % (name, dtype, n), cost=tr.cost[n], judge=judge)
    if dtype == "bfloat16":
        judge.finish()


@pytest.mark.parametrize("seed", [3, 11, 26])
def test_random_traces(model_folders, tmp_path, seed):
    """Requests cut at random: which of up to four live requests go into a step, how
    many tokens each brings (1 to all that is left), which places are wanted, and in
    which order they stand in the step are all drawn; later requests start in the pages
    earlier ones gave back."""
    import random
    rng = random.Random(seed)
    name = rng.choice(sorted(TINY))
    cfg, w = P.load_model_folder(model_folders[name])
    lens = [rng.choice([1, 2, 3, 17, 40, 64, 65, 100, 130, 257, 300]) for _ in range(rng.randint(3, 8))]
    seqs = {"q%d" % i: random_tokens(cfg["vocab_size"], L, 7000 * seed + i) for i, L in enumerate(lens)}
    plain = {i: Oracle(cfg, w, t) for i, t in seqs.items()}
    waiting, live, steps, expect, costs = list(seqs), {}, [], {}, {}
    while waiting or live:
        while waiting and len(live) < 4 and (not live or rng.random() < 0.7):
            live[waiting.pop(0)] = 0
        entries, end, rows, row_costs = [], [], [], []
        order = list(live)
        rng.shuffle(order)
        for i in order:
            if len(live) > 1 and rng.random() < 0.25:
                continue  # sits this step out
            k = min(len(seqs[i]) - live[i], rng.choice([1, 1, 1, 2, 3, 5, 8, 13, 31, 32, 33, 64, 100, 1000]))
            want = sorted(rng.sample(range(k), rng.choice([0, 1, min(k, 3), k])))
            entries.append({"id": i, "tokens": seqs[i][live[i]:live[i] + k], "want": want})
            rows += [plain[i][live[i] + w_] for w_ in want]
            row_costs += [plain[i].cost[live[i] + w_] for w_ in want]
            live[i] += k
            if live[i] == len(seqs[i]):
                end.append(i)
                del live[i]
        steps.append({"step": len(steps), "entries": entries, "end": end})
        if rows:
            expect[len(steps) - 1] = np.stack(rows)
            costs[len(steps) - 1] = np.array(row_costs)
    pool = sum(sorted(-(-L // 64) * 64 for L in lens)[-4:])
    for dtype in ("float32", "bfloat16"):
        got = run_trace(model_folders[name], dtype, steps, pool, str(tmp_path / dtype), page_size=TINY[name]["page_size"])
        assert sorted(got) == sorted(expect)
        judge = RoundingJudge.of(plain.values(), "random trace %d (%s)" % (seed, name))
        for n in sorted(expect):
            assert_close(got[n], expect[n], dtype, "%s %s seed %d step %d" % (name, dtype, seed, n), cost=costs[n],
                         judge=judge)
        if dtype == "bfloat16":
            judge.finish()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_of_twelve_requests_in_a_padded_captured_step(model_folders, tmp_path, dtype):
    """More than eight requests decode together: the step is padded to a bucket of 16 rows
    (rows that read page 0 and write nothing) and runs as a captured graph.  The logits
    of every real row are compared; requests end one after the other, so the batch
    shrinks through 12, 11, 10 and 9 rows of the same bucket and then below it.  (The
    reference's mixed-batch test holds 13 sequences in one batch:
    tests/metal_batched_kernels_parity.rs:297-359.)"""
    folder = model_folders["tiny_d"]
    cfg, w = P.load_model_folder(folder)
    lens = [300, 20, 530, 41, 17, 260, 33, 90, 700, 64, 129, 48]   # some need two and three pieces of 256 keys
    new = [14, 9, 12, 10, 16, 8, 11, 13, 15, 7, 17, 18]
    seqs = {"s%d" % i: random_tokens(cfg["vocab_size"], L + n, 500 + i) for i, (L, n) in enumerate(zip(lens, new))}
    plain = {i: Oracle(cfg, w, t) for i, t in seqs.items()}
    tr = Trace()
    ids = list(seqs)
    for at in range(0, 12, 3):   # the prompts, three requests a step
        tr.add([(i, seqs[i][:lens[k]], [lens[k] - 1], 0) for k, i in enumerate(ids) if at <= k < at + 3], plain=plain)
    pos = {i: lens[k] for k, i in enumerate(ids)}
    sizes = []
    while pos:
        entries, end = [], []
        for i in list(pos):
            entries.append((i, [seqs[i][pos[i]]], [0], pos[i]))
            pos[i] += 1
            if pos[i] == len(seqs[i]):
                end.append(i)
                del pos[i]
        sizes.append(len(entries))
        tr.add(entries, end=end, plain=plain)
    assert sizes[0] == 12 and {9, 10, 11, 12} <= set(sizes) and min(sizes) == 1
    pool = sum(-(-len(t) // 64) * 64 for t in seqs.values())
    got = run_trace(folder, dtype, tr.steps, pool, str(tmp_path / "out"), page_size=16, max_requests=16)
    assert sorted(got) == sorted(tr.expect)
    judge = RoundingJudge.of(plain.values(), "twelve live requests")
    for n in sorted(tr.expect):
        assert_close(got[n], tr.expect[n], dtype, "twelve live, step %d (%d rows)" % (n, len(tr.steps[n]["entries"])),
                     cost=tr.cost[n], judge=judge)
    if dtype == "bfloat16":
        judge.finish()
