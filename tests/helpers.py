"""Tiny configurations and helpers shared by the tests.

Configurations of the architecture that differ in every size and option:

            layers hidden heads kv  head_dim inter vocab theta  eps   head    bias  window      page
  tiny_a      2     64     4    2     16     128   256   1e4    1e-6  tied    no    none          4
  tiny_b      3     96     8    2     32     160   384   1e6    1e-5  untied  yes   20 (layers    8
                                                                                    1 and 2)
  tiny_c      2     128    4    2     64     192   300   5e5    1e-6  untied  no    40 (layer 1)  16
  tiny_d      2     256    4    2     128    384   320   1e6    1e-6  tied    no    200 (layer 1) 16
"""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

TINY = {
    "tiny_a": dict(
        seed=0, page_size=4,
        config=dict(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                    num_attention_heads=4, head_dim=16, attention_bias=False, num_key_value_heads=2,
                    max_position_embeddings=512, tie_word_embeddings=True, rope_theta=10000.0,
                    rms_norm_eps=1e-6, hidden_act="silu")),
    "tiny_b": dict(
        seed=1, page_size=8,
        config=dict(vocab_size=384, hidden_size=96, intermediate_size=160, num_hidden_layers=3,
                    num_attention_heads=8, head_dim=32, attention_bias=True, num_key_value_heads=2,
                    max_position_embeddings=1024, tie_word_embeddings=False, rope_theta=1000000.0,
                    rms_norm_eps=1e-5, hidden_act="silu", use_sliding_window=True, sliding_window=20,
                    max_window_layers=1)),
    # head size 64 and pages of 16: the sizes the tensor-core attention kernels take
    "tiny_c": dict(
        seed=2, page_size=16,
        config=dict(vocab_size=300, hidden_size=128, intermediate_size=192, num_hidden_layers=2,
                    num_attention_heads=4, head_dim=64, attention_bias=False, num_key_value_heads=2,
                    max_position_embeddings=2048, tie_word_embeddings=False, rope_theta=500000.0,
                    rms_norm_eps=1e-6, hidden_act="silu", use_sliding_window=True, sliding_window=40,
                    max_window_layers=1)),
    # head size 128, two query heads per kv head: the sizes the tcgen05 attention kernel takes
    "tiny_d": dict(
        seed=3, page_size=16,
        config=dict(vocab_size=320, hidden_size=256, intermediate_size=384, num_hidden_layers=2,
                    num_attention_heads=4, head_dim=128, attention_bias=False, num_key_value_heads=2,
                    max_position_embeddings=4096, tie_word_embeddings=True, rope_theta=1000000.0,
                    rms_norm_eps=1e-6, hidden_act="silu", use_sliding_window=True, sliding_window=200,
                    max_window_layers=1)),
}

FP32_ATOL = 1e-4
# bfloat16 logits are held to what rounding costs.  The plain implementation with every
# stored activation rounded to bfloat16 (`store=store_bfloat16`) lies at some root-mean-
# square distance from the exact logits of a row: the row's `cost`.  The engine rounds at
# the same places but not to the same bits, so its distance from the exact logits is
# another draw of the same random quantity.  At a width of 4,096 that quantity hardly
# varies from draw to draw (tests/test_real_sizes_gpu.py holds every row to 1.25 times its
# cost); at the tiny models' widths of 50 to 256 a single row's distance scatters by tens of
# per cent around its mean.  So three things are asked (`RoundingJudge`):
#   pooled over all rows of a test, the engine's rms distance is at most RMS_SLACK times
#     the pooled cost (the scatter averages out over hundreds of rows; a part that rounds
#     once more than it has to shows here: 1.4 to 1.7 times);
#   no row's rms distance exceeds ROW_SLACK times its cost (or the pooled cost, if larger:
#     the largest seen over some 15,000 rows of the tiny models is 1.3);
#   no single value is further off than MAX_SLACK times that.
# A wrong or missing key, a stale page or a wrong position moves logits by many times what
# rounding does.  (An elementwise bound of 3e-2 + 3e-2 |x|, which the reference's kernel
# tests use, tests/metal_decode_parity.rs:131-136, is a tenth of the spread of the tiny
# models' logits and could hardly fail.)
RMS_SLACK, ROW_SLACK, MAX_SLACK = 1.25, 2.0, 8.0
REPORT = []   # (what, rows, pooled ratio, largest row ratio, largest single-value ratio) per judged test


def tiny_config(name):
    from velox_b200.config import Qwen3Config
    return Qwen3Config.from_dict(TINY[name]["config"])


def write_tiny(name, folder, dtype="bfloat16"):
    from velox_b200.weights import write_random_model
    return write_random_model(folder, tiny_config(name), TINY[name]["seed"], dtype=dtype)


def random_tokens(vocab, length, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, size=length)]


class Oracle:
    """The plain implementation's logits of one whole sequence: `exact` [T, V] (float64)
    and `cost` [T], the root-mean-square distance per row of the same computation with
    every stored activation rounded to bfloat16.  `oracle[row]` is the exact row."""

    def __init__(self, cfg, w, tokens, rows=None):
        import plain_qwen3 as P
        self.exact = P.forward_logits(cfg, w, tokens, rows=rows)
        rounded = P.forward_logits(cfg, w, tokens, store=P.store_bfloat16, rows=rows)
        self.cost = np.sqrt(np.mean(np.square(rounded - self.exact), axis=1))

    def __getitem__(self, row):
        return self.exact[row]


class RoundingJudge:
    """Judges the bfloat16 results of one test against what rounding costs (see above).
    `typical`: the pooled cost of the test's oracles, known before anything runs."""

    def __init__(self, what, typical=0.0):
        self.what, self.typical = what, float(typical)
        self.err2 = self.cost2 = 0.0
        self.rows, self.worst_row, self.worst_value = 0, 0.0, 0.0

    @staticmethod
    def of(oracles, what):
        costs = np.concatenate([np.ravel(o.cost) for o in oracles])
        return RoundingJudge(what, np.sqrt(np.mean(costs * costs)))

    def check(self, got, want, cost, what=""):
        got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
        cost = np.asarray(cost, np.float64)
        assert got.shape == want.shape, "%s: shape %s vs %s" % (what, got.shape, want.shape)
        assert np.isfinite(got).all(), "%s: non-finite values in the engine's output" % what
        err = np.abs(got - want)
        rms = np.sqrt(np.mean(err * err, axis=1))
        scale = np.maximum(cost, self.typical)
        r_row, r_val = rms / scale, err.max(axis=1) / scale
        self.err2 += float(np.sum(rms * rms))
        self.cost2 += float(np.sum(cost * cost))
        self.rows += len(rms)
        self.worst_row, self.worst_value = max(self.worst_row, r_row.max()), max(self.worst_value, r_val.max())
        bad = (r_row > ROW_SLACK) | (r_val > MAX_SLACK)
        if bad.any():
            rows = np.nonzero(bad)[0]
            k = rows[np.argmax(r_row[rows])]
            raise AssertionError(
                "%s: %d rows beyond what rounding to bfloat16 costs; first wrong row %d, wrong rows %s; row %d: rms "
                "distance %.4g (rounding alone %.4g, pooled %.4g: ratio %.2f), largest single error %.4g (ratio %.1f)"
                % (what, len(rows), rows[0], rows[:20].tolist(), k, rms[k], cost[k], self.typical, r_row[k],
                   err[k].max(), r_val[k]))

    def finish(self):
        """The pooled measure, once every step of the test has been checked."""
        assert self.rows > 0, "%s: nothing was judged" % self.what
        ratio = (self.err2 / self.cost2) ** 0.5
        REPORT.append((self.what, self.rows, ratio, self.worst_row, self.worst_value))
        assert ratio <= RMS_SLACK, (
            "%s: over %d rows the engine lies %.3f times as far from the exact logits as rounding to bfloat16 "
            "alone does (at most %.2f)" % (self.what, self.rows, ratio, RMS_SLACK))


def assert_close(got, want, dtype, what="", cost=None, judge=None):
    """float32: every value within FP32_ATOL.  bfloat16: by `judge` (a RoundingJudge,
    whose `finish()` the test calls at its end) with `cost` [rows]."""
    if dtype != "float32":
        assert cost is not None and judge is not None, "bfloat16 results are judged by what rounding costs"
        judge.check(got, want, cost, what)
        return
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, "%s: shape %s vs %s" % (what, got.shape, want.shape)
    assert np.isfinite(got).all(), "%s: non-finite values in the engine's output" % what
    err = np.abs(got - want)
    bad = err > FP32_ATOL
    if bad.any():
        idx = np.unravel_index(np.argmax(err), err.shape)
        rows = np.unique(np.nonzero(bad)[0])
        raise AssertionError("%s: %d values beyond %g (float32); worst at %s: got %.6g want %.6g; first wrong row %d, wrong rows %s"
                             % (what, int(bad.sum()), FP32_ATOL, idx, got[idx], want[idx], rows[0], rows[:20].tolist()))


def run_trace(model_dir, dtype, steps, max_tokens, out_dir, page_size=16, poison=True, timeout=600, max_requests=None):
    """Runs bin/trace_run as a user would: steps on stdin one at a time, waiting
    for `done <step>` after each.  Returns {step: float32 array [wanted, vocab]}."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens), "--page-size", str(page_size)]
    if poison:
        cmd.append("--poison-cache")
    if max_requests is not None:
        cmd += ["--max-requests", str(max_requests)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
    try:
        for rec in steps:
            proc.stdin.write(json.dumps(rec) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline()
            assert line.strip() == "done %s" % rec["step"], "trace_run answered %r to step %r" % (line, rec["step"])
        proc.stdin.close()
        assert proc.wait(timeout=timeout) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    with open(os.path.join(model_dir, "config.json")) as f:
        vocab = json.load(f)["vocab_size"]
    out = {}
    for rec in steps:
        p = os.path.join(out_dir, "%s.f32" % rec["step"])
        if os.path.exists(p):
            out[rec["step"]] = np.fromfile(p, dtype="<f4").reshape(-1, vocab)
    return out
