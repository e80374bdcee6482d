#!/usr/bin/env python3
"""Benchmark of velox_b200: decode tokens per second of a Qwen3-8B-shaped model
with random weights on one B200, plus prefill, batch-1 and batch-64 points and
roofline fractions.  Prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]

A "step" is one decode step of the whole batch.  The timed decode steps are the
last K before the requests reach the context length, so the cache they read is
as long as it gets.  Weights (15 GB) and cache are far larger than L2, so every
step reads them from memory; nothing is flushed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen3-8B shape: the benchmark configuration (36 layers, hidden 4096, 32 query
# heads, 8 kv heads of 128, intermediate 12288, vocabulary 151936, untied head).
MODEL = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
             num_attention_heads=32, head_dim=128, attention_bias=False, num_key_value_heads=8,
             max_position_embeddings=40960, tie_word_embeddings=False, rope_theta=1000000.0,
             rms_norm_eps=1e-6, hidden_act="silu")
# Other shapes of the same architecture, for measurements beside the benchmark's (`--shape`).
SHAPES = {
    "0.6b": dict(hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16, tie_word_embeddings=True),
    "1.7b": dict(hidden_size=2048, intermediate_size=6144, num_hidden_layers=28, num_attention_heads=16, tie_word_embeddings=True),
    "4b": dict(hidden_size=2560, intermediate_size=9728, num_hidden_layers=36, num_attention_heads=32, tie_word_embeddings=True),
    "8b": {},
    "14b": dict(hidden_size=5120, intermediate_size=17408, num_hidden_layers=40, num_attention_heads=40),
    "32b": dict(hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64),
}
CONTEXT, PROMPT, PAGE, BATCH, SEED = 4096, 2048, 16, 8, 2
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                raw = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(raw.get(k), (int, float)):
                    out[k] = float(raw[k])
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(mhz)}


def weight_bytes(cfg, layers, elt=2):
    E, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, Hk, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    return (layers * ((H + 2 * Hk) * D * E + E * H * D + 3 * I * E) + 2 * V * E) * elt


def decode_bytes(cfg, layers, batch, kv_len, elt=2):
    """Bytes a decode step has to read: every weight once, and the live requests' cache."""
    E, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, Hk, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = ((H + 2 * Hk) * D * E + E * H * D + 3 * I * E) * elt
    weights = layers * per_layer + V * E * elt  # head; the embedding rows read are negligible
    kv = layers * 2 * Hk * D * elt * batch * kv_len
    return weights + kv


def prefill_flops(cfg, layers, tokens):
    E, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, Hk, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    linear = 2 * tokens * layers * ((H + 2 * Hk) * D * E + E * H * D + 3 * I * E)
    attn = layers * H * 2 * D * tokens * tokens  # causal: half of 4 D T^2
    return linear + attn + 2 * V * E


def stream_workload(args, cfg, layers):
    """Continuous batching under arrivals: 64 requests with prompts of 128 to 4,096
    random tokens and 256 new tokens each arrive as a Poisson stream; every step goes
    through `Engine.step`.  Reports generated tokens a second over the whole run,
    time to the first token and time between tokens (host clock around the steps,
    which end with the read of the sampled ids), and the scheduler's counters."""
    import random

    import torch
    from velox_b200 import Engine, EngineConfig, SamplingParams

    n_req, new_tokens, longest = 64, 256, 4096
    rng = random.Random(SEED + 1)
    lens = [rng.randint(128, longest) for _ in range(n_req)]
    arrivals, t = [], 0.0
    for _ in range(n_req):
        t += rng.expovariate(args.arrival_rate)
        arrivals.append(t)
    pool = args.pool_tokens or n_req * (longest + new_tokens + PAGE)
    engine = Engine(model_config=cfg, random_seed=SEED, config=EngineConfig(
        dtype="bfloat16", page_size=PAGE, num_pages=-(-pool // PAGE), max_running_requests=n_req,
        max_batch_tokens=args.max_batch_tokens, max_model_len=longest + new_tokens + PAGE))
    gen = torch.Generator().manual_seed(SEED + 2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist() for n in lens]
    # warm-up: kernels, graphs of a few batch sizes, the library's handles
    engine.generate([prompts[0][:300], prompts[1][:40]], SamplingParams(max_tokens=4, ignore_eos=True))
    # as a server does before it listens: the decode steps' graphs are captured now, not under load
    t_cap = time.perf_counter()
    captured = 0 if args.lazy_graphs else engine.capture_decode_graphs()
    torch.cuda.synchronize()
    t_cap = time.perf_counter() - t_cap
    first, last, gaps, submitted_at = {}, {}, [], {}
    nxt, done = 0, 0
    t0 = time.perf_counter()
    while done < n_req:
        now = time.perf_counter() - t0
        while nxt < n_req and arrivals[nxt] <= now:
            rid = engine.add_request(prompts[nxt], SamplingParams(max_tokens=new_tokens, ignore_eos=True))
            submitted_at[rid] = arrivals[nxt]
            nxt += 1
        if not engine.scheduler.has_work():
            time.sleep(max(0.0, arrivals[nxt] - (time.perf_counter() - t0)))
            continue
        out = engine.step()
        now = time.perf_counter() - t0
        for rid, _tok, finished in out:
            if rid in last:
                gaps.append(now - last[rid])
            else:
                first[rid] = now - submitted_at[rid]
            last[rid] = now
            done += bool(finished)
    wall = time.perf_counter() - t0
    st = engine.stats()

    def pct(v, q):
        v = sorted(v)
        return round(1000.0 * v[min(len(v) - 1, int(q * len(v)))], 2)
    return {"metric": "generated tok/s, continuous batching, Qwen3-%s bf16" % args.shape.upper(), "unit": "tokens/s",
            "value": round(n_req * new_tokens / wall, 1), "wall_s": round(wall, 3), "n_gpus": 1,
            "requests": n_req, "prompt_tokens": sum(lens), "new_tokens": n_req * new_tokens,
            "arrival_rate": args.arrival_rate, "pool_tokens": pool, "max_batch_tokens": args.max_batch_tokens,
            "ttft_ms": {"p50": pct(first.values(), 0.5), "p90": pct(first.values(), 0.9), "p99": pct(first.values(), 0.99)},
            "itl_ms": {"p50": pct(gaps, 0.5), "p90": pct(gaps, 0.9), "p99": pct(gaps, 0.99)},
            "steps": st["steps"], "preemptions": st["preemptions"], "layers": layers,
            "mean_step_ms": round(st["total_step_us"] / max(st["steps"], 1) / 1000.0, 3),   # (the scheduler's own clock)
            "graphs_captured_before": captured, "capture_s": round(t_cap, 2),
            "data": "synthetic: random weights, uniform random token ids, seeded arrivals"}


def main() -> int:
    global CONTEXT, PROMPT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (recorded in config)")
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--workload", default="decode", choices=["decode", "stream"],
                    help="decode: the benchmark (steady decoding at a fixed batch). stream: continuous batching "
                         "under arrivals (64 requests, prompts of 128-4,096 tokens, 256 new tokens each, Poisson "
                         "arrivals); prints its own JSON line")
    ap.add_argument("--arrival-rate", type=float, default=16.0, help="stream: mean arrivals a second")
    ap.add_argument("--lazy-graphs", action="store_true",
                    help="stream: capture each decode graph when a step first needs it, inside the run")
    ap.add_argument("--pool-tokens", type=int, default=0, help="stream: cache pool in tokens (0: room for all)")
    ap.add_argument("--max-batch-tokens", type=int, default=2048,
                    help="stream: new tokens of one step (a decoded token that rides with a prompt portion waits for it)")
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES),
                    help="layer sizes: 8b is the benchmark's; the others are Qwen3-0.6B / 1.7B / 4B / 14B / 32B")
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 / 64 and prefill")
    ap.add_argument("--context", type=int, default=CONTEXT,
                    help="context length the decoding requests reach (the benchmark's is %d; others for measurements "
                         "beside it; the prefill point is a prompt of half of it)" % CONTEXT)
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust project whose GPU path is Apple Metal: pip finds neither setup.py "
                          "nor pyproject.toml, there is no Rust toolchain, and no Metal device on this box"}))
        return 0
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus %d is not supported" % args.gpus)
        return 2
    K, W = max(1, args.steps), max(3, args.warmup)
    CONTEXT, PROMPT = int(args.context), int(args.context) // 2

    import torch
    from velox_b200 import Engine, EngineConfig, Qwen3Config, SamplingParams
    from velox_b200.csrc import ops
    from velox_b200.engine import StepEntry

    model = dict(MODEL, **SHAPES[args.shape])
    layers = args.layers or model["num_hidden_layers"]
    raw = dict(model, num_hidden_layers=layers)
    cfg = Qwen3Config.from_dict(raw)
    pk = peaks()
    if args.workload == "stream":
        with ClockSampler() as clocks:
            res = stream_workload(args, cfg, layers)
        res["clocks"] = clocks.summary()
        print(json.dumps(res))
        return 0
    # the points' largest batch: 64, or what the cache of so many requests at this context leaves room for
    per_token = 2 * layers * cfg.num_key_value_heads * cfg.head_dim * 2
    free_bytes = torch.cuda.mem_get_info()[0] - weight_bytes(raw, layers)
    big = 64
    while big > args.batch and big * (CONTEXT + PAGE) * per_token > 0.8 * free_bytes:
        big //= 2
    max_batch = max(big, args.batch) if not args.skip_points else args.batch
    engine = Engine(model_config=cfg, random_seed=SEED, config=EngineConfig(
        dtype="bfloat16", page_size=PAGE, num_pages=max_batch * (CONTEXT // PAGE + 1) + 8,
        max_running_requests=max_batch, max_batch_tokens=2048, max_model_len=CONTEXT + PAGE))
    gen = torch.Generator().manual_seed(SEED)

    def prompts(n, length):
        return torch.randint(0, cfg.vocab_size, (n, length), generator=gen).tolist()

    def timed(fn, steps):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    def decode_run(batch, steps, warmup, context=None):
        context = context or CONTEXT
        """`batch` requests prefilled so that the timed steps end at the context
        length.  Times `steps` steps through the public entry point (host ids in,
        sampled ids out, every step), then `steps` steps of the step function and
        sampler alone (ids stay on the device).  Returns (ms end to end, ms on the
        device, kernel launches per device step, mean cached tokens per request
        during the device steps)."""
        # Requests whose prompts are done start decoding while the others' prompts
        # are still going in (2,048 new tokens a step), so the first one decodes
        # `stagger` tokens more than the last; it is the one that ends at CONTEXT.
        budget = 2 * steps + warmup + 1
        stagger = -(-batch * context // 2048) + 2 if batch > 1 else 0
        start = context - budget - stagger
        sp = SamplingParams(max_tokens=budget + stagger, ignore_eos=True)
        for p in prompts(batch, start):
            engine.add_request(p, SamplingParams(**vars(sp)))
        while engine.scheduler.waiting or any(engine.cache.length(r) < start for r in engine.scheduler.running):
            engine.step()
        assert len(engine.scheduler.running) == batch, "a request ended during the prompts"
        for _ in range(warmup):
            engine.step()
        e2e_ms = timed(engine.step, steps)
        assert len(engine.scheduler.running) == batch
        entries = [StepEntry(r.request_id, [r.last_token], [0]) for r in engine.scheduler.running.values()]
        zeros, ones = [0.0] * batch, [1.0] * batch
        held = sum(engine.cache.length(r) for r in engine.scheduler.running) / batch

        def device_step():
            engine.runner.step_and_sample(entries, zeros, ones, zeros)
        n0 = ops.launch_count()
        dev_ms = timed(device_step, steps)
        launches = (ops.launch_count() - n0) // steps
        assert max(engine.cache.length(r) for r in engine.scheduler.running) <= context
        for r in list(engine.scheduler.running.values()):
            engine.scheduler._finish(r, "length")
        return e2e_ms, dev_ms, launches, held + steps / 2.0

    out = {"metric": "decode tok/s @ batch %d, Qwen3-%s bf16, context %d" % (args.batch, args.shape.upper(), CONTEXT),
           "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights N(0,0.02) seed 2, uniform random token ids"}

    with ClockSampler() as clocks:
        e2e_ms, ms, launches, kv_mid = decode_run(args.batch, K, W)
    out["clocks"] = clocks.summary()
    out.update({"value": round(args.batch * 1000.0 / ms, 1), "ms_per_step": round(ms, 4),
                "gpu_launches": int(launches * K)})
    # per step through the entry point: the step's description (token ids, positions,
    # block tables, slot mapping) goes up in one pinned copy, the sampled ids come back
    h2d = max(4 * g.host.numel() for (b, _), g in engine.runner.graphs.graphs.items() if b == args.batch)
    out["e2e"] = {"value": round(args.batch * 1000.0 / e2e_ms, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                  "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch}
    nbytes = decode_bytes(raw, layers, args.batch, kv_mid)
    ach = nbytes / (ms * 1e-3) / 1e9
    out["roofline"] = {"bound": "hbm", "achieved": round(ach, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                       "frac": round(ach / pk["hbm_gbs"], 4), "peak_source": pk["source"]}

    if not args.skip_points:
        # prefill: one prompt of 2,048 tokens in one step
        toks = prompts(1, PROMPT)[0]

        last_logits = []

        def one_prefill():
            engine.cache.add_request("prefill")
            last_logits[:] = [engine.run_step([StepEntry("prefill", toks, [PROMPT - 1])])]
            engine.cache.release("prefill")
        for _ in range(3):
            one_prefill()
        pms = timed(one_prefill, 5)
        # a kernel whose bounded wait gave up returns early and would be timed as fast:
        # `run_step` reads the kernels' error word after every step, and the result must be finite
        ops.check_device_errors()
        assert bool(torch.isfinite(last_logits[0]).all()), "the timed prefill gave non-finite logits"
        fl = prefill_flops(raw, layers, PROMPT)
        out["prefill"] = {"value": round(PROMPT * 1000.0 / pms, 1), "tokens": PROMPT, "ms": round(pms, 3),
                          "frac": round(fl / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        pts = {}
        steps = min(K, 32)
        for b in ((1, 32, big) if args.shape == "32b" and big > 32 else (1, big)):
            _, m, _, _ = decode_run(b, steps, 4)
            pts["decode_b%d" % b] = round(b * 1000.0 / m, 1)
        for b in (1, args.batch, big):  # the same with half the context behind each request
            _, m, _, _ = decode_run(b, steps, 4, context=CONTEXT // 2)
            pts["decode_b%d_ctx%d" % (b, CONTEXT // 2)] = round(b * 1000.0 / m, 1)
        out["points"] = pts

    out["config"] = {"model": "Qwen3-%s shape" % args.shape.upper(), "layers": layers,
                     "layers_full": model["num_hidden_layers"],
                     "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                     "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                     "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT, "page_size": PAGE,
                     "parallelism": "single GPU", "l2": "inputs larger than L2 (weights %.0f GB)" % (weight_bytes(raw, layers) / 1e9),
                     "peaks": pk["source"]}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
