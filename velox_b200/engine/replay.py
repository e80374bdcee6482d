"""Trace replay: feeds given token ids through the model step by step and writes
logits.  It samples nothing, and it has no forward pass, cache or loader of its
own: it drives the engine's `ModelRunner.step`, cache manager and kernels, the
ones generation uses.

Steps come on standard input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, `<out>/<step>.f32` gets the logits at the
wanted places, in the order of the entries and of `want`, as little-endian float32
[wanted, vocab].  After every step a line `done <step>` is printed and flushed.
The reference has no such tool; its nearest code is the hand-rolled decode loop
of tests/spec_decode.rs:65-116.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--max-requests", type=int, default=8, help="requests that may be live at once")
    ap.add_argument("--poison-cache", action="store_true",
                    help="fill the cache pool with NaN first, so that a read of a stale or foreign slot shows")
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    if args.max_tokens <= 0 or 64 % args.page_size:
        sys.stderr.write("trace_run: --max-tokens must be positive and --page-size must divide 64\n")
        return 2
    os.makedirs(args.out, exist_ok=True)
    sys.stderr.write("[velox_b200] trace_run: preparing kernels and model\n")
    sys.stderr.flush()
    from ..csrc import ops
    ops.library()  # compiles at the first call of a fresh checkout; prints progress
    from ..config.engine_config import EngineConfig
    from .batch import StepEntry
    from .engine import Engine

    pool_tokens = -(-args.max_tokens // 64) * 64
    cfg = EngineConfig(dtype=args.dtype, page_size=args.page_size, max_cache_tokens=pool_tokens,
                       max_running_requests=args.max_requests, max_model_len=pool_tokens)
    engine = Engine(args.model, cfg, poison_cache=args.poison_cache)
    runner, cache = engine.runner, engine.cache
    sys.stderr.write("[velox_b200] trace_run: ready (%s, %d pages of %d tokens per group)\n"
                     % (args.dtype, cache.groups[0].allocator.num_pages if cache.groups else 0, args.page_size))
    sys.stderr.flush()

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if not cache.has_request(rid):
                if cache.add_request(rid) is None:
                    raise RuntimeError("step %r: more than %d live requests" % (step, args.max_requests))
            entries.append(StepEntry(rid, [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        if entries:
            logits = runner.step(entries)
            if logits is not None:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, "%s.f32.tmp" % step)
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, "%s.f32" % step))
        for rid in rec.get("end", []):
            if cache.has_request(rid):
                cache.release(rid)
        runner.check_errors()
        sys.stdout.write("done %s\n" % step)
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
