"""Command line: `python -m velox_b200 <command>` (or `bin/velox`).

The reference's binary has `pull` (fetch a model into --model-dir) and `serve`
(src/main.rs:18-78).  There is no network and no server here, so:

  random-model   stands where `pull` stands: puts a model into --model-dir, made
                 from a config.json and a seed instead of downloaded;
  generate       stands where `serve` stands: runs requests through the same
                 scheduler and engine, read from the command line instead of HTTP.

Options keep the reference's names and meanings where it has them:
--model-dir (directory that holds models, each in a folder of its own;
src/main.rs:30-31, 42-43), --max-concurrent (requests served at once,
src/main.rs:58-60), --max-model-memory ("auto", "32GB", "80%"; src/main.rs:49-51;
here it bounds the cache pool), and per request max_tokens, temperature, top_p,
prompt_tokens (src/backend/traits.rs:30-40).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional


def _model_folder(model_dir: str, model: Optional[str]) -> str:
    model_dir = os.path.expanduser(model_dir)
    if model:
        cand = os.path.join(model_dir, model)
        if not os.path.isfile(os.path.join(cand, "config.json")):
            raise SystemExit("no model %r in %s (no config.json in %s)" % (model, model_dir, cand))
        return cand
    if os.path.isfile(os.path.join(model_dir, "config.json")):
        return model_dir
    found = sorted(d for d in os.listdir(model_dir) if os.path.isfile(os.path.join(model_dir, d, "config.json"))) \
        if os.path.isdir(model_dir) else []
    if len(found) == 1:
        return os.path.join(model_dir, found[0])
    raise SystemExit("--model-dir %s holds %d models %s; name one with --model" % (model_dir, len(found), found))


def _memory_bytes(text: str, device) -> Optional[int]:
    """"auto" -> None; "32GB" -> bytes; "80%" -> that share of the device's free memory."""
    import torch
    t = text.strip().lower()
    if t == "auto":
        return None
    if t.endswith("%"):
        free, _ = torch.cuda.mem_get_info(device)
        return int(free * float(t[:-1]) / 100.0)
    for suffix, mul in (("gb", 1 << 30), ("mb", 1 << 20), ("g", 1 << 30), ("m", 1 << 20)):
        if t.endswith(suffix):
            return int(float(t[: -len(suffix)]) * mul)
    return int(t)


def _ints(text: str) -> List[int]:
    return [int(x) for x in text.replace(" ", "").split(",") if x]


def cmd_random_model(args) -> int:
    from . import models  # noqa: F401
    from .config.registry import resolve_architecture
    from .weights import write_random_model
    with open(args.config) as f:
        raw = json.load(f)
    arch = resolve_architecture(raw)
    cfg = arch.config_class.from_dict(raw)
    out = os.path.join(os.path.expanduser(args.model_dir), args.model) if args.model else os.path.expanduser(args.model_dir)
    write_random_model(out, cfg, args.seed, dtype=args.store_dtype)
    print(json.dumps({"model": out, "architecture": arch.name, "seed": args.seed}))
    return 0


def cmd_generate(args) -> int:
    import numpy as np
    import torch
    from . import Engine, EngineConfig, SamplingParams
    folder = _model_folder(args.model_dir, args.model)
    prompts: List[List[int]] = [_ints(p) for p in (args.prompt_tokens or [])]
    if args.prompt_lens:
        with open(os.path.join(folder, "config.json")) as f:
            vocab = json.load(f)["vocab_size"]
        rng = np.random.default_rng(args.prompt_seed)
        prompts += [[int(t) for t in rng.integers(0, vocab, n)] for n in _ints(args.prompt_lens)]
    if not prompts:
        raise SystemExit("give --prompt-tokens 1,2,3 (repeatable) or --prompt-lens 5,11,17")
    cfg = EngineConfig(dtype=args.dtype, device=args.device, page_size=args.page_size, num_pages=args.num_pages,
                       max_running_requests=args.max_concurrent, max_batch_tokens=args.max_batch_tokens,
                       chunk_size=args.chunk_size, max_model_len=args.max_model_len, seed=args.seed)
    limit = _memory_bytes(args.max_model_memory, torch.device(args.device))
    engine = Engine(folder, cfg, cache_memory_limit=limit)
    stops = [[int(t) for t in q.split(",") if t.strip()] for q in (args.stop or [])]
    params = [SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, top_p=args.top_p,
                             seed=None if args.seed is None else args.seed + i, ignore_eos=args.ignore_eos,
                             stop_sequences=[list(q) for q in stops])
              for i in range(len(prompts))]
    dumped, dump_index = [], []
    if args.dump_logits:
        def keep_logits(request_ids, logits):
            dumped.append(logits.detach().to("cpu").numpy().astype("<f4"))
            dump_index.extend(int(r) for r in request_ids)
        engine.on_logits = keep_logits
    outs = engine.generate(prompts, params)
    if args.dump_logits:
        # rows in the order the tokens were sampled; FILE.json says whose each row is
        (np.concatenate(dumped) if dumped else np.zeros((0, 0), "<f4")).tofile(args.dump_logits)
        with open(args.dump_logits + ".json", "w") as f:
            json.dump({"dtype": "<f4", "rows": len(dump_index), "request_of_row": dump_index}, f)
    for i, (p, o, why) in enumerate(zip(prompts, outs, engine.last_finish_reasons)):
        print(json.dumps({"request": i, "prompt_tokens": len(p), "tokens": o, "finish_reason": why}))
    if args.stats:
        sys.stderr.write(json.dumps(engine.stats()) + "\n")
    return 0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="velox", description="velox_b200: a Qwen3 inference engine for one B200")
    sub = ap.add_subparsers(dest="command", required=True)

    rm = sub.add_parser("random-model", help="write a model folder with random weights into --model-dir")
    rm.add_argument("--config", required=True, help="a config.json of a registered architecture")
    rm.add_argument("--model-dir", default="~/.velox/models", help="where models live, each in <dir>/<model>")
    rm.add_argument("--model", default=None, help="folder name under --model-dir (default: --model-dir itself)")
    rm.add_argument("--seed", type=int, default=0)
    rm.add_argument("--store-dtype", choices=["bfloat16", "float32"], default="bfloat16")
    rm.set_defaults(fn=cmd_random_model)

    g = sub.add_parser("generate", help="generate tokens for prompts given as token ids")
    g.add_argument("--model-dir", default="~/.velox/models", help="a model folder, or a directory of them")
    g.add_argument("--model", default=None, help="which model of --model-dir")
    g.add_argument("--max-model-memory", default="auto", help='memory for the cache pool: "auto", "32GB", "80%%"')
    g.add_argument("--max-concurrent", type=int, default=8, help="requests that run at once")
    g.add_argument("--prompt-tokens", action="append", help="comma-separated token ids; may be given several times")
    g.add_argument("--prompt-lens", default=None, help="comma-separated lengths of random prompts")
    g.add_argument("--prompt-seed", type=int, default=0)
    g.add_argument("--max-tokens", type=int, default=16)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=0, help="sampling seed (request i uses seed + i)")
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--stop", action="append", help="comma-separated token ids; generation stops after this run of "
                                                    "tokens (may be given several times)")
    g.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    g.add_argument("--device", default="cuda:0")
    g.add_argument("--page-size", type=int, default=16)
    g.add_argument("--num-pages", type=int, default=None)
    g.add_argument("--max-batch-tokens", type=int, default=2048)
    g.add_argument("--chunk-size", type=int, default=None)
    g.add_argument("--max-model-len", type=int, default=None)
    g.add_argument("--dump-logits", default=None, metavar="FILE",
                   help="write the float32 logits every token was sampled from to FILE ([rows, vocab], in sampling "
                        "order) and the request of each row to FILE.json")
    g.add_argument("--stats", action="store_true", help="print the scheduler's counters to stderr at the end")
    g.set_defaults(fn=cmd_generate)
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
