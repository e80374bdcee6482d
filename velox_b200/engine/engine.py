"""The engine: a model on one GPU with its cache, step function, scheduler and
sampler, and the Python entry point for generation.

    engine = Engine("path/to/model", EngineConfig(dtype="bfloat16"))
    outputs = engine.generate([[1, 2, 3], [4, 5]], SamplingParams(max_tokens=8))

The model class is chosen by config.json through the architecture registry; the
reference's loader does the same from `model_type` (src/backend/candle.rs:126-195).
Its pool is fixed at 256 pages of 16 tokens (src/backend/candle.rs:158-165); here
the pool is sized from `EngineConfig` or from the memory that is free.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import models as _models  # noqa: F401  (registers architectures)
from ..cache.manager import CacheManager
from ..config.engine_config import EngineConfig
from ..config.model_config import ModelConfig
from ..config.registry import load_config, resolve_architecture
from ..models.decoder import DecoderModel
from ..cache.kinds import cache_kind
from ..parts.base import Runtime
from ..sampling.params import SamplingParams
from ..sampling.rng import uniform
from ..weights.loader import load_weights
from ..weights.random_init import bind_random_weights
from .batch import StepEntry
from .scheduler import Request, Scheduler
from .step import ModelRunner

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _eos_ids(folder: Optional[str], raw: Dict) -> List[int]:
    """End-of-sequence ids: the union of what generation_config.json and
    config.json name (the reference also asks the tokenizer's files,
    src/backend/candle.rs:570-598; there is no tokenizer here)."""
    found: List[int] = []
    sources = [raw]
    if folder:
        p = os.path.join(folder, "generation_config.json")
        if os.path.isfile(p):
            with open(p) as f:
                sources.append(json.load(f))
    for src in sources:
        v = src.get("eos_token_id")
        for x in (v if isinstance(v, list) else [v]):
            if isinstance(x, int) and x not in found:
                found.append(x)
    return found


class Engine:
    def __init__(self, model_dir: Optional[str] = None, config: Optional[EngineConfig] = None, *,
                 model_config: Optional[ModelConfig] = None, random_seed: Optional[int] = None,
                 poison_cache: bool = False, cache_memory_limit: Optional[int] = None):
        """Loads `model_dir` (config.json + safetensors).  Without a folder, a
        typed `model_config` and a `random_seed` give a model with random
        weights made on the device."""
        self.config = config or EngineConfig()
        self.cache_memory_limit = cache_memory_limit
        if not torch.cuda.is_available():
            raise RuntimeError("velox_b200 runs on a CUDA device (sm_100a); none is visible")
        self.device = torch.device(self.config.device)
        torch.cuda.set_device(self.device)
        self.runtime = Runtime(_TORCH_DTYPES[self.config.dtype], self.device)
        if model_dir is not None:
            self.architecture, self.model_config = load_config(model_dir)
            with open(os.path.join(model_dir, "config.json")) as f:
                raw = json.load(f)
        else:
            if model_config is None or random_seed is None:
                raise ValueError("give a model folder, or a model_config with a random_seed")
            self.model_config = model_config
            raw = model_config.to_dict()
            self.architecture = resolve_architecture(raw)
        self.plan = self.architecture.plan(self.model_config)
        self.model = DecoderModel(self.plan)
        if model_dir is not None:
            load_weights(self.model, model_dir, self.runtime)
        else:
            bind_random_weights(self.model, self.runtime, int(random_seed))
        self.eos_token_ids = _eos_ids(model_dir, raw)
        self.last_finish_reasons: List[Optional[str]] = []  # of the latest `generate`, per prompt
        # called after every step that sampled, with (request ids, float32 logits [sampled, vocab]
        # on the device): the rows the step's tokens were drawn from
        self.on_logits = None

        cfg = self.config
        self.max_model_len = int(cfg.max_model_len or self.plan.max_positions or 4096)
        S = cfg.page_size
        max_blocks = -(-self.max_model_len // S)
        specs = self.model.cache_specs()
        num_pages = self._pool_pages(specs, max_blocks)
        self.cache = CacheManager(specs, self.model.cache_sources(), S, num_pages,
                                  cfg.max_running_requests, max_blocks, self.runtime.dtype, self.device,
                                  poison=poison_cache)
        self.runner = ModelRunner(self.model, self.cache, self.device, self.plan.vocab_size,
                                  cuda_graphs=cfg.cuda_graphs)
        self.scheduler = Scheduler(self.cache, cfg.max_running_requests, cfg.max_batch_tokens, cfg.chunk_size,
                                   self.max_model_len)

    def _pool_pages(self, specs, max_blocks: int) -> int:
        cfg = self.config
        if cfg.num_pages:
            return int(cfg.num_pages)
        if cfg.max_cache_tokens:
            return -(-int(cfg.max_cache_tokens) // cfg.page_size)
        elt = 2 if self.runtime.dtype == torch.bfloat16 else 4
        kinds = [(cache_kind(s), s) for s in specs if s is not None]
        per_page = sum(k.page_bytes(s, cfg.page_size, elt) for k, s in kinds if k.paged)
        wanted = cfg.max_running_requests * max_blocks
        if per_page == 0:
            return max(1, min(wanted, 1024))
        free, _ = torch.cuda.mem_get_info(self.device)
        room = int(free * 0.85)
        if self.cache_memory_limit is not None:
            room = min(room, int(self.cache_memory_limit))
        return max(1, min(wanted, room // per_page))

    # -- requests ---------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        params = params or SamplingParams()
        if not params.eos_token_ids and self.eos_token_ids:
            params.eos_token_ids = list(self.eos_token_ids)
        vocab = self.plan.vocab_size
        for t in prompt:
            if not 0 <= int(t) < vocab:
                raise ValueError("token id %r outside [0, %d)" % (t, vocab))
        return self.scheduler.submit(prompt, params)

    def step(self) -> List[Tuple[int, int, bool]]:
        """One scheduler step: (request id, new token, finished) per request that
        got a token."""
        entries, _ended = self.scheduler.plan()
        if not entries:
            return []
        temps, tops, us = [], [], []
        for e in entries:
            if not e.want:
                continue
            p = self.scheduler.params_of(e.request_id)
            if p.greedy:
                temps.append(0.0)
                tops.append(1.0)
                us.append(0.0)
                continue
            temps.append(p.temperature)
            tops.append(p.top_p if p.nucleus else 1.0)
            # one uniform number per (request, token): the same sequence whatever the batching
            seed = p.seed if p.seed is not None else self.config.seed * 1000003 + e.request_id
            us.append(uniform(seed, 0, self.scheduler.request(e.request_id).num_generated))
        logits, ids = self.runner.step_and_sample(entries, temps, tops, us)
        sampled: List[int] = ids.tolist() if ids is not None else []
        if self.on_logits is not None and logits is not None:
            # (a captured step's logits live in the graph's buffer until the next step only)
            self.on_logits([e.request_id for e in entries if e.want], logits[:len(sampled)])
        self.runner.check_errors()
        return self.scheduler.update(entries, sampled)

    def capture_decode_graphs(self, max_batch: Optional[int] = None, max_tokens: Optional[int] = None) -> int:
        """Captures the decode steps' graphs for up to `max_batch` requests (default:
        `max_running_requests`) of up to `max_tokens` tokens each (default: the longest
        a request may get) before the first request comes, instead of one by one
        when a step first needs them.  Returns how many were captured."""
        if self.runner.graphs is None:
            return 0
        return self.runner.graphs.capture_all(max_batch or self.scheduler.max_running_requests,
                                              max_tokens or self.scheduler.max_model_len)

    def run_step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """The raw step function, for callers that schedule themselves."""
        logits = self.runner.step(entries)
        self.runner.check_errors()
        return logits

    def generate(self, prompts: Sequence[Sequence[int]], params=None) -> List[List[int]]:
        """Generates for every prompt (host token ids in, host token ids out).
        `params`: one `SamplingParams` for all, or one per prompt."""
        if params is None or isinstance(params, SamplingParams):
            plist = [SamplingParams(**vars(params)) if params else SamplingParams() for _ in prompts]
        else:
            plist = list(params)
            if len(plist) != len(prompts):
                raise ValueError("%d prompts but %d sampling params" % (len(prompts), len(plist)))
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, plist)]
        while self.scheduler.has_work():
            self.step()
        outs, self.last_finish_reasons = [], []
        for i in ids:
            r = self.scheduler.finished[i]
            outs.append(list(r.generated))
            self.last_finish_reasons.append(r.finish_reason)
            # the record is dropped once its tokens are read (the reference drops a
            # request when it finishes, src/paged/scheduler.rs:505-520), so an engine
            # that lives long does not grow
            self.scheduler.forget(i)
        return outs

    def cancel(self, request_id: int) -> bool:
        """Withdraws a request that waits or runs (between two calls of `step`): what
        it holds of the cache is free at once, its finish reason is "cancelled".
        False if it had finished already."""
        return self.scheduler.cancel(request_id)

    def request(self, request_id: int) -> Request:
        return self.scheduler.request(request_id)

    def stats(self) -> Dict:
        d = dict(vars(self.scheduler.stats))
        d["free_pages"] = self.cache.free_pages()
        d["running"] = len(self.scheduler.running)
        d["waiting"] = len(self.scheduler.waiting)
        return d
