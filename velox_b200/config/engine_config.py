"""Settings of the engine around a model: precision, cache pool, scheduler limits.

The scheduler limits carry the names and meanings of the reference's
`SchedulerConfig` (src/paged/scheduler.rs:37-60): `max_running_requests` caps the
requests that hold cache at once, `max_batch_tokens` caps the new tokens of one
step.  The reference fixes its pool at 256 pages of 16 tokens
(src/backend/candle.rs:158-165); here the pool is sized by the caller.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

DTYPE_NAMES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32", "f32": "float32"}


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"
    device: str = "cuda:0"
    page_size: int = 16
    # Size of the pool: either pages for every group, or a token capacity that
    # each group's page count is derived from.
    num_pages: Optional[int] = None
    max_cache_tokens: Optional[int] = None
    max_running_requests: int = 64
    max_batch_tokens: int = 2048
    # A fixed portion size for prompts (None: whatever the budget leaves).
    chunk_size: Optional[int] = None
    # Longest sequence a request may reach; None: max_position_embeddings.
    max_model_len: Optional[int] = None
    # Capture decode-only steps in CUDA graphs.
    cuda_graphs: bool = True
    seed: int = 0

    def __post_init__(self) -> None:
        if self.dtype not in DTYPE_NAMES:
            raise ValueError("dtype %r is not one of %s" % (self.dtype, sorted(set(DTYPE_NAMES))))
        self.dtype = DTYPE_NAMES[self.dtype]
        if self.page_size <= 0:
            raise ValueError("page_size must be positive")
        if self.max_running_requests <= 0:
            raise ValueError("max_running_requests must be positive")
        if self.max_batch_tokens <= 0:
            raise ValueError("max_batch_tokens must be positive")
        if self.chunk_size is not None and self.chunk_size <= 0:
            raise ValueError("chunk_size must be positive")
