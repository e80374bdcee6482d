"""Per-request sampling options, with the names and meanings of the reference's
`GenerateRequest` (src/backend/traits.rs:30-40) where it has them:
`max_tokens` (at least 1), `temperature` (clamped to >= 0; <= 1e-7 means
greedy, src/paged/scheduler.rs:545-559), `top_p` (clamped to [0, 1]; <= 0 or
>= 1 means the whole distribution, src/paged/scheduler.rs:547-551).  The
reference seeds a fresh sampler from the system's entropy for every row of every
step (src/paged/scheduler.rs:545-553, 619), which cannot be repeated; here a
request has a `seed`, and the same seed gives the same tokens.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

GREEDY_BELOW = 1e-7


@dataclass
class SamplingParams:
    max_tokens: int = 16
    temperature: float = 0.0
    top_p: float = 1.0
    seed: Optional[int] = None
    # generation stops after one of these tokens (it is kept, as in the
    # reference: src/paged/scheduler.rs:426, 465-470)
    eos_token_ids: List[int] = field(default_factory=list)
    stop_token_ids: List[int] = field(default_factory=list)
    # ... or after a run of generated tokens that equals one of these.  The
    # reference's `stop_sequences` are strings searched in the decoded text
    # (src/backend/traits.rs:39, src/backend/candle.rs:798-799); the engine sees
    # token ids only, so these are runs of token ids.
    stop_sequences: List[List[int]] = field(default_factory=list)
    ignore_eos: bool = False

    def __post_init__(self) -> None:
        self.max_tokens = max(1, int(self.max_tokens))
        self.temperature = max(0.0, float(self.temperature))
        self.top_p = min(1.0, max(0.0, float(self.top_p)))

    @property
    def greedy(self) -> bool:
        return self.temperature <= GREEDY_BELOW

    @property
    def nucleus(self) -> bool:
        return 0.0 < self.top_p < 1.0
