"""Turns rows of logits into tokens: greedy, temperature, temperature + top-p,
mixed freely within a batch, in one kernel launch and one small copy back.

The reference takes one device argmax when every row is greedy and otherwise
copies whole rows to the host and samples there (src/paged/scheduler.rs:591-625).
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..csrc import ops
from .params import SamplingParams
from .rng import uniform


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               counters: Sequence[int]) -> List[int]:
        """One token per row.  `seeds[i]`, `counters[i]`: the row's request seed
        and how many tokens that request has sampled before."""
        n = logits.shape[0]
        if n == 0:
            return []
        if all(p.greedy for p in params):
            ids = ops.sample(logits)
        else:
            host = torch.empty((3, n), dtype=torch.float32, pin_memory=self.device.type == "cuda")
            for i, p in enumerate(params):
                host[0, i] = 0.0 if p.greedy else p.temperature
                host[1, i] = p.top_p if p.nucleus else 1.0
                host[2, i] = uniform(seeds[i], 0, counters[i])
            dev = host.to(self.device, non_blocking=True)
            ids = ops.sample(logits, dev[0], dev[1], dev[2])
        return ids.tolist()
