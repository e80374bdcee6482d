"""RMSNorm: x * rsqrt(mean(x^2) + eps) * weight, statistics in float32.

The reference calls its tensor library's rms_norm with `rms_norm_eps`
(src/paged/qwen3.rs:923-928, 933, 936); the weight multiplies, with no offset.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from .base import Norm, Runtime, TensorSpec


class RMSNorm(Norm):
    cuda_graph_safe = True  # reads nothing of a step but device tensors and sizes fixed per graph

    def __init__(self, prefix: str, size: int, eps: float):
        super().__init__(prefix)
        self.size, self.eps = int(size), float(eps)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.prefix + "weight", (self.size,), "norm")]

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        self.weight = tensors[self.prefix + "weight"]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps)

    def add_norm(self, residual, delta, rows=None):
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, self.runtime.dtype, rows=rows)
