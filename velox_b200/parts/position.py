"""Position encodings that a mixer applies to its queries and keys.

`RotaryPosition`: the half-split rotation of the reference
(src/paged/metal_kernels.rs:199-202, 230-236): pairs (i, i + rot/2) turned by
position * inv_freq[i], inv_freq[i] = 1 / theta^(2i/rot), the power taken in
float64 and the quotient in float32 as the reference does
(src/paged/qwen3.rs:281-284).  The reference then tabulates cosines and sines
and rounds the table to the model's element type (src/paged/qwen3.rs:287-293);
here angle, sine and cosine are float32 inside the kernel and never rounded.

`NoPosition`: nothing is applied.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from .base import Position


class RotaryPosition(Position):
    cuda_graph_safe = True

    def __init__(self, prefix: str = "", head_dim: int = 0, theta: float = 10000.0, rotary_dim: Optional[int] = None):
        super().__init__(prefix)
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.rotary_dim = int(rotary_dim) if rotary_dim else self.head_dim
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError("rotary_dim %d must be even and within head_dim %d" % (self.rotary_dim, self.head_dim))
        self._table = {}

    def inverse_frequencies(self) -> np.ndarray:
        r = self.rotary_dim
        vals = [np.float32(1.0) / np.float32(self.theta ** (i / r)) for i in range(0, r, 2)]
        return np.asarray(vals, dtype=np.float32)

    def rotary_table(self, device) -> Optional[Tuple[torch.Tensor, int]]:
        key = str(device)
        if key not in self._table:
            self._table[key] = torch.from_numpy(self.inverse_frequencies()).to(device)
        return self._table[key], self.rotary_dim


class NoPosition(Position):
    cuda_graph_safe = True

    def __init__(self, prefix: str = "", **_ignored):
        super().__init__(prefix)
