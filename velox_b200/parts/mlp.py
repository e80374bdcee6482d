"""The gated feed-forward of Qwen3: down(act(gate(x)) * up(x)), never biased
(src/paged/qwen3.rs:313-340).  Gate and up are one matrix here ([Wgate; Wup],
the gate rows first), which the reference keeps apart (:334-336); activation
and product are formed in float32.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from .base import FeedForward, Runtime, TensorSpec
from .linear import Linear


class GatedMLP(FeedForward):
    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, activation: str = "silu"):
        super().__init__(prefix)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        if activation not in ops.ACTIVATIONS:
            raise ValueError("activation %r is not one of %s" % (activation, sorted(ops.ACTIVATIONS)))
        self.activation = activation
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def tensor_specs(self) -> List[TensorSpec]:
        p, e, i = self.prefix, self.hidden_size, self.intermediate_size
        return [TensorSpec(p + "gate_proj.weight", (i, e), "matrix"),
                TensorSpec(p + "up_proj.weight", (i, e), "matrix"),
                TensorSpec(p + "down_proj.weight", (e, i), "matrix")]

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        p = self.prefix
        self.gate_up = Linear(torch.cat([tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]], 0).contiguous())
        self.down = Linear(tensors[p + "down_proj.weight"])

    def forward(self, h: torch.Tensor, ctx=None) -> torch.Tensor:
        return self.down(ops.gated_act(self.gate_up(h), self.activation))
