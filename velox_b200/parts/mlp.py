"""The gated feed-forward of Qwen3: down(act(gate(x)) * up(x)), never biased
(src/paged/qwen3.rs:313-340).  Gate and up are one matrix here, which the
reference keeps apart (:334-336): its rows come in tiles of 16, 8 gate rows
followed by the 8 up rows of the same features, so that a matrix-product kernel
that owns a tile holds gate and up of a feature together and can apply
act(gate) * up before anything is written (if the intermediate size is no
multiple of 8, all gate rows are followed by all up rows and the product is taken
by a kernel of its own).  Activation and product are formed in float32.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from .base import FeedForward, Runtime, TensorSpec
from .linear import Linear


GATE_TILE = 8
FUSED_TCGEN05_MIN_ROWS = 128


class GatedMLP(FeedForward):
    cuda_graph_safe = True  # reads nothing of a step but device tensors and sizes fixed per graph

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
        gate, up = tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]
        i, e = self.intermediate_size, self.hidden_size
        if i % GATE_TILE == 0:
            self.tile = GATE_TILE
            w = torch.stack([gate.view(i // GATE_TILE, GATE_TILE, e), up.view(i // GATE_TILE, GATE_TILE, e)], 1)
            self.gate_up = Linear(w.reshape(2 * i, e).contiguous())
        else:
            self.tile = 0
            self.gate_up = Linear(torch.cat([gate, up], 0).contiguous())
        self.down = Linear(tensors[p + "down_proj.weight"])

    def forward(self, h: torch.Tensor, ctx=None) -> torch.Tensor:
        w = self.gate_up.weight
        fused = self.tile and h.dtype == torch.bfloat16
        if fused and ops.skinny_supported(h.shape[0], h.shape[1], h, w):
            # a decode step: W streamed once, act(gate) * up taken on the accumulators
            a = ops.gemm_skinny(h, w, None, h.dtype, gated_activation=self.activation)
        elif fused and h.shape[0] >= FUSED_TCGEN05_MIN_ROWS and ops.tcgen05_supported(h, w):
            # a prompt portion: tcgen05 product with the same epilogue (measured no slower than
            # the library product followed by the activation kernel from 128 rows, faster from 512)
            a = ops.gemm_tcgen05(h, w, None, gated_activation=self.activation,
                                 pair=ops.tcgen05_pair_better(h.shape[0], w.shape[0], h.device))
        elif h.dtype == torch.bfloat16:
            # the library product hands over its float32 sums: gate and up are not rounded
            # before the activation, as in the fused kernels
            a = ops.gated_act(self.gate_up(h, torch.float32), self.activation, self.tile, out_dtype=h.dtype)
        else:
            a = ops.gated_act(self.gate_up(h), self.activation, self.tile)
        return self.down(a)
