"""Token embedding and output head.

x[t] = embed_tokens.weight[id[t]] (src/paged/qwen3.rs:958, 998); logits =
rows W^T with W the head's own matrix, or the embedding table when the two are
tied (src/paged/qwen3.rs:966-976).  The embedding feeds the float32 residual
stream; logits are always float32 (the reference leaves them in the model's
element type, src/paged/qwen3.rs:1015).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from .base import Embedding, Part, Runtime, TensorSpec
from .linear import matmul


class TokenEmbedding(Embedding):
    cuda_graph_safe = True  # reads nothing of a step but device tensors and sizes fixed per graph

    def __init__(self, prefix: str, vocab_size: int, hidden_size: int):
        super().__init__(prefix)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.prefix + "weight", (self.vocab_size, self.hidden_size), "table")]

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        self.weight = tensors[self.prefix + "weight"]

    def forward(self, ctx) -> torch.Tensor:
        return ops.embedding(ctx.token_ids, self.weight)


class OutputHead(Part):
    cuda_graph_safe = True  # reads nothing of a step but device tensors and sizes fixed per graph

    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, tied: bool = False):
        super().__init__(prefix)
        self.vocab_size, self.hidden_size, self.tied = int(vocab_size), int(hidden_size), bool(tied)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        if self.tied:
            return []
        return [TensorSpec(self.prefix + "weight", (self.vocab_size, self.hidden_size), "matrix")]

    def ignored_tensors(self) -> List[str]:
        # a tied checkpoint may still carry a copy of the head
        return [self.prefix + "weight"] if self.tied else []

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        if not self.tied:
            self.weight = tensors[self.prefix + "weight"]

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table

    def forward(self, rows: torch.Tensor) -> torch.Tensor:
        return matmul(rows, self.weight, None, torch.float32)
