"""A decoder put together from a `ModelPlan`: embedding, blocks in the plan's
running order, final norm, output head.  Which architecture the plan came from
is not known here.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..parts.base import Part, Runtime, TensorSpec
from ..parts.plan import ModelPlan
from ..parts.registry import build_part, part_class


class DecoderModel:
    def __init__(self, plan: ModelPlan):
        plan.validate()
        self.plan = plan
        self.embedding = build_part("embedding", plan.embedding)
        self.blocks = []
        for spec in plan.layers:
            block_cls = part_class("block", spec.block)
            self.blocks.append(block_cls(
                build_part("mixer", spec.mixer) if spec.mixer is not None else None,
                build_part("feed_forward", spec.feed_forward) if spec.feed_forward is not None else None,
                {name: build_part("norm", n) for name, n in spec.norms.items()}))
        self.final_norm = build_part("norm", plan.final_norm)
        self.head = build_part("head", plan.head)
        self.order = plan.running_order()
        self.runtime: Optional[Runtime] = None

    # -- weights -------------------------------------------------------------
    def parts(self) -> List[Part]:
        out: List[Part] = [self.embedding]
        for b in self.blocks:
            out.extend(b.parts())
        out.extend([self.final_norm, self.head])
        return out

    def tensor_specs(self) -> List[TensorSpec]:
        return [s for p in self.parts() for s in p.tensor_specs()]

    def ignored_tensors(self) -> List[str]:
        return [n for p in self.parts() for n in p.ignored_tensors()]

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        for p in self.parts():
            p.bind(tensors, runtime)
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding.weight)

    # -- cache ---------------------------------------------------------------
    # Caches belong to the places of the running order, not to layers: a layer
    # that the order names twice shares its weights between the two places, but
    # each place keeps keys, values or state of its own, so that a position's
    # result does not depend on how the tokens were cut into steps.
    def cache_specs(self) -> list:
        """Per place of the running order: the mixer's cache need, or None for a
        place without a cache of its own (none at all, or another's)."""
        return [None if self.plan.layers[i].cache_of is not None or self.blocks[i].mixer is None
                else self.blocks[i].mixer.cache_spec() for i in self.order]

    def cache_sources(self) -> list:
        """Per place of the running order: None, or the earlier place whose cache
        it reads (the latest earlier run of layer `cache_of`)."""
        out = []
        for k, i in enumerate(self.order):
            j = self.plan.layers[i].cache_of
            if j is None:
                out.append(None)
                continue
            earlier = [m for m in range(k) if self.order[m] == j]
            if not earlier:
                raise ValueError("layer %d reads the cache of layer %d, which has not run before it" % (i, j))
            out.append(earlier[-1])
        return out

    # -- step ----------------------------------------------------------------
    def forward_hidden(self, ctx, cache):
        """Runs the step's tokens through every layer; returns (residual, delta),
        whose sum is the last layer's output [tokens, hidden]."""
        residual = self.embedding.forward(ctx)
        delta = None
        for place, i in enumerate(self.order):
            residual, delta = self.blocks[i].forward(residual, delta, ctx, cache.layer(place))
        return residual, delta

    def logits(self, residual, delta, rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [len(rows), vocab] at the given token rows (int32)."""
        h = self.final_norm.add_norm(residual, delta, rows=rows)
        return self.head.forward(h)
