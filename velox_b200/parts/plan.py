"""The description of a model as data: which parts each layer is made of, and
the order in which layers run.

A `ModelPlan` is what an architecture's plan function makes out of its typed
configuration.  It names parts by kind (looked up in `parts.registry`) and gives
each its sizes and constants as parameters, layer by layer, so that one model
can have different mixers and feed-forwards in different layers.  `order` is the
list of layer indices in running order; it may name a layer twice: the two runs
share the layer's weights, and each has a cache of its own.  A layer with
`cache_of = j` keeps no cache and reads (and does not write) the cache that the
latest earlier run of layer j filled.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass(frozen=True)
class PartSpec:
    kind: str
    # prefix of this part's tensor names in the weight file, e.g.
    # "model.layers.3.self_attn."
    prefix: str = ""
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """A layer: a mixer, a feed-forward (or none), and its norms by the names that
    its block arrangement gives them ("mixer" and "feed_forward" in the pre-norm
    block; another arrangement may ask for one, four or none)."""
    mixer: Optional[PartSpec]
    feed_forward: Optional[PartSpec] = None
    norms: Dict[str, PartSpec] = field(default_factory=dict)
    block: str = "pre_norm"
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    vocab_size: int
    hidden_size: int
    embedding: PartSpec
    layers: List[LayerSpec]
    final_norm: PartSpec
    head: PartSpec
    order: List[int] = field(default_factory=list)
    max_positions: int = 0

    def running_order(self) -> List[int]:
        return list(self.order) if self.order else list(range(len(self.layers)))

    def validate(self) -> None:
        n = len(self.layers)
        for i in self.running_order():
            if not 0 <= i < n:
                raise ValueError("order names layer %d but the plan has %d layers" % (i, n))
        for i, layer in enumerate(self.layers):
            j = layer.cache_of
            if j is None:
                continue
            if not 0 <= j < n or j == i:
                raise ValueError("layer %d reads the cache of layer %r" % (i, j))
            if self.layers[j].cache_of is not None:
                raise ValueError("layer %d reads the cache of layer %d, which has none of its own" % (i, j))
            order = self.running_order()
            if i in order and (j not in order or order.index(j) > order.index(i)):
                raise ValueError("layer %d runs before layer %d, whose cache it reads" % (i, j))
