"""Interfaces of the parts a layer is put together from.

A part is built from a `PartSpec`: its kind picks the class, `prefix` is where
its tensors live in the weight file, `params` are its sizes and constants.  No
part knows which model it is in.

    Part          tensor_specs() -> what it wants from the weight file
                  bind(tensors, runtime) -> takes them (already on the device)
    Norm          forward(x) ; add_norm(residual, delta) -> normed
    Position      an encoding of positions that a mixer applies to q and k
    Mixer         cache_spec() -> PagedKV | FixedState | a spec of a registered cache kind | None
                  forward(h, ctx, cache) -> y          h, y: [tokens, hidden]
    FeedForward   forward(h, ctx) -> y
    Block         forward(residual, delta, ctx, cache) -> (residual, delta)
                  built from a mixer, a feed-forward (or None) and norms by name
    Embedding     forward(ctx) -> float32 residual [tokens, hidden]

`h` and `y` have the engine's element type; the residual stream is float32.
`ctx` is the step's `StepContext` (engine/batch.py): positions, which request
each token belongs to, block tables and slot mappings per cache group, state
slots.  `cache` is the layer's `LayerCache` (cache/kinds.py).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part wants.  `role` decides how random weights are drawn and
    in which element type the tensor is held:
      matrix, table: N(0, 0.02); held in the engine's element type
      norm:          1 + N(0, 0.05); held in float32 (an exact widening)
      bias:          N(0, 0.02); held in float32
      int_table:     integers; held as int32"""
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"


@dataclass(frozen=True)
class Runtime:
    dtype: torch.dtype
    device: torch.device


@dataclass(frozen=True)
class PagedKV:
    """Keys and values of every position in pages; with a window only the last
    `window` positions are ever read, and older pages are given back."""
    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class FixedState:
    """State of fixed size per request, in a slot that lives as long as the
    request; zeroed when the slot is handed out."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


class Part:
    # True if `forward` reads nothing of a step but device tensors (and sizes that
    # are fixed for a given batch size): only then may a step be captured in a
    # CUDA graph.  Parts that look at the step's host-side lists leave it False.
    cuda_graph_safe = False

    def __init__(self, prefix: str = ""):
        self.prefix = prefix

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def ignored_tensors(self) -> List[str]:
        """Names that may be in the file and are not an error to find there."""
        return []

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime


class Norm(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor],
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """residual (float32, updated in place when `rows` is None) += delta;
        returns the normed sum in the engine's element type.  With `rows` only
        those rows are normed and `residual` is left as it is."""
        raise NotImplementedError


class Position(Part):
    """A position encoding applied to queries and keys inside a mixer."""

    def rotary_table(self, device) -> Optional[Tuple[torch.Tensor, int]]:
        """(float32 inverse frequencies [rot/2], rot) if the encoding is a
        half-split rotation that the fused kernel can apply; else None."""
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor):
        """For encodings the fused kernel does not know: returns (q, k)."""
        return q, k


class Mixer(Part):
    def cache_spec(self):
        return None

    def forward(self, h: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    """What opens a step: the float32 residual stream [tokens, hidden] from the
    step's context (its token ids, and whatever else of the step an input
    encoding needs: positions, the request of each token)."""

    def forward(self, ctx) -> torch.Tensor:
        raise NotImplementedError


class Block:
    """An arrangement of a layer's parts.  A subclass names the norms it wants in
    `norm_names` and says whether it can do without a mixer or a feed-forward;
    the layer's plan gives the norms by those names."""
    norm_names: Tuple[str, ...] = ()
    needs_mixer = True
    needs_feed_forward = True

    def __init__(self, mixer: Optional[Mixer], feed_forward: Optional[FeedForward], norms: Dict[str, Norm]):
        kind = type(self).__name__
        if sorted(norms) != sorted(self.norm_names):
            raise ValueError("%s takes the norms %s; the layer's plan gives %s"
                             % (kind, sorted(self.norm_names), sorted(norms)))
        if mixer is None and self.needs_mixer:
            raise ValueError("%s needs a mixer; the layer's plan gives none" % kind)
        if feed_forward is None and self.needs_feed_forward:
            raise ValueError("%s needs a feed-forward; the layer's plan gives none" % kind)
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, dict(norms)

    def parts(self) -> List[Part]:
        out: List[Part] = [self.norms[n] for n in self.norm_names]
        return out + [p for p in (self.mixer, self.feed_forward) if p is not None]

    def forward(self, residual, delta, ctx, cache):
        raise NotImplementedError
