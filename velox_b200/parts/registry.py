"""Registries from a part's kind to its class, one per category.

Another mixer, feed-forward, norm, position encoding, block arrangement,
embedding or head is added by registering a class here (from anywhere: a test
registers toy parts without touching this package) and naming its kind in a
plan.  A class is called as `cls(prefix=..., **params)`.
"""
from __future__ import annotations

from typing import Dict

from .plan import PartSpec

CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")
_REGISTRY: Dict[str, Dict[str, type]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, cls: type) -> type:
    if category not in _REGISTRY:
        raise KeyError("part category %r is not one of %s" % (category, CATEGORIES))
    _REGISTRY[category][kind] = cls
    return cls


def unregister_part(category: str, kind: str) -> None:
    _REGISTRY[category].pop(kind, None)


def part_class(category: str, kind: str) -> type:
    try:
        return _REGISTRY[category][kind]
    except KeyError:
        raise KeyError("no %s of kind %r is registered; registered: %s"
                       % (category, kind, sorted(_REGISTRY.get(category, {}))))


def build_part(category: str, spec: PartSpec):
    return part_class(category, spec.kind)(prefix=spec.prefix, **spec.params)


def register_mixer(kind, cls): return register_part("mixer", kind, cls)
def register_feed_forward(kind, cls): return register_part("feed_forward", kind, cls)
def register_norm(kind, cls): return register_part("norm", kind, cls)
def register_position(kind, cls): return register_part("position", kind, cls)
def register_block(kind, cls): return register_part("block", kind, cls)
