"""One registry from an architecture's name to its configuration class and plan.

The reference picks the model by `config.json["model_type"]`, else by the
lower-cased `architectures[0]` (src/backend/candle.rs:529-543), and its paged
path only accepts the former (src/backend/candle.rs:135-152, 227).  Here both
names lead to the same entry.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Type

from .model_config import ConfigError, ModelConfig, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    model_type: str
    config_class: Type[ModelConfig]
    # (typed config) -> parts.plan.ModelPlan
    plan: Callable[[Any], Any]


_BY_NAME: Dict[str, Architecture] = {}
_BY_MODEL_TYPE: Dict[str, Architecture] = {}


def register_architecture(name: str, model_type: str, config_class: Type[ModelConfig],
                          plan: Callable[[Any], Any]) -> Architecture:
    """Make `architectures: [name]` / `model_type` resolve to this model."""
    arch = Architecture(name, model_type, config_class, plan)
    _BY_NAME[name] = arch
    if model_type:
        _BY_MODEL_TYPE[model_type] = arch
    return arch


def unregister_architecture(name: str) -> None:
    arch = _BY_NAME.pop(name, None)
    if arch is not None and _BY_MODEL_TYPE.get(arch.model_type) is arch:
        del _BY_MODEL_TYPE[arch.model_type]


def registered_architectures():
    return sorted(_BY_NAME)


def _register_built_in() -> None:
    """The package's own architectures register themselves when their modules are
    imported; a caller that only imported the configuration gets them here."""
    import importlib
    importlib.import_module(__package__.rsplit(".", 1)[0] + ".models")


def resolve_architecture(raw: Dict[str, Any]) -> Architecture:
    """The entry that a raw config.json names."""
    _register_built_in()
    names = raw.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    for n in names:
        if n in _BY_NAME:
            return _BY_NAME[n]
    mt = raw.get("model_type")
    if mt in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[mt]
    raise ConfigError(
        "config.json names architectures=%r, model_type=%r; registered are %s"
        % (names, mt, registered_architectures())
    )


def load_config(folder: str):
    """(Architecture, typed config) of a model folder."""
    raw = read_config_json(folder)
    arch = resolve_architecture(raw)
    return arch, arch.config_class.from_dict(raw)
