"""Typed model configurations, read from an architecture's own config.json keys.

`Qwen3Config` holds exactly the keys that the reference's `Qwen3Config`
deserialises (src/paged/qwen3.rs:30-60): thirteen required keys, three
optional ones about the sliding window, unknown keys ignored.  Nothing here
knows a model size: every number comes from the file or from the caller.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass
from typing import Any, ClassVar, Dict, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot describe a model: lists every fault found."""


def _typed(name: str, value: Any, kind: type, faults: list) -> Any:
    if kind is float and isinstance(value, (int, float)) and not isinstance(value, bool):
        return float(value)
    if kind is int and isinstance(value, int) and not isinstance(value, bool):
        return value
    if kind is bool and isinstance(value, bool):
        return value
    if kind is str and isinstance(value, str):
        return value
    faults.append("key %r: expected %s, got %r" % (name, kind.__name__, value))
    return None


@dataclass(frozen=True)
class ModelConfig:
    """Base of the typed configurations.  A subclass lists its keys as
    dataclass fields; a field without a default is a required key."""

    architecture: ClassVar[str] = ""
    model_type: ClassVar[str] = ""

    # keys that, when present and not null, name something this engine does not do
    unsupported_keys: ClassVar[Dict[str, str]] = {}

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ModelConfig":
        faults: list = []
        values: Dict[str, Any] = {}
        for key, why in cls.unsupported_keys.items():
            if raw.get(key) is not None:
                faults.append("key %r: %s" % (key, why))
        for f in dataclasses.fields(cls):
            required = f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING
            if f.name not in raw or raw[f.name] is None:
                if required:
                    faults.append("missing key %r" % f.name)
                continue
            kind = f.metadata.get("kind", f.type)
            values[f.name] = _typed(f.name, raw[f.name], kind, faults)
        if faults:
            raise ConfigError("config.json for %s: %s" % (cls.__name__, "; ".join(faults)))
        cfg = cls(**values)
        cfg.validate()
        return cfg

    @classmethod
    def from_folder(cls, folder: str) -> "ModelConfig":
        return cls.from_dict(read_config_json(folder))

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that `from_dict` reads back to this configuration."""
        out: Dict[str, Any] = {"architectures": [self.architecture], "model_type": self.model_type}
        out.update(dataclasses.asdict(self))
        return out

    def validate(self) -> None:  # pragma: no cover - overridden
        pass


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError("no config.json in %s" % folder)
    with open(path) as f:
        raw = json.load(f)
    if not isinstance(raw, dict):
        raise ConfigError("%s does not hold a JSON object" % path)
    return raw


def _field(kind: type, **kw):
    return dataclasses.field(metadata={"kind": kind}, **kw)


SUPPORTED_ACTIVATIONS: Tuple[str, ...] = ("silu", "gelu", "gelu_pytorch_tanh", "relu")


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    """Qwen3 dense decoder (src/paged/qwen3.rs:30-60).

    `head_dim` is its own key and need not be hidden_size / heads
    (src/paged/qwen3.rs:36, 390).  The window keys are optional and default
    to "no window" (src/paged/qwen3.rs:41-48)."""

    architecture: ClassVar[str] = "Qwen3ForCausalLM"
    model_type: ClassVar[str] = "qwen3"
    # the reference reads 4-bit checkpoints through these (src/paged/qwen3.rs:51-59)
    unsupported_keys: ClassVar[Dict[str, str]] = {
        "quantization": "quantized weights are not supported; the engine holds bfloat16 or float32",
        "quantization_config": "quantized weights are not supported; the engine holds bfloat16 or float32",
    }

    vocab_size: int = _field(int)
    hidden_size: int = _field(int)
    intermediate_size: int = _field(int)
    num_hidden_layers: int = _field(int)
    num_attention_heads: int = _field(int)
    head_dim: int = _field(int)
    attention_bias: bool = _field(bool)
    num_key_value_heads: int = _field(int)
    max_position_embeddings: int = _field(int)
    tie_word_embeddings: bool = _field(bool)
    rope_theta: float = _field(float)
    rms_norm_eps: float = _field(float)
    hidden_act: str = _field(str)
    sliding_window: Optional[int] = _field(int, default=None)
    max_window_layers: int = _field(int, default=0)
    use_sliding_window: bool = _field(bool, default=False)

    def validate(self) -> None:
        faults = []
        for name in (
            "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
            "num_attention_heads", "head_dim", "num_key_value_heads", "max_position_embeddings",
        ):
            if getattr(self, name) <= 0:
                faults.append("%s must be positive, got %d" % (name, getattr(self, name)))
        if not faults:
            # the reference divides without checking (src/paged/qwen3.rs:385)
            if self.num_attention_heads % self.num_key_value_heads:
                faults.append(
                    "num_attention_heads (%d) is not a multiple of num_key_value_heads (%d)"
                    % (self.num_attention_heads, self.num_key_value_heads)
                )
            if self.head_dim % 2:
                faults.append("head_dim (%d) must be even for the rotation" % self.head_dim)
        if not self.rope_theta > 0:
            faults.append("rope_theta must be positive, got %r" % self.rope_theta)
        if not self.rms_norm_eps > 0:
            faults.append("rms_norm_eps must be positive, got %r" % self.rms_norm_eps)
        if self.hidden_act not in SUPPORTED_ACTIVATIONS:
            faults.append("hidden_act %r is not one of %s" % (self.hidden_act, list(SUPPORTED_ACTIVATIONS)))
        if self.use_sliding_window and not (self.sliding_window and self.sliding_window > 0):
            faults.append("use_sliding_window needs a positive sliding_window")
        if self.max_window_layers < 0:
            faults.append("max_window_layers must not be negative")
        if faults:
            raise ConfigError("Qwen3 configuration: " + "; ".join(faults))

    def window_of_layer(self, layer: int) -> int:
        """Keys a layer's queries see besides themselves, 0 for all.  The
        reference gives `sliding_window` to every layer when
        `use_sliding_window` is set (src/paged/qwen3.rs:373-381) and reads
        `max_window_layers` without using it (default 0, :43-44).  Here the
        first `max_window_layers` layers see everything and the later ones the
        window; at the default of 0 that is the reference's behaviour."""
        if not self.use_sliding_window or not self.sliding_window:
            return 0
        return int(self.sliding_window) if layer >= self.max_window_layers else 0
