"""Random weights: a model folder (config.json, model.safetensors) from a
configuration and a seed.

Matrices and tables are N(0, 0.02), norm weights 1 + N(0, 0.05), biases
N(0, 0.02), integer tables uniform.  Every tensor has its own generator keyed by
(seed, tensor name), so a tensor's values do not depend on which other tensors
the model has or on the order they are made in.  Values are rounded to the
stored element type (bfloat16 by default), so that an engine in either
precision and an independent implementation read exactly the same numbers.
The reference has no such mode.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Optional

import torch

from ..config.model_config import ModelConfig
from ..config.registry import resolve_architecture
from ..parts.base import TensorSpec
from .safetensors_io import write_safetensors

MATRIX_STD, NORM_STD, BIAS_STD = 0.02, 0.05, 0.02


def _generator(seed: int, name: str, device="cpu") -> torch.Generator:
    digest = hashlib.sha256(("%d:%s" % (seed, name)).encode()).digest()
    g = torch.Generator(device=device)
    g.manual_seed(int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF)
    return g


def random_tensor(spec: TensorSpec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    g = _generator(seed, spec.name, device)
    if spec.role == "int_table":
        return torch.randint(0, 1 << 15, spec.shape, generator=g, dtype=torch.int32, device=device)
    x = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device)
    if spec.role == "norm":
        x = 1.0 + NORM_STD * x
    elif spec.role == "bias":
        x = BIAS_STD * x
    else:
        x = MATRIX_STD * x
    return x.to(dtype)


def write_random_model(folder: str, config: ModelConfig, seed: int, dtype: str = "bfloat16",
                       extra_config: Optional[Dict] = None) -> str:
    """Writes config.json and model.safetensors for `config` into `folder`."""
    from ..models.decoder import DecoderModel

    store = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    raw = config.to_dict()
    raw["torch_dtype"] = dtype
    if extra_config:
        raw.update(extra_config)
    arch = resolve_architecture(raw)
    model = DecoderModel(arch.plan(config))
    specs = {s.name: s for s in model.tensor_specs()}
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f, indent=1)
    layout = [(s.name, torch.int32 if s.role == "int_table" else store, tuple(s.shape)) for s in specs.values()]
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      lambda name: random_tensor(specs[name], seed, store),
                      metadata={"format": "pt", "seed": seed}, layout=layout)
    return folder


def bind_random_weights(model, runtime, seed: int) -> None:
    """Random weights made on the device, without a file: for measurements on
    large shapes.  (The values differ from `write_random_model`'s, whose
    generator runs on the host.)"""
    from .loader import OnDemand, held_dtype

    specs = {s.name: s for s in model.tensor_specs()}

    def make(name: str) -> torch.Tensor:
        s = specs[name]
        t = random_tensor(s, seed, torch.float32 if s.role in ("norm", "bias") else runtime.dtype, runtime.device)
        return t.to(held_dtype(s.role, t.dtype, runtime)).contiguous()
    model.bind(OnDemand(make, specs), runtime)   # (made when a part binds them: see `load_weights`)
