"""Binding a model's tensors to a safetensors checkpoint by name.

The model says what it wants (`DecoderModel.tensor_specs()`); the files say what
they hold.  Every disagreement (a missing tensor, an unexpected one, a wrong
shape, an element type that cannot be used) is collected and raised as ONE
error that lists them all.  The reference stops at the first
(src/backend/candle.rs:139-140) and silently skips absent q/k norms
(src/paged/qwen3.rs:393-394); here those are required like any other tensor.

Element types on the device:
  matrices and tables: the engine's element type (bfloat16 files stay
    bfloat16 in a bfloat16 engine; the 32-bit engine widens them exactly);
  norm weights and biases: float32 (exact for bfloat16 files; a tensor stored in
    32 bits stays so);
  integer tables: int32.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Mapping

import torch

from ..parts.base import Runtime, TensorSpec
from .safetensors_io import SafetensorsFile, model_files


class WeightError(ValueError):
    """The checkpoint does not fit the model; `missing`, `unexpected`,
    `wrong_shape` and `wrong_dtype` hold the details."""

    def __init__(self, folder, missing, unexpected, wrong_shape, wrong_dtype):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = ["weights in %s do not fit the model:" % folder]
        if self.missing:
            lines.append("  missing (%d): %s" % (len(self.missing), ", ".join(self.missing)))
        if self.unexpected:
            lines.append("  unexpected (%d): %s" % (len(self.unexpected), ", ".join(self.unexpected)))
        for name, want, got in self.wrong_shape:
            lines.append("  wrong shape: %s expected %s, file has %s" % (name, list(want), list(got)))
        for name, got in self.wrong_dtype:
            lines.append("  unusable element type: %s is %s" % (name, got))
        super().__init__("\n".join(lines))


_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INTS = (torch.int32, torch.int64, torch.int16, torch.int8, torch.uint8)


def held_dtype(role: str, stored: torch.dtype, runtime: Runtime) -> torch.dtype:
    if role == "int_table":
        return torch.int32
    if role in ("norm", "bias"):
        return torch.float32
    return runtime.dtype


class OnDemand(Mapping):
    """name -> tensor on the device, made by `fetch` at every lookup and not kept."""

    def __init__(self, fetch: Callable[[str], torch.Tensor], names):
        self._fetch, self._names = fetch, names

    def __getitem__(self, name: str) -> torch.Tensor:
        if name not in self._names:
            raise KeyError(name)
        return self._fetch(name)

    def __iter__(self):
        return iter(self._names)

    def __len__(self) -> int:
        return len(self._names)


def load_weights(model, folder: str, runtime: Runtime) -> None:
    """Reads the folder's safetensors and binds them to `model` on the device."""
    files = [SafetensorsFile(p) for p in model_files(folder)]
    where: Dict[str, SafetensorsFile] = {}
    for f in files:
        for name in f.keys():
            where[name] = f
    specs: List[TensorSpec] = model.tensor_specs()
    wanted = {s.name for s in specs}
    ignored = set(model.ignored_tensors())
    missing = [s.name for s in specs if s.name not in where]
    unexpected = sorted(n for n in where if n not in wanted and n not in ignored)
    wrong_shape, wrong_dtype = [], []
    for s in specs:
        if s.name not in where:
            continue
        dt, shape = where[s.name].info(s.name)
        if tuple(shape) != tuple(s.shape):
            wrong_shape.append((s.name, s.shape, shape))
        ok = dt in _INTS if s.role == "int_table" else dt in _FLOATS
        if not ok:
            wrong_dtype.append((s.name, str(dt).replace("torch.", "")))
    if missing or unexpected or wrong_shape or wrong_dtype:
        for f in files:
            f.close()
        raise WeightError(folder, missing, unexpected, wrong_shape, wrong_dtype)
    by_name = {s.name: s for s in specs}

    def fetch(name: str) -> torch.Tensor:
        s = by_name[name]
        src = where[name].tensor(name)
        return src.to(device=runtime.device, dtype=held_dtype(s.role, src.dtype, runtime)).contiguous()
    # A tensor goes to the device when its part binds it and is kept by nobody else: a part
    # that fuses matrices (q, k, v; gate and up) holds the originals only while it does so,
    # and the peak stays near the size of the model, not near twice that.
    model.bind(OnDemand(fetch, by_name), runtime)
    for f in files:
        f.close()
