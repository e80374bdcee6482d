"""Reading and writing the safetensors container without a library.

Layout of a file: 8 bytes little-endian header length n, n bytes of JSON
(`{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": ...}`),
then the tensors' bytes, offsets counted from the end of the header.  Files are
memory-mapped; a tensor is a view into the map until it is copied to the device.

Which files make up a model follows the reference
(src/backend/candle.rs:642-666): the sorted, distinct values of
`model.safetensors.index.json`'s `weight_map`, else `model.safetensors`.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, List, Tuple

import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(IOError):
    pass


class SafetensorsFile:
    """One memory-mapped safetensors file."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError("%s: too short for a safetensors header" % path)
        self._fh = open(path, "rb")
        (n,) = struct.unpack("<Q", self._fh.read(8))
        if n <= 0 or 8 + n > size:
            raise SafetensorsError("%s: header length %d does not fit the file (%d bytes)" % (path, n, size))
        try:
            header = json.loads(self._fh.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError("%s: header is not JSON: %s" % (path, e))
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + n
        self._entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            dt, shape = e["dtype"], tuple(int(s) for s in e["shape"])
            b, end = (int(x) for x in e["data_offsets"])
            if dt not in _DTYPES:
                raise SafetensorsError("%s: tensor %s has unsupported dtype %s" % (path, name, dt))
            count = 1
            for s in shape:
                count *= s
            if end - b != count * _DTYPES[dt][1] or self._data_start + end > size:
                raise SafetensorsError("%s: tensor %s: offsets [%d,%d) do not match shape %s %s"
                                       % (path, name, b, end, list(shape), dt))
            self._entries[name] = (dt, shape, b, end)
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)

    def keys(self) -> List[str]:
        return list(self._entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dt, shape, _, _ = self._entries[name]
        return _DTYPES[dt][0], shape

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only CPU view of the tensor's bytes in the map."""
        dt, shape, b, end = self._entries[name]
        tdt = _DTYPES[dt][0]
        if end == b:
            return torch.empty(shape, dtype=tdt)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the map is read-only; nobody writes through the view
            flat = torch.frombuffer(self._map, dtype=torch.uint8, count=end - b, offset=self._data_start + b)
        return flat.view(tdt).reshape(shape)

    def close(self) -> None:
        try:
            self._map.close()
        except (BufferError, ValueError):
            pass  # views still alive: the map goes when they do
        self._fh.close()


def model_files(folder: str) -> List[str]:
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index) as f:
            names = sorted(set(json.load(f).get("weight_map", {}).values()))
        if names:
            return [os.path.join(folder, n) for n in names]
    single = os.path.join(folder, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    raise SafetensorsError("no safetensors found in %s" % folder)


def write_safetensors(path: str, tensors, metadata=None, layout=None) -> None:
    """Write tensors to `path`.

    `tensors` is a dict name -> CPU tensor, or, with `layout` (a list of
    (name, dtype, shape)), a callable name -> tensor that is asked for one
    tensor at a time in the layout's order, so that a large model never has to
    be held whole."""
    if layout is None:
        layout = [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()]
        produce = tensors.__getitem__
    else:
        produce = tensors
    header: Dict[str, dict] = {}
    offset = 0
    for name, dtype, shape in layout:
        if dtype not in _NAMES:
            raise SafetensorsError("tensor %s: dtype %s cannot be stored" % (name, dtype))
        count = 1
        for s_ in shape:
            count *= int(s_)
        nbytes = count * _DTYPES[_NAMES[dtype]][1]
        header[name] = {"dtype": _NAMES[dtype], "shape": [int(s_) for s_ in shape],
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, dtype, shape in layout:
            t = produce(name).detach().contiguous().cpu()
            if t.dtype != dtype or tuple(t.shape) != tuple(shape):
                raise SafetensorsError("tensor %s: produced %s %s, announced %s %s"
                                       % (name, t.dtype, list(t.shape), dtype, list(shape)))
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
