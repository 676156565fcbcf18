"""Reading and writing safetensors files.

Layout and checks as the reference's header parser makes them
(src/Starlings.Roost.Worker/Weights/SafetensorsHeader.cs:89-172): an 8-byte little-endian header length, a
JSON object whose entries give dtype, shape and ``data_offsets`` relative to the end of the header;
``__metadata__`` is skipped; every tensor's byte range must equal shape x element size, and the ranges,
sorted, must tile the data region exactly (no gap, overlap or trailing bytes). Only the tensors a caller
asks for are materialised (src/Starlings.Roost.Worker/Weights/ModelWeightLoader.cs:198-221).
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

MAX_HEADER_BYTES = 100 * 1024 * 1024

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: tuple
    begin: int
    end: int


class SafetensorsFile:
    """A parsed header over a memory-mapped file. ``tensor(name)`` copies one tensor out of the map."""

    def __init__(self, path):
        self.path = Path(path)
        try:
            self._fh = open(self.path, "rb")
        except FileNotFoundError:
            raise SafetensorsError(f"{self.path}: no such file") from None
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: {size} bytes is too short for a safetensors header")
        (n,) = struct.unpack("<Q", self._fh.read(8))
        if n > MAX_HEADER_BYTES or n > size - 8:
            raise SafetensorsError(f"{self.path}: header length {n} is beyond the file or the {MAX_HEADER_BYTES}-byte limit")
        try:
            header = json.loads(self._fh.read(n))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise SafetensorsError(f"{self.path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{self.path}: header is not a JSON object")
        self.data_start = 8 + n
        data_len = size - self.data_start
        self.entries: dict[str, TensorEntry] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            try:
                dt, shape, (a, b) = meta["dtype"], tuple(int(x) for x in meta["shape"]), meta["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{self.path}: entry '{name}' lacks dtype, shape or data_offsets") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{self.path}: entry '{name}' has dtype '{dt}', which is not known")
            count = 1
            for s in shape:
                if s < 0:
                    raise SafetensorsError(f"{self.path}: entry '{name}' has a negative dimension")
                count *= s
            if not (0 <= a <= b <= data_len) or b - a != count * _DTYPES[dt][1]:
                raise SafetensorsError(f"{self.path}: entry '{name}' spans bytes [{a}, {b}) but its shape {list(shape)} of {dt} needs {count * _DTYPES[dt][1]}")
            self.entries[name] = TensorEntry(name, dt, shape, a, b)
        at = 0
        for e in sorted(self.entries.values(), key=lambda e: (e.begin, e.end)):
            if e.begin != at:
                raise SafetensorsError(f"{self.path}: tensors do not tile the data region (entry '{e.name}' begins at {e.begin}, expected {at})")
            at = e.end
        if at != data_len:
            raise SafetensorsError(f"{self.path}: {data_len - at} trailing bytes after the last tensor")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self):
        return self.entries.keys()

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        dt, _ = _DTYPES[e.dtype]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=dt)
        raw = np.frombuffer(self._map, dtype=np.uint8, count=e.end - e.begin, offset=self.data_start + e.begin).copy()
        t = torch.from_numpy(raw)
        return (t.view(dt) if dt != torch.bool else t.to(torch.bool)).reshape(e.shape)

    def close(self):
        if self._map is not None:
            self._map.close()
            self._map = None
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def write_safetensors(path, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Writes tensors in the given order, contiguous, with an 8-byte-aligned header."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    at = 0
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}' has dtype {t.dtype}, which safetensors cannot hold")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + n]}
        at += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for t in tensors.values():
            t = t.detach().contiguous().cpu()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dtype != torch.bool else t.to(torch.uint8).numpy().tobytes())
