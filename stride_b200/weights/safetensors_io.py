"""Reader and writer of the safetensors container: an unsigned 64-bit little-endian
header length, a JSON header {name: {dtype, shape, data_offsets}} (the entry
"__metadata__" is skipped), then the raw little-endian data.

Restates the checks of arhaamatiq/stride's reader (src/safetensors.cpp:14-59): the file
must hold the header it announces, and every tensor's offsets must lie inside the data
and match shape x element size. The file is memory-mapped; tensors are views of the map
until the caller copies them to the device.
"""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from pathlib import Path

import numpy as np
import torch


class SafetensorsError(RuntimeError):
    pass


_DTYPES = {
    "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4), "F64": (torch.float64, 8),
    "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "I16": (torch.int16, 2), "I32": (torch.int32, 4),
    "I64": (torch.int64, 8), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    def __init__(self, path):
        self.path = Path(path)
        try:
            self._f = open(self.path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open {self.path}: {e.strerror}") from e
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: file too small to be safetensors ({size} bytes)")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if 8 + hlen > size:
            raise SafetensorsError(f"{self.path}: header of {hlen} bytes overruns the file of {size} bytes")
        try:
            header = json.loads(bytes(self._map[8:8 + hlen]))
        except ValueError as e:
            raise SafetensorsError(f"{self.path}: header is not JSON: {e}") from e
        self._data_start = 8 + hlen
        data_size = size - self._data_start
        self.entries: dict = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            dt = meta.get("dtype")
            if dt not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor '{name}' has unsupported dtype {dt}")
            shape = tuple(int(d) for d in meta["shape"])
            begin, end = (int(x) for x in meta["data_offsets"])
            count = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if begin < 0 or end < begin or end > data_size or end - begin != count * _DTYPES[dt][1]:
                raise SafetensorsError(f"{self.path}: bad offsets for tensor '{name}'")
            self.entries[name] = (dt, shape, begin, end)

    def names(self):
        return list(self.entries)

    def has(self, name: str) -> bool:
        return name in self.entries

    def shape(self, name: str) -> tuple:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name][0]][0]

    def get(self, name: str) -> torch.Tensor:
        """A read-only view of the mapped file (copy it before the file is closed)."""
        if name not in self.entries:
            raise SafetensorsError(f"{self.path}: missing tensor '{name}'")
        dt, shape, begin, end = self.entries[name]
        tdt = _DTYPES[dt][0]
        if end == begin:
            return torch.empty(shape, dtype=tdt)
        buf = memoryview(self._map)[self._data_start + begin:self._data_start + end]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)     # the map is read-only; callers copy, never write
            flat = torch.frombuffer(buf, dtype=tdt)
        return flat.reshape(shape)

    def close(self):
        try:
            self._map.close()
        except BufferError:
            pass          # views are still alive; the map goes with them
        self._f.close()


def write_safetensors(path, tensors: dict, metadata: dict | None = None) -> None:
    """Write `tensors` (name -> CPU tensor) in name order."""
    header, at = {}, 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}' has dtype {t.dtype}, which safetensors cannot hold")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + nbytes]}
        at += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())
