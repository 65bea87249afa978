"""Reading and writing the safetensors container: 8 bytes of little-endian header length, a JSON
header {name: {dtype, shape, data_offsets}}, then the raw little-endian data.

The reference stores weights as burn `.mpk` records (crates/burn-lm-llama/src/nn/llama/base.rs:
149-158) and has no safetensors support; this reader is written from the format's description.
Files are memory-mapped; a tensor is copied only when it is taken.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings

import torch

_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """An open, memory-mapped safetensors file: `names()`, `shape(name)`, `dtype(name)`, `get(name)`."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except FileNotFoundError:
            raise SafetensorsError(f"{path}: no such file") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file ({size} bytes)")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + hlen
        self._entries = {}
        for name, e in header.items():
            try:
                dt, shape, (lo, hi) = e["dtype"], tuple(e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for {name!r}") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt}")
            n = 1
            for s in shape:
                n *= s
            if hi - lo != n * _DTYPES[dt][1] or lo < 0 or self._base + hi > size:
                raise SafetensorsError(f"{path}: tensor {name!r} has offsets [{lo}, {hi}) that do not fit "
                                       f"its shape {shape} or the file")
            self._entries[name] = (dt, shape, lo, hi)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self):
        return list(self._entries)

    def __contains__(self, name):
        return name in self._entries

    def shape(self, name):
        return self._entries[name][1]

    def dtype(self, name) -> torch.dtype:
        return _DTYPES[self._entries[name][0]][0]

    def get(self, name) -> torch.Tensor:
        """The tensor as a CPU tensor that views the mapping (copy or move it before closing)."""
        dt, shape, lo, hi = self._entries[name]
        if hi == lo:
            return torch.empty(shape, dtype=_DTYPES[dt][0])
        buf = memoryview(self._mm)[self._base + lo: self._base + hi]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)   # the read-only mapping is only ever read
            return torch.frombuffer(buf, dtype=_DTYPES[dt][0]).reshape(shape)

    def close(self):
        try:
            if self._mm is not None:
                self._mm.close()
        except BufferError:
            pass  # a view is still alive; the mapping goes with it
        self._f.close()


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    """Write CPU tensors under their names (sorted, 8-byte aligned header)."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
