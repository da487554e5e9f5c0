"""Reading and writing the safetensors container without any library.

Layout: an unsigned 64-bit little-endian header length N, N bytes of JSON mapping each tensor
name to {"dtype", "shape", "data_offsets": [begin, end]} (offsets relative to the end of the
header), then the raw little-endian tensor data.  Files are memory-mapped; a tensor is a view
of the map until it is copied to the device.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch

DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One mapped file; `tensor(name)` gives a CPU tensor that views the map."""

    def __init__(self, path):
        self.path = Path(path)
        if not self.path.is_file():
            raise SafetensorsError(f"{self.path}: no such weights file")
        self._f = open(self.path, "rb")
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: too short to be a safetensors file")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (n,) = struct.unpack("<Q", self._map[:8])
        if 8 + n > size:
            raise SafetensorsError(f"{self.path}: header length {n} exceeds the file size {size}")
        try:
            header = json.loads(self._map[8:8 + n])
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{self.path}: header is not JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + n
        self.entries = header
        for name, meta in header.items():
            if meta.get("dtype") not in DTYPES:
                raise SafetensorsError(f"{self.path}: tensor '{name}' has unsupported dtype {meta.get('dtype')!r}")
            a, b = meta["data_offsets"]
            numel = 1
            for s in meta["shape"]:
                numel *= s
            if b - a != numel * DTYPES[meta["dtype"]].itemsize or self._base + b > size:
                raise SafetensorsError(f"{self.path}: tensor '{name}' has a data range that does not fit its shape")

    def names(self):
        return list(self.entries)

    def shape(self, name) -> tuple:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name) -> torch.dtype:
        return DTYPES[self.entries[name]["dtype"]]

    def tensor(self, name) -> torch.Tensor:
        meta = self.entries[name]
        a, b = meta["data_offsets"]
        dtype = DTYPES[meta["dtype"]]
        if b == a:
            return torch.empty(meta["shape"], dtype=dtype)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")                 # the map is read-only; tensors are never written
            flat = torch.frombuffer(self._map, dtype=dtype, count=(b - a) // dtype.itemsize,
                                    offset=self._base + a)
        return flat.reshape(meta["shape"])

    def close(self):
        try:
            self._map.close()
        except BufferError:                                  # views still alive; the map closes with them
            pass
        self._f.close()


def write_safetensors(path, tensors: dict, metadata: dict | None = None) -> None:
    """Write CPU tensors under their names, in name order, data aligned to 8 bytes."""
    header, offset, blobs = {}, 0, []
    for name in sorted(tensors):
        t = tensors[name].detach().contiguous().cpu()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.dtype.itemsize
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        blobs.append(t)
        offset += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    raw = json.dumps(header, separators=(",", ":")).encode()
    raw += b" " * (-(len(raw) + 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for t in blobs:
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
