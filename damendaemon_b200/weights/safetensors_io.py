"""Minimal safetensors reader and writer (the file format only; no model code).

Layout: 8-byte little-endian header length, a JSON header mapping tensor names to
``{"dtype", "shape", "data_offsets"}``, then the raw little-endian tensor bytes.
The header is validated before any tensor byte is touched, in the manner of the
reference (damendaemon/safetensor_header.py:65-95, damendaemon/checkpoint.py:29-68):
bounded header size, unique keys, in-range and non-overlapping data ranges.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch

MAX_HEADER_BYTES = 16 * 1024 * 1024

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class CheckpointFormatError(ValueError):
    pass


def _unique(pairs):
    out = {}
    for key, value in pairs:
        if key in out:
            raise CheckpointFormatError(f"safetensors header: duplicate entry {key!r}")
        out[key] = value
    return out


def read_header(path) -> tuple:
    """Return ({name: (dtype, shape, begin, end)}, data_start, file_size)."""
    path = Path(path)
    size = path.stat().st_size
    with path.open("rb") as f:
        first = f.read(8)
        if len(first) != 8:
            raise CheckpointFormatError(f"{path}: too short for a safetensors file")
        (n,) = struct.unpack("<Q", first)
        if n > MAX_HEADER_BYTES or 8 + n > size:
            raise CheckpointFormatError(f"{path}: bad safetensors header length {n}")
        try:
            header = json.loads(f.read(n).decode("utf-8"), object_pairs_hook=_unique)
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise CheckpointFormatError(f"{path}: unreadable safetensors header: {error}") from error
    if not isinstance(header, dict):
        raise CheckpointFormatError(f"{path}: safetensors header must be an object")
    data_start = 8 + n
    entries, spans = {}, []
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype = _DTYPES[meta["dtype"]]
            shape = tuple(int(x) for x in meta["shape"])
            begin, end = (int(x) for x in meta["data_offsets"])
        except (KeyError, TypeError, ValueError) as error:
            raise CheckpointFormatError(f"{path}: bad header entry for {name!r}") from error
        count = 1
        for x in shape:
            if x < 0:
                raise CheckpointFormatError(f"{path}: negative dimension in {name!r}")
            count *= x
        if begin < 0 or end < begin or data_start + end > size or end - begin != count * dtype.itemsize:
            raise CheckpointFormatError(f"{path}: data range of {name!r} does not match its shape")
        entries[name] = (dtype, shape, begin, end)
        spans.append((begin, end, name))
    spans.sort()
    for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
        if b1 < e0:
            raise CheckpointFormatError(f"{path}: tensors {n0!r} and {n1!r} overlap")
    return entries, data_start, size


class SafetensorsFile:
    """Random access to the tensors of one file through a read-only memory map."""

    def __init__(self, path):
        self.path = Path(path)
        self.entries, self._start, _ = read_header(self.path)
        self._file = self.path.open("rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if self.path.stat().st_size else None

    def names(self):
        return list(self.entries)

    def describe(self, name):
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def tensor(self, name) -> torch.Tensor:
        """A CPU tensor that owns its bytes (copied out of the map)."""
        dtype, shape, begin, end = self.entries[name]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        view = memoryview(self._map)[self._start + begin:self._start + end]
        return torch.frombuffer(bytearray(view), dtype=dtype).reshape(shape)

    def close(self):
        if self._map is not None:
            self._map.close()
            self._map = None
        self._file.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path, tensors: dict, metadata: dict | None = None):
    """Write ``tensors`` (name -> CPU or device tensor) in name order, atomically."""
    path = Path(path)
    header, offset = {}, 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise CheckpointFormatError(f"cannot store dtype {t.dtype} ({name})")
        size = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + size]}
        offset += size
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * (-len(raw) % 8)
    tmp = path.with_name(path.name + ".tmp")
    with tmp.open("wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
    tmp.replace(path)
