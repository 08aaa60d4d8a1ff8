"""Reader and writer for the safetensors container.

Layout: 8 bytes little-endian header length n, n bytes of JSON
{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}},
then the tensors' bytes, offsets counted from the end of the header. The
reference's own container (crates/cellm-model/src/cellm_file.rs:58-124) checks
magic, header length and that every tensor lies inside the file; the same
checks are made here before any tensor is handed out.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass

import torch

from .errors import WeightError

_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    begin: int
    end: int


class SafetensorsFile:
    """A memory-mapped safetensors file; `tensor(name)` returns a CPU view."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
        except OSError:
            raise WeightError(f"{path}: no such file") from None
        if size < 8:
            raise WeightError(f"{path}: {size} bytes is too short for a safetensors header")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > _MAX_HEADER or 8 + n > size:
            raise WeightError(f"{path}: header length {n} does not fit the file of {size} bytes")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightError(f"{path}: header is not valid JSON: {e}") from None
        if not isinstance(header, dict):
            raise WeightError(f"{path}: header is not a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + n
        data_len = size - self._data_start
        self.entries: dict[str, TensorEntry] = {}
        for name, info in header.items():
            try:
                dt, shape, (b, e) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise WeightError(f"{path}: malformed entry for tensor {name!r}") from None
            if dt not in _DTYPES:
                raise WeightError(f"{path}: tensor {name!r} has unsupported dtype {dt}")
            numel = 1
            for s in shape:
                numel *= s
            if not (0 <= b <= e <= data_len) or e - b != numel * _DTYPES[dt][1]:
                raise WeightError(f"{path}: tensor {name!r} ({dt}{list(shape)}) has data offsets [{b}, {e}) "
                                  f"that do not match its size or lie outside the {data_len} data bytes "
                                  f"(truncated file?)")
            self.entries[name] = TensorEntry(name, _DTYPES[dt][0], shape, b, e)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self):
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        buf = memoryview(self._mm)[self._data_start + e.begin:self._data_start + e.end]
        with warnings.catch_warnings():
            # the map is read-only and torch says so; callers only read or copy the view
            warnings.simplefilter("ignore", UserWarning)
            return torch.frombuffer(buf, dtype=e.dtype).reshape(e.shape)

    def close(self):
        # Views handed out keep the map alive; dropping our references is enough.
        self._mm = None
        self._f.close()


def save_file(tensors: dict[str, torch.Tensor], path: str, metadata: dict | None = None) -> None:
    """Writes CPU tensors in the order of their names."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise WeightError(f"cannot store tensor {name!r} of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy())
    os.replace(tmp, path)
