"""Reading and writing the safetensors container.

The format: an 8-byte little-endian header length, a JSON header mapping each
tensor name to {dtype, shape, data_offsets}, then the raw little-endian tensor
bytes.  The reference reads it through a memory map and converts per tensor
(`engine/src/weights.rs:20-33`, `:54-94`); so does this.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from typing import Dict, Mapping, Optional, Tuple

import torch

_DTYPES = {
    "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "F64": torch.float64, "I64": torch.int64, "I32": torch.int32, "I16": torch.int16,
    "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    start: int
    end: int


class SafetensorsFile:
    """A memory-mapped safetensors file; tensors are read by name."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._file = open(path, "rb")
        except FileNotFoundError:
            raise SafetensorsError(f"no such weights file: {path}") from None
        head = self._file.read(8)
        if len(head) != 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", head)
        size = self._file.seek(0, 2)
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file")
        self._file.seek(8)
        try:
            header = json.loads(self._file.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self._base = 8 + n
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            start, end = info["data_offsets"]
            entry = TensorEntry(name, info["dtype"], tuple(info["shape"]), start, end)
            if entry.dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype "
                                       f"{entry.dtype}")
            numel = 1
            for s in entry.shape:
                numel *= s
            want = numel * torch.empty((), dtype=_DTYPES[entry.dtype]).element_size()
            if end - start != want or self._base + end > size:
                raise SafetensorsError(f"{path}: tensor {name!r} has {end - start} bytes, "
                                       f"its shape {list(entry.shape)} needs {want}")
            self.entries[name] = entry
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self):
        return list(self.entries)

    def __contains__(self, name: str) -> bool:
        return name in self.entries

    def get(self, name: str) -> torch.Tensor:
        """A CPU tensor holding a copy of the stored values, in the stored dtype."""
        try:
            e = self.entries[name]
        except KeyError:
            raise SafetensorsError(f"no tensor named {name!r} in {self.path}") from None
        dtype = _DTYPES[e.dtype]
        nbytes = e.end - e.start
        if nbytes == 0:
            return torch.empty(e.shape, dtype=dtype)
        raw = bytearray(self._map[self._base + e.start:self._base + e.end])
        flat = torch.frombuffer(raw, dtype=torch.uint8, count=nbytes)
        return flat.view(dtype).reshape(e.shape)

    def close(self) -> None:
        if self._map is not None:
            self._map.close()
            self._map = None
        self._file.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Optional[Mapping[str, str]] = None) -> None:
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    blobs = []
    for name in order:
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)
