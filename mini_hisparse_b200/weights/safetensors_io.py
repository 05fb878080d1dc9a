"""A small reader and writer for the safetensors format.

Layout of a file: 8 bytes little-endian header length n, n bytes of JSON mapping each tensor
name to {"dtype", "shape", "data_offsets": [begin, end]} (offsets relative to the end of the
header), then the raw little-endian data.  The reference leaves file reading to a library
(mini_hisparse/model.py:100-114); this engine reads tensors by name itself.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable, Mapping

import torch

DTYPES = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
NAMES = {v: k for k, v in DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    begin: int
    end: int
    file: Path


class SafetensorsFile:
    """One file, memory-mapped; tensors are materialised one at a time."""

    def __init__(self, path):
        self.path = Path(path)
        with open(self.path, "rb") as f:
            head = f.read(8)
            if len(head) != 8:
                raise SafetensorsError(f"{self.path}: too short to be a safetensors file")
            (n,) = struct.unpack("<Q", head)
            size = self.path.stat().st_size
            if n > size - 8:
                raise SafetensorsError(f"{self.path}: header length {n} exceeds the file")
            try:
                header = json.loads(f.read(n))
            except json.JSONDecodeError as e:
                raise SafetensorsError(f"{self.path}: header is not JSON ({e})") from None
        self.data_start = 8 + n
        self.metadata = header.pop("__metadata__", {})
        self.tensors: dict[str, TensorInfo] = {}
        for name, meta in header.items():
            if meta["dtype"] not in DTYPES:
                raise SafetensorsError(f"{self.path}: tensor {name} has unsupported dtype {meta['dtype']}")
            begin, end = meta["data_offsets"]
            info = TensorInfo(name, DTYPES[meta["dtype"]], tuple(meta["shape"]), begin, end, self.path)
            want = info.dtype.itemsize
            for s in info.shape:
                want *= s
            if end - begin != want or self.data_start + end > size:
                raise SafetensorsError(f"{self.path}: tensor {name} has inconsistent offsets")
            self.tensors[name] = info
        self._map = None

    def _mapped(self):
        if self._map is None:
            with open(self.path, "rb") as f:
                self._map = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        return self._map

    def read(self, name: str) -> torch.Tensor:
        info = self.tensors[name]
        if info.end == info.begin:
            return torch.empty(info.shape, dtype=info.dtype)
        buf = self._mapped()[self.data_start + info.begin : self.data_start + info.end]
        return torch.frombuffer(bytearray(buf), dtype=info.dtype).reshape(info.shape)

    def close(self):
        if self._map is not None:
            self._map.close()
            self._map = None


class Checkpoint:
    """All tensors of a model folder: ``model.safetensors`` or the shards its index names."""

    def __init__(self, folder):
        self.folder = Path(folder)
        index = self.folder / "model.safetensors.index.json"
        single = self.folder / "model.safetensors"
        if index.exists():
            names = sorted(set(json.loads(index.read_text())["weight_map"].values()))
            paths = [self.folder / n for n in names]
        elif single.exists():
            paths = [single]
        else:
            paths = sorted(self.folder.glob("*.safetensors"))
        if not paths:
            raise SafetensorsError(f"{self.folder}: no model.safetensors found")
        self.files = [SafetensorsFile(p) for p in paths]
        self.tensors: dict[str, tuple[SafetensorsFile, TensorInfo]] = {}
        for f in self.files:
            for name, info in f.tensors.items():
                self.tensors[name] = (f, info)

    def names(self) -> Iterable[str]:
        return self.tensors.keys()

    def info(self, name: str) -> TensorInfo:
        return self.tensors[name][1]

    def read(self, name: str) -> torch.Tensor:
        f, _ = self.tensors[name]
        return f.read(name)

    def close(self):
        for f in self.files:
            f.close()


def write_safetensors(path, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] | None = None):
    """Write tensors (CPU, any supported dtype) in the order given."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in NAMES:
            raise SafetensorsError(f"tensor {name}: dtype {t.dtype} cannot be stored")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    head = json.dumps(header, separators=(",", ":")).encode()
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for raw in blobs:
            f.write(raw)
