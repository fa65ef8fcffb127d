"""Reading and writing the safetensors container (header JSON + raw little-endian data).

The reference's container is GGUF (garuda/src/gguf/mod.rs:247-329: a
bounds-checked header, then tensors looked up by name, :400-402). This is the
same job for the safetensors layout: an 8-byte little-endian header length, a
JSON object ``name -> {dtype, shape, data_offsets}``, then the bytes.
Every offset is checked against the file before it is used
(garuda/src/gguf/mod.rs:393-395 refuses data past the end of the file).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "F64": (torch.float64, 8),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
    "I8": (torch.int8, 1),
    "I16": (torch.int16, 2),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int
    file: str

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype][0]


class SafetensorsFile:
    """One memory-mapped .safetensors file."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._fh = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open {path}: {e}") from None
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to hold a safetensors header")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} runs past the end of the file")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        self.data_start = 8 + hlen
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: Dict[str, TensorEntry] = {}
        data_len = size - self.data_start
        for name, info in header.items():
            dtype = info.get("dtype")
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dtype!r}")
            shape = tuple(int(s) for s in info["shape"])
            begin, end = (int(v) for v in info["data_offsets"])
            count = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if begin < 0 or end < begin or end > data_len:
                raise SafetensorsError(f"{path}: tensor '{name}' data [{begin},{end}) lies outside the file")
            if end - begin != count * _DTYPES[dtype][1]:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' has {end - begin} bytes for shape {list(shape)} of {dtype}")
            self.entries[name] = TensorEntry(name, dtype, shape, begin, end, path)
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (read-only; copy before writing)."""
        e = self.entries[name]
        count = int(np.prod(e.shape, dtype=np.int64)) if e.shape else 1
        if count == 0:
            return torch.empty(e.shape, dtype=e.torch_dtype)
        buf = memoryview(self._map)[self.data_start + e.begin: self.data_start + e.end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the mapping is read-only; nothing writes through it
            t = torch.frombuffer(buf, dtype=e.torch_dtype, count=count)
        return t.reshape(e.shape)


class SafetensorsFolder:
    """All tensors of a model folder: ``model.safetensors`` or the files its
    ``model.safetensors.index.json`` names."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self.files: Dict[str, SafetensorsFile] = {}
        self.entries: Dict[str, TensorEntry] = {}
        if os.path.exists(index):
            with open(index, "r", encoding="utf-8") as f:
                weight_map = json.load(f).get("weight_map", {})
            for fname in sorted(set(weight_map.values())):
                self._add(os.path.join(model_dir, fname))
        elif os.path.exists(single):
            self._add(single)
        else:
            raise SafetensorsError(f"{model_dir} holds neither model.safetensors nor model.safetensors.index.json")

    def _add(self, path: str) -> None:
        f = SafetensorsFile(path)
        self.files[path] = f
        for name, e in f.entries.items():
            if name in self.entries:
                raise SafetensorsError(f"tensor '{name}' appears in both {self.entries[name].file} and {path}")
            self.entries[name] = e

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def tensor(self, name: str) -> torch.Tensor:
        return self.files[self.entries[name].file].tensor(name)


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    """Write CPU tensors, in the given order, as one safetensors file."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes()
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
