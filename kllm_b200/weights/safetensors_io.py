"""Reading and writing safetensors files without a library.

Format: 8-byte little-endian header length, a JSON header (tensor name ->
dtype, shape, data_offsets relative to the end of the header), then the raw
little-endian data.  The checks follow the reference's reader
(engine/loader/safetensors.go:105-177): header length within 512 MiB and within
the file, a known dtype, no negative or overflowing dimension, offsets inside the
data section, and end - begin == numel * element size.  A model folder is a single
``model.safetensors``, or shards named by ``model.safetensors.index.json``, or every
``*.safetensors`` in the folder in sorted order; a tensor name in two shards is an
error (:240-294).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass
from typing import Dict, Iterable, Iterator, List, Tuple

import torch

MAX_HEADER = 512 << 20

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int  # absolute file offsets
    end: int
    path: str


class SafetensorsFile:
    """One file, memory-mapped; tensors are read lazily by name."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors header")
        self._fh = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen > MAX_HEADER or 8 + hlen > size:
            self._fh.close()
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file or 512 MiB")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            self._fh.close()
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        if not isinstance(header, dict):
            self._fh.close()
            raise SafetensorsError(f"{path}: header is not an object")
        data_start = 8 + hlen
        data_len = size - data_start
        self.entries: Dict[str, TensorEntry] = {}
        try:
            for name, ent in header.items():
                if name == "__metadata__":
                    continue
                self.entries[name] = _parse_entry(path, name, ent, data_start, data_len)
        except SafetensorsError:
            self._fh.close()
            raise
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> List[str]:
        return sorted(self.entries)

    def read(self, name: str, copy: bool = True) -> torch.Tensor:
        """The tensor on the CPU.  ``copy=False`` returns a read-only view of the
        mapping, which must be dropped before ``close()``."""
        e = self.entries[name]
        numel = 1
        for s in e.shape:
            numel *= s
        if numel == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the mapping is read-only
            t = torch.frombuffer(self._mm, dtype=e.dtype, count=numel, offset=e.begin).reshape(e.shape)
        return t.clone() if copy else t

    def close(self):
        if getattr(self, "_mm", None) is not None:
            self._mm.close()
            self._mm = None
        self._fh.close()


def _parse_entry(path, name, ent, data_start, data_len) -> TensorEntry:
    if not isinstance(ent, dict):
        raise SafetensorsError(f"{path}: entry {name!r} is not an object")
    dt = ent.get("dtype")
    if dt not in _DTYPES:
        raise SafetensorsError(f"{path}: tensor {name!r} has unknown dtype {dt!r}")
    dtype, esize = _DTYPES[dt]
    shape = ent.get("shape")
    if not isinstance(shape, list) or any(isinstance(s, bool) or not isinstance(s, int) for s in shape):
        raise SafetensorsError(f"{path}: tensor {name!r} has a malformed shape {shape!r}")
    numel = 1
    for s in shape:
        if s < 0:
            raise SafetensorsError(f"{path}: tensor {name!r} has a negative dimension")
        numel *= s
        if numel > (1 << 62):
            raise SafetensorsError(f"{path}: tensor {name!r} overflows")
    off = ent.get("data_offsets")
    if (not isinstance(off, list) or len(off) != 2
            or any(isinstance(o, bool) or not isinstance(o, int) for o in off)):
        raise SafetensorsError(f"{path}: tensor {name!r} has malformed data_offsets")
    b, e = off
    if b < 0 or e < b or e > data_len:
        raise SafetensorsError(f"{path}: tensor {name!r} data [{b},{e}) lies outside the file")
    if e - b != numel * esize:
        raise SafetensorsError(
            f"{path}: tensor {name!r} has {e - b} bytes for {numel} elements of {esize} bytes")
    return TensorEntry(name, dtype, tuple(shape), data_start + b, data_start + e, path)


class ModelFiles:
    """All safetensors of a model folder behind one name -> tensor view."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self.files: List[SafetensorsFile] = []
        self.where: Dict[str, SafetensorsFile] = {}
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.isfile(single):
            paths = [single]
        elif os.path.isfile(index):
            try:
                with open(index, "r", encoding="utf-8") as f:
                    wm = json.load(f)["weight_map"]
                paths = [os.path.join(model_dir, p) for p in sorted(set(wm.values()))]
            except (KeyError, json.JSONDecodeError, AttributeError, TypeError) as e:
                raise SafetensorsError(f"{index}: no usable weight_map: {e}") from None
        else:
            try:
                listing = sorted(os.listdir(model_dir))
            except OSError as e:
                raise SafetensorsError(f"{model_dir}: {e}") from None
            paths = [os.path.join(model_dir, p) for p in listing if p.endswith(".safetensors")]
            if not paths:
                raise SafetensorsError(f"{model_dir}: no safetensors file")
        try:
            for p in paths:
                if not os.path.isfile(p):
                    raise SafetensorsError(f"{p}: shard named by the index is missing")
                f = SafetensorsFile(p)
                self.files.append(f)
                for name in f.entries:
                    if name in self.where:
                        raise SafetensorsError(
                            f"tensor {name!r} is in both {self.where[name].path} and {p}")
                    self.where[name] = f
        except SafetensorsError:
            self.close()
            raise

    def names(self) -> List[str]:
        return sorted(self.where)

    def entry(self, name: str) -> TensorEntry:
        return self.where[name].entries[name]

    def read(self, name: str, copy: bool = True) -> torch.Tensor:
        return self.where[name].read(name, copy=copy)

    def close(self):
        for f in self.files:
            f.close()
        self.files = []

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, Tuple[int, ...], torch.dtype]],
                      produce) -> None:
    """Stream a file: ``tensors`` lists (name, shape, dtype) in file order and
    ``produce(name)`` returns each CPU tensor when its turn comes, so only one
    tensor is held in memory at a time."""
    header = {}
    offset = 0
    order = []
    for name, shape, dtype in tensors:
        if dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {dtype}")
        numel = 1
        for s in shape:
            numel *= int(s)
        nbytes = numel * _DTYPES[_NAMES[dtype]][1]
        header[name] = {"dtype": _NAMES[dtype], "shape": [int(s) for s in shape],
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        order.append((name, tuple(int(s) for s in shape), dtype, nbytes))
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".part"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, shape, dtype, nbytes in order:
            t = produce(name)
            if tuple(t.shape) != shape or t.dtype != dtype:
                raise SafetensorsError(f"tensor {name!r}: produced {tuple(t.shape)} {t.dtype}, "
                                       f"declared {shape} {dtype}")
            t = t.contiguous().cpu()
            raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
            if len(raw) != nbytes:
                raise SafetensorsError(f"tensor {name!r}: {len(raw)} bytes, expected {nbytes}")
            f.write(raw)
    os.replace(tmp, path)


def save_tensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    write_safetensors(path, [(n, tuple(t.shape), t.dtype) for n, t in tensors.items()],
                      lambda n: tensors[n])
