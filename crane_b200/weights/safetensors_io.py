"""Reading and writing safetensors files by tensor name.

Format: 8 bytes little-endian header length N; N bytes of JSON
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``;
then the raw little-endian tensor data.  Files are memory-mapped; a tensor is
materialised only when it is asked for.

Which files make up a model follows the reference
(crane-core/src/utils/utils.rs:16-57): ``model.safetensors.index.json`` names
the shards in its ``weight_map`` (each must exist), else ``model.safetensors``.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One memory-mapped file: ``names()``, ``info(name)``, ``tensor(name)``."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: truncated (no header length)")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file size {size}")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON: {e}") from None
        self.metadata = header.pop("__metadata__", None) or {}
        self._data_start = 8 + n
        self._entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            dt = _DTYPES.get(e.get("dtype"))
            if dt is None:
                raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype {e.get('dtype')}")
            shape = tuple(int(s) for s in e["shape"])
            b, end = (int(v) for v in e["data_offsets"])
            numel = 1
            for s in shape:
                numel *= s
            width = torch.empty((), dtype=dt).element_size()
            if end - b != numel * width:
                raise SafetensorsError(f"{path}: tensor {name} spans {end - b} bytes, its shape "
                                       f"{list(shape)} of {e['dtype']} needs {numel * width}")
            if self._data_start + end > size:
                raise SafetensorsError(f"{path}: truncated, tensor {name} ends at byte "
                                       f"{self._data_start + end} of {size}")
            self._entries[name] = (dt, shape, b, end)
        # private copy-on-write mapping: torch wants a writable buffer, the file stays untouched
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None

    def names(self) -> List[str]:
        return list(self._entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dt, shape, _, _ = self._entries[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        dt, shape, b, end = self._entries[name]
        if end == b:
            return torch.empty(shape, dtype=dt)
        flat = torch.frombuffer(self._mm, dtype=dt, count=(end - b) // torch.empty((), dtype=dt).element_size(),
                                offset=self._data_start + b)
        return flat.view(shape)

    def close(self) -> None:
        # tensors handed out keep the mapping alive through the buffer protocol
        self._f.close()


def model_files(folder: str) -> List[str]:
    index = os.path.join(folder, "model.safetensors.index.json")
    single = os.path.join(folder, "model.safetensors")
    if os.path.isfile(index):
        with open(index) as f:
            try:
                weight_map = json.load(f)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError) as e:
                raise SafetensorsError(f"{index}: no readable weight_map: {e}") from None
        files = sorted(set(weight_map.values()))
        for name in files:
            if not os.path.isfile(os.path.join(folder, name)):
                raise SafetensorsError(f"Missing shard file: {os.path.join(folder, name)}")
        return [os.path.join(folder, n) for n in files]
    if os.path.isfile(single):
        return [single]
    raise SafetensorsError(f"No valid model files found in {folder}. Need either "
                           "model.safetensors.index.json or model.safetensors")


class TensorSource:
    """All tensors of a model folder by name, over one or more shards."""

    def __init__(self, files: Iterable[str]):
        self.files = [SafetensorsFile(p) for p in files]
        self._where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for n in f.names():
                if n in self._where:
                    raise SafetensorsError(f"tensor {n} is in both {self._where[n].path} and {f.path}")
                self._where[n] = f

    def names(self) -> List[str]:
        return list(self._where)

    def info(self, name: str):
        return self._where[name].info(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)


class DictSource:
    """The same interface over tensors already in memory (random weights)."""

    def __init__(self, tensors: Mapping[str, torch.Tensor]):
        self._t = dict(tensors)

    def names(self) -> List[str]:
        return list(self._t)

    def info(self, name: str):
        t = self._t[name]
        return t.dtype, tuple(t.shape)

    def tensor(self, name: str) -> torch.Tensor:
        return self._t[name]


def _raw_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous().cpu()
    return t.view(torch.uint8).numpy().tobytes() if t.numel() else b""


def save_file(tensors: Mapping[str, torch.Tensor], path: str, metadata=None) -> None:
    """Write tensors (any iteration order; stored sorted by name) to one file."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name}: dtype {t.dtype} cannot be stored")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + n]}
        offset += n
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            f.write(_raw_bytes(tensors[name]))
    os.replace(tmp, path)
