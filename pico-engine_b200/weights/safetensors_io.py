"""Reading and writing the safetensors container: an 8-byte little-endian header length,
a JSON header ``{name: {dtype, shape, data_offsets}}`` and the raw little-endian data.

This replaces pico-engine's GGUF parser and dequantizer (src/pico_engine/gguf.py,
src/pico_engine/dequant.py; tensors are read by name there too, engine.py:80-98); nothing
quantized is read here.
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

_NP_OF = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I64": np.int64,
          "I32": np.int32, "I16": np.int16, "I8": np.int8, "U8": np.uint8, "BOOL": np.bool_}
_NAME_OF_TORCH = {torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
                  torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8",
                  torch.uint8: "U8", torch.bool: "BOOL"}
_ITEMSIZE = {k: np.dtype(v).itemsize for k, v in _NP_OF.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str                     # safetensors dtype string, e.g. "BF16"
    shape: Tuple[int, ...]
    begin: int                     # byte offsets within the file's data section
    end: int
    file: str


class SafetensorsFile:
    """One ``.safetensors`` file, memory-mapped; tensors are materialised on ``read``."""

    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) != 8:
                raise SafetensorsError(f"{path}: too short for a safetensors header")
            (n,) = struct.unpack("<Q", head)
            size = os.path.getsize(path)
            if n <= 0 or 8 + n > size:
                raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
            try:
                header = json.loads(f.read(n).decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as e:
                raise SafetensorsError(f"{path}: header is not JSON: {e}") from None
        self._data_start = 8 + n
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            dt, shape, (b, e) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            if dt not in _NP_OF:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt}")
            count = 1
            for s in shape:
                count *= s
            if e - b != count * _ITEMSIZE[dt] or self._data_start + e > size:
                raise SafetensorsError(f"{path}: tensor {name!r} {dt}{list(shape)} does not match its "
                                       f"data_offsets [{b}, {e}]")
            self.entries[name] = TensorEntry(name, dt, shape, b, e, path)
        self._mmap = None

    def _map(self):
        if self._mmap is None:
            with open(self.path, "rb") as f:
                self._mmap = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        return self._mmap

    def read(self, name: str) -> torch.Tensor:
        """The tensor as stored (a private copy in host memory)."""
        e = self.entries[name]
        arr = np.frombuffer(self._map(), dtype=_NP_OF[e.dtype], count=(e.end - e.begin) // _ITEMSIZE[e.dtype],
                            offset=self._data_start + e.begin)
        t = torch.from_numpy(arr.copy()).reshape(e.shape)
        return t.view(torch.bfloat16) if e.dtype == "BF16" else t


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata: dict | None = None) -> None:
    """Write ``(name, tensor)`` pairs in the given order."""
    items = [(n, t.detach().to("cpu").contiguous()) for n, t in tensors]
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    for name, t in items:
        if t.dtype not in _NAME_OF_TORCH:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAME_OF_TORCH[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-(8 + len(blob)) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in items:
            raw = t.view(torch.uint16) if t.dtype == torch.bfloat16 else t
            f.write(raw.numpy().tobytes())
    os.replace(tmp, path)


class Checkpoint:
    """All tensors of a model folder: ``model.safetensors``, or the files named by
    ``model.safetensors.index.json``."""

    def __init__(self, folder: str):
        self.folder = folder
        single = os.path.join(folder, "model.safetensors")
        index = os.path.join(folder, "model.safetensors.index.json")
        if os.path.isfile(single):
            paths = [single]
        elif os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as f:
                names = sorted(set(json.load(f)["weight_map"].values()))
            paths = [os.path.join(folder, n) for n in names]
        else:
            raise SafetensorsError(f"no model.safetensors (or model.safetensors.index.json) in {folder!r}")
        self.files = [SafetensorsFile(p) for p in paths]
        self.entries: Dict[str, TensorEntry] = {}
        self._file_of: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for name, e in f.entries.items():
                if name in self.entries:
                    raise SafetensorsError(f"tensor {name!r} is stored twice ({self.entries[name].file}, {f.path})")
                self.entries[name] = e
                self._file_of[name] = f

    def read(self, name: str) -> torch.Tensor:
        return self._file_of[name].read(name)
