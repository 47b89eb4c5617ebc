"""Reading and writing the safetensors container: an 8-byte little-endian header
length, a JSON header {name: {dtype, shape, data_offsets}}, then the raw bytes.
A model folder holds `model.safetensors`, or `model.safetensors.index.json` naming
shards (the two layouts the reference opens,
crates/braidinfer-core/src/safetensors.rs:102-158).  Files are memory-mapped and a
tensor is a view of the map until it is copied to the device.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Mapping, Tuple

import numpy as np
import torch

_DTYPES = {
    "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One memory-mapped .safetensors file."""

    def __init__(self, path: str) -> None:
        self.path = path
        self._f = open(path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (n,) = struct.unpack("<Q", self._map[:8])
        if 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file size {size}")
        try:
            header = json.loads(self._map[8:8 + n].decode("utf-8"))
        except Exception as e:
            raise SafetensorsError(f"{path}: the header is not valid JSON: {e}") from None
        self.metadata = header.pop("__metadata__", {})
        self.entries: Dict[str, dict] = header
        self._base = 8 + n
        self._size = size

    def names(self) -> List[str]:
        return list(self.entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        e = self.entries[name]
        if e["dtype"] not in _DTYPES:
            raise SafetensorsError(f"{self.path}: tensor {name} has unsupported dtype {e['dtype']}")
        return _DTYPES[e["dtype"]], tuple(e["shape"])

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped bytes (read-only; copy before writing)."""
        dtype, shape = self.info(name)
        b, e = self.entries[name]["data_offsets"]
        numel = int(np.prod(shape)) if shape else 1
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        if e - b != nbytes or self._base + e > self._size:
            raise SafetensorsError(f"{self.path}: tensor {name} spans {e - b} bytes, its shape needs {nbytes}")
        if numel == 0:
            return torch.empty(shape, dtype=dtype)
        buf = memoryview(self._map)[self._base + b:self._base + e]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)     # the map is read-only on purpose
            return torch.frombuffer(buf, dtype=dtype, count=numel).reshape(shape)

    def close(self) -> None:
        try:
            self._map.close()
        except BufferError:
            pass            # views of the map are still alive; the OS unmaps at exit
        self._f.close()


def open_model_folder(folder: str) -> Dict[str, Tuple[SafetensorsFile, str]]:
    """name -> (file, name) for every tensor of a model folder."""
    single = os.path.join(folder, "model.safetensors")
    index = os.path.join(folder, "model.safetensors.index.json")
    out: Dict[str, Tuple[SafetensorsFile, str]] = {}
    if os.path.isfile(single):
        f = SafetensorsFile(single)
        for n in f.names():
            out[n] = (f, n)
        return out
    if os.path.isfile(index):
        with open(index) as fh:
            wm = json.load(fh).get("weight_map", {})
        files: Dict[str, SafetensorsFile] = {}
        for n, shard in wm.items():
            if shard not in files:
                files[shard] = SafetensorsFile(os.path.join(folder, shard))
            if n not in files[shard].entries:
                raise SafetensorsError(f"{index}: {n} is mapped to {shard}, which does not hold it")
            out[n] = (files[shard], n)
        return out
    raise FileNotFoundError(f"{folder}: neither model.safetensors nor model.safetensors.index.json")


def save_file(tensors: Mapping[str, torch.Tensor], path: str, metadata: Mapping[str, str] = None) -> None:
    """Write tensors (CPU) to `path` in the order given."""
    header = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    off = 0
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store {name} of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, t in tensors.items():
            c = t.detach().contiguous().cpu()
            if c.numel():
                f.write(c.reshape(-1).view(torch.uint8).numpy().tobytes())
