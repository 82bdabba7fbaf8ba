"""Reading and writing the safetensors container: an 8-byte little-endian header length,
a JSON header (name -> dtype, shape, data_offsets), then the raw little-endian tensor
bytes.  Tensors are read through a memory map, by name."""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Tuple

import numpy as np
import torch

_NP = {"F32": np.float32, "F16": np.float16, "F64": np.float64, "I32": np.int32, "I64": np.int64,
       "I16": np.int16, "I8": np.int8, "U8": np.uint8, "BOOL": np.bool_}
_TORCH_TO_ST = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.float64: "F64",
                torch.int32: "I32", torch.int64: "I64", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8"}


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        head = self._f.read(8)
        if len(head) < 8:
            raise ValueError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", head)
        size = os.path.getsize(path)
        if n > size - 8:
            raise ValueError(f"{path}: header length {n} exceeds the file")
        try:
            header = json.loads(self._f.read(n))
        except json.JSONDecodeError as e:
            raise ValueError(f"{path}: header is not JSON: {e}") from None
        self.metadata = header.pop("__metadata__", {})
        self.entries: Dict[str, dict] = header
        self.data_start = 8 + n
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        for name, e in self.entries.items():
            a, b = e["data_offsets"]
            if not (0 <= a <= b <= size - self.data_start):
                raise ValueError(f"{path}: tensor '{name}' lies outside the file")

    def names(self):
        return list(self.entries)

    def info(self, name: str) -> Tuple[str, Tuple[int, ...]]:
        e = self.entries[name]
        return e["dtype"], tuple(e["shape"])

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that owns its memory, in the stored dtype."""
        e = self.entries[name]
        a, b = e["data_offsets"]
        shape = tuple(e["shape"])
        dt = e["dtype"]
        buf = memoryview(self._mm)[self.data_start + a:self.data_start + b]
        if dt == "BF16":
            arr = np.frombuffer(buf, dtype=np.int16).reshape(shape)
            return torch.from_numpy(arr.copy()).view(torch.bfloat16)
        if dt not in _NP:
            raise ValueError(f"{self.path}: tensor '{name}' has dtype {dt}, which this loader does not read; "
                             "refusing to load rather than misread it")
        arr = np.frombuffer(buf, dtype=_NP[dt]).reshape(shape)
        return torch.from_numpy(arr.copy())

    def close(self):
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _TORCH_TO_ST:
            raise ValueError(f"cannot store tensor '{name}' of dtype {t.dtype}")
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        header[name] = {"dtype": _TORCH_TO_ST[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)
