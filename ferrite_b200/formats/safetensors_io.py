"""safetensors reader and writer (single files and sharded folders with `model.safetensors.index.json`).

Reads tensors straight out of a memory map, so a 50 GB checkpoint costs page cache, not heap; `posix_fadvise
(DONTNEED)` after each tensor keeps the page cache from filling (reference: pread through a pinned stage +
`posix_fadvise`, `crates/fe-model/src/safetensors.rs:41-128`)."""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterator, List, Optional, Tuple

import numpy as np
import torch

_DTYPES = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
           "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
           "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2,
           "U16": torch.uint16, "U32": torch.uint32}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafeFile:
    def __init__(self, path: str):
        self.path = path
        self.f = open(path, "rb")
        n = struct.unpack("<Q", self.f.read(8))[0]
        self.header = json.loads(self.f.read(n))
        self.base = 8 + n
        self.meta = self.header.pop("__metadata__", {})
        self.mm = mmap.mmap(self.f.fileno(), 0, access=mmap.ACCESS_READ)

    def names(self) -> List[str]:
        return list(self.header)

    def info(self, name: str) -> Tuple[str, List[int], int, int]:
        h = self.header[name]
        a, b = h["data_offsets"]
        return h["dtype"], h["shape"], self.base + a, b - a

    def get(self, name: str) -> torch.Tensor:
        dt, shape, off, nbytes = self.info(name)
        dtype = _DTYPES[dt]
        buf = np.frombuffer(self.mm, dtype=np.uint8, count=nbytes, offset=off)
        t = torch.from_numpy(buf.copy()).view(dtype).reshape(shape)
        try:
            os.posix_fadvise(self.f.fileno(), off, nbytes, os.POSIX_FADV_DONTNEED)
        except (AttributeError, OSError):
            pass
        return t

    def close(self) -> None:
        self.mm.close()
        self.f.close()


class SafeTensors:
    """All `.safetensors` files of a folder behind one name -> tensor lookup (reference `SafeTensors::open_dir`)."""

    def __init__(self, path: str):
        self.files: List[SafeFile] = []
        self.where: Dict[str, int] = {}
        paths = [path] if os.path.isfile(path) else sorted(
            os.path.join(path, f) for f in os.listdir(path) if f.endswith(".safetensors"))
        if not paths:
            raise FileNotFoundError(f"no .safetensors under {path}")
        for i, p in enumerate(paths):
            sf = SafeFile(p)
            self.files.append(sf)
            for n in sf.names():
                self.where[n] = i

    def has(self, name: str) -> bool:
        return name in self.where

    def names(self) -> List[str]:
        return list(self.where)

    def shape(self, name: str) -> List[int]:
        return self.files[self.where[name]].info(name)[1]

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.files[self.where[name]].info(name)[0]]

    def get(self, name: str) -> torch.Tensor:
        return self.files[self.where[name]].get(name)

    def cat(self, names: List[str], dim: int = 0) -> torch.Tensor:
        """Concatenate several tensors (fused projections are stored separately in HF checkpoints)."""
        return torch.cat([self.get(n) for n in names], dim)

    def close(self) -> None:
        for f in self.files:
            f.close()


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None) -> None:
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = metadata
    off = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
