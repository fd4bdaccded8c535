"""GGUF v2/v3 reader (header, key/value metadata, tensor infos, shards, mmap) and block decoders for the ggml
quantisation types, plus simple encoders and a writer used by the tests.

Counterparts in the reference: `crates/fe-gguf/src/lib.rs` (`Gguf`, `TensorInfo`, `GgmlType::block`) and the host
dequantisers of `crates/fe-ggq/src/refq.rs` (device side `kernels/k-gguf/src/dec.rs`, `vq.rs`, `tables.rs`). Decoders
follow ggml's public `dequantize_row_*` definitions, the codebook types (IQ1_S/M, IQ2_XXS/XS/S, IQ3_XXS/S) through the
grids of `gguf_tables.py`; the tests hold every decoder to the `gguf` Python package's own dequantiser, bit for bit."""
from __future__ import annotations

import mmap
import os
import struct
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch

GGUF_MAGIC = 0x46554747
# type id -> (name, values per block, bytes per block)
TYPES: Dict[int, Tuple[str, int, int]] = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22), 7: ("Q5_1", 32, 24),
    8: ("Q8_0", 32, 34), 9: ("Q8_1", 32, 36), 10: ("Q2_K", 256, 84), 11: ("Q3_K", 256, 110), 12: ("Q4_K", 256, 144),
    13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210), 15: ("Q8_K", 256, 292), 16: ("IQ2_XXS", 256, 66), 17: ("IQ2_XS", 256, 74),
    18: ("IQ3_XXS", 256, 98), 19: ("IQ1_S", 256, 50), 20: ("IQ4_NL", 32, 18), 21: ("IQ3_S", 256, 110), 22: ("IQ2_S", 256, 82),
    23: ("IQ4_XS", 256, 136), 24: ("I8", 1, 1), 25: ("I16", 1, 2), 26: ("I32", 1, 4), 27: ("I64", 1, 8), 28: ("F64", 1, 8),
    29: ("IQ1_M", 256, 56), 30: ("BF16", 1, 2), 39: ("MXFP4", 32, 17), 42: ("Q2_0", 64, 18),
}
TYPE_ID = {v[0]: k for k, v in TYPES.items()}
KVALUES_IQ4NL = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.float32)
KVALUES_MXFP4 = np.array([0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12], dtype=np.float32)


@dataclass
class TensorInfo:
    name: str
    shape: List[int]          # ggml order reversed to row-major: [rows..., cols]
    type_id: int
    offset: int               # absolute file offset
    nbytes: int
    shard: int = 0

    @property
    def type_name(self) -> str:
        return TYPES[self.type_id][0]


class _Reader:
    def __init__(self, mm, pos=0):
        self.mm, self.pos = mm, pos

    def u(self, fmt):
        n = struct.calcsize(fmt)
        v = struct.unpack_from(fmt, self.mm, self.pos)[0]
        self.pos += n
        return v

    def string(self):
        n = self.u("<Q")
        s = bytes(self.mm[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, t):
        fmts = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
        if t in fmts:
            return self.u(fmts[t])
        if t == 8:
            return self.string()
        if t == 9:
            et, n = self.u("<I"), self.u("<Q")
            if et in fmts and et != 7:
                code = fmts[et][1]
                arr = np.frombuffer(self.mm, dtype=np.dtype("<" + code), count=n, offset=self.pos)
                self.pos += arr.nbytes
                return arr.tolist() if n <= 1 << 16 else arr.copy()
            return [self.value(et) for _ in range(n)]
        raise ValueError(f"unknown GGUF value type {t}")


class Gguf:
    def __init__(self, path: str):
        self.paths = [path]
        self.files, self.mms = [], []
        self.meta: Dict[str, Any] = {}
        self.tensors: Dict[str, TensorInfo] = {}
        self._open(path, 0)
        n_split = int(self.meta.get("split.count", 1) or 1)
        if n_split > 1 and "-00001-of-" in path:
            for i in range(2, n_split + 1):
                p = path.replace("-00001-of-", f"-{i:05d}-of-")
                self.paths.append(p)
                self._open(p, i - 1)

    def _open(self, path: str, shard: int) -> None:
        f = open(path, "rb")
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        self.files.append(f)
        self.mms.append(mm)
        r = _Reader(mm)
        if r.u("<I") != GGUF_MAGIC:
            raise ValueError(f"{path}: not a GGUF file")
        version = r.u("<I")
        if version not in (2, 3):
            raise ValueError(f"{path}: GGUF version {version} not supported")
        n_t, n_kv = r.u("<Q"), r.u("<Q")
        meta = {}
        for _ in range(n_kv):
            k = r.string()
            meta[k] = r.value(r.u("<I"))
        if shard == 0:
            self.meta = meta
            self.version = version
        infos = []
        for _ in range(n_t):
            name = r.string()
            nd = r.u("<I")
            dims = [r.u("<Q") for _ in range(nd)]
            tid, off = r.u("<I"), r.u("<Q")
            infos.append((name, dims, tid, off))
        align = int(meta.get("general.alignment", 32))
        base = (r.pos + align - 1) // align * align
        for name, dims, tid, off in infos:
            if tid not in TYPES:
                raise ValueError(f"{name}: unknown ggml type {tid}")
            _, bv, bb = TYPES[tid]
            n = int(np.prod(dims)) if dims else 1
            self.tensors[name] = TensorInfo(name, list(reversed(dims)), tid, base + off, n // bv * bb, shard)

    def raw(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        return np.frombuffer(self.mms[t.shard], dtype=np.uint8, count=t.nbytes, offset=t.offset)

    def get(self, name: str, dtype=torch.float32) -> torch.Tensor:
        t = self.tensors[name]
        return torch.from_numpy(dequantize(self.raw(name), t.type_id)).reshape(t.shape).to(dtype)

    def close(self) -> None:
        for mm in self.mms:
            mm.close()
        for f in self.files:
            f.close()


# ---- block decoders -------------------------------------------------------------------------------------

def _f16(b: np.ndarray) -> np.ndarray:
    return b.copy().view(np.float16).astype(np.float32)


def _scale_min_k4(sc: np.ndarray):
    """The 8 six-bit (scale, min) pairs packed in 12 bytes of a K-quant super-block. sc: [nb, 12] -> two [nb, 8]."""
    s = np.empty(sc.shape[:-1] + (8,), np.float32)
    m = np.empty_like(s)
    for j in range(8):
        if j < 4:
            s[..., j] = sc[..., j] & 63
            m[..., j] = sc[..., j + 4] & 63
        else:
            s[..., j] = (sc[..., j + 4] & 0xF) | ((sc[..., j - 4] >> 6) << 4)
            m[..., j] = (sc[..., j + 4] >> 4) | ((sc[..., j] >> 6) << 4)
    return s, m


_NATIVE_TYPES = ("Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "IQ4_NL", "IQ4_XS",
                 "IQ2_XXS", "IQ2_XS", "IQ2_S", "IQ3_XXS", "IQ3_S", "IQ1_S", "IQ1_M")
_NATIVE_GRID = {"IQ2_XXS": "iq2xxs", "IQ2_XS": "iq2xs", "IQ2_S": "iq2s", "IQ3_XXS": "iq3xxs", "IQ3_S": "iq3s", "IQ1_S": "iq1s",
                "IQ1_M": "iq1s"}
_native_tables: Dict[str, Any] = {}


def _native_args(name: str):
    """The tables a C++ decoder wants beside the bytes (codebook, sign masks, 4-bit levels), as tensors made once."""
    import torch
    if name in ("IQ4_NL", "IQ4_XS"):
        if "kvalues" not in _native_tables:
            _native_tables["kvalues"] = torch.from_numpy(KVALUES_IQ4NL.copy())
        return _native_tables["kvalues"], None
    key = _NATIVE_GRID.get(name)
    if key is None:
        return None, None
    if key not in _native_tables:
        from .gguf_tables import GRID, KSIGNS
        _native_tables[key] = torch.from_numpy(np.ascontiguousarray(GRID[key], dtype=np.int8))
        _native_tables.setdefault("ksigns", torch.from_numpy(np.ascontiguousarray(KSIGNS, dtype=np.uint8)))
    return _native_tables[key], _native_tables["ksigns"]


def dequantize(raw: np.ndarray, type_id: int) -> np.ndarray:
    name, bv, bb = TYPES[type_id]
    if name == "F32":
        return raw.view(np.float32).copy()
    if name == "F16":
        return raw.view(np.float16).astype(np.float32)
    if name == "BF16":
        return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
    if name in ("I8", "I16", "I32", "I64", "F64"):
        return raw.view({"I8": np.int8, "I16": np.int16, "I32": np.int32, "I64": np.int64, "F64": np.float64}[name]).astype(np.float32)
    if name in _NATIVE_TYPES:
        # block formats decode in C++ (`csrc/host_gguf.cpp`) when the extension is built: the same bits as the statements
        # below, without their temporaries, the blocks spread over the host's cores
        from .._ext import host
        h = host()
        if h is not None and hasattr(h, "gguf_dequant_host"):
            import torch
            grid, ksigns = _native_args(name)
            flat = np.ascontiguousarray(raw).reshape(-1).view(np.uint8)
            if not flat.flags.writeable:
                flat = flat.copy()                           # torch wants a writable buffer (a read-only mmap is not one)
            return h.gguf_dequant_host(torch.from_numpy(flat), name, grid, ksigns).numpy()
    b = raw.reshape(-1, bb)
    nb = b.shape[0]
    if name == "Q8_0":
        return (_f16(b[:, :2]) * b[:, 2:].view(np.int8).astype(np.float32)).reshape(-1)
    if name in ("Q4_0", "Q4_1", "IQ4_NL"):
        d = _f16(b[:, :2])
        o = 2
        m = None
        if name == "Q4_1":
            m = _f16(b[:, 2:4])
            o = 4
        qs = b[:, o:o + 16]
        lo, hi = (qs & 0xF), (qs >> 4)
        q = np.concatenate([lo, hi], 1)
        if name == "Q4_0":
            return (d * (q.astype(np.float32) - 8)).reshape(-1)
        if name == "Q4_1":
            return (d * q.astype(np.float32) + m).reshape(-1)
        return (d * KVALUES_IQ4NL[q]).reshape(-1)
    if name in ("Q5_0", "Q5_1"):
        d = _f16(b[:, :2])
        o = 2
        m = None
        if name == "Q5_1":
            m = _f16(b[:, 2:4])
            o = 4
        qh = b[:, o:o + 4].copy().view(np.uint32)[:, 0]
        qs = b[:, o + 4:o + 20]
        j = np.arange(16)
        h0 = ((qh[:, None] >> j) & 1).astype(np.uint8) << 4
        h1 = ((qh[:, None] >> (j + 16)) & 1).astype(np.uint8) << 4
        q = np.concatenate([(qs & 0xF) | h0, (qs >> 4) | h1], 1).astype(np.float32)
        return (d * (q - 16)).reshape(-1) if name == "Q5_0" else (d * q + m).reshape(-1)
    if name == "MXFP4":
        e = b[:, 0].astype(np.int32)
        d = np.ldexp(np.float32(0.5), e - 127)[:, None].astype(np.float32)
        qs = b[:, 1:17]
        q = np.concatenate([qs & 0xF, qs >> 4], 1)
        return (d * KVALUES_MXFP4[q]).reshape(-1)
    if name == "Q2_0":
        d = _f16(b[:, :2])
        qs = b[:, 2:18]
        q = np.stack([(qs >> s) & 3 for s in (0, 2, 4, 6)], -1).reshape(nb, 64).astype(np.float32)
        return (d * (q - 1)).reshape(-1)
    if name == "Q4_K":
        d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
        s, m = _scale_min_k4(b[:, 4:16])
        qs = b[:, 16:144].reshape(nb, 4, 32)
        lo, hi = (qs & 0xF).astype(np.float32), (qs >> 4).astype(np.float32)
        q = np.stack([lo, hi], 2).reshape(nb, 8, 32)
        return (d[:, :, None] * s[:, :, None] * q - dmin[:, :, None] * m[:, :, None]).reshape(-1)
    if name == "Q5_K":
        d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
        s, m = _scale_min_k4(b[:, 4:16])
        qh = b[:, 16:48]
        qs = b[:, 48:176].reshape(nb, 4, 32)
        out = np.empty((nb, 8, 32), np.float32)
        for j in range(4):
            out[:, 2 * j] = (qs[:, j] & 0xF) + (((qh >> (2 * j)) & 1) << 4)
            out[:, 2 * j + 1] = (qs[:, j] >> 4) + (((qh >> (2 * j + 1)) & 1) << 4)
        return (d[:, :, None] * s[:, :, None] * out - dmin[:, :, None] * m[:, :, None]).reshape(-1)
    if name == "Q6_K":
        ql = b[:, 0:128].reshape(nb, 2, 64)
        qh = b[:, 128:192].reshape(nb, 2, 32)
        sc = b[:, 192:208].view(np.int8).astype(np.float32).reshape(nb, 2, 8)
        d = _f16(b[:, 208:210])
        out = np.empty((nb, 2, 128), np.float32)
        for h in range(2):
            l0, l1, hh = ql[:, h, :32], ql[:, h, 32:], qh[:, h]
            q1 = ((l0 & 0xF) | (((hh >> 0) & 3) << 4)).astype(np.int32) - 32
            q2 = ((l1 & 0xF) | (((hh >> 2) & 3) << 4)).astype(np.int32) - 32
            q3 = ((l0 >> 4) | (((hh >> 4) & 3) << 4)).astype(np.int32) - 32
            q4 = ((l1 >> 4) | (((hh >> 6) & 3) << 4)).astype(np.int32) - 32
            idx = np.arange(32) // 16
            for k, q in enumerate((q1, q2, q3, q4)):
                out[:, h, 32 * k:32 * k + 32] = sc[:, h, idx + 2 * k] * q
        return (d[:, :, None] * out).reshape(-1)
    if name == "IQ4_XS":
        d = _f16(b[:, 0:2])
        sh = b[:, 2:4].copy().view(np.uint16)[:, 0].astype(np.int32)
        sl = b[:, 4:8]
        qs = b[:, 8:136].reshape(nb, 8, 16)
        out = np.empty((nb, 8, 32), np.float32)
        for ib in range(8):
            ls = ((sl[:, ib // 2] >> (4 * (ib % 2))) & 0xF).astype(np.int32) | (((sh >> (2 * ib)) & 3) << 4)
            dl = d[:, 0] * (ls - 32)
            out[:, ib, :16] = dl[:, None] * KVALUES_IQ4NL[qs[:, ib] & 0xF]
            out[:, ib, 16:] = dl[:, None] * KVALUES_IQ4NL[qs[:, ib] >> 4]
        return out.reshape(-1)
    if name == "Q2_K":
        sc, qs = b[:, 0:16], b[:, 16:80].reshape(nb, 2, 32)
        d, dmin = _f16(b[:, 80:82]), _f16(b[:, 82:84])
        out = np.empty((nb, 16, 16), np.float32)
        for n in range(2):
            for j in range(4):
                for half in range(2):
                    i = n * 8 + j * 2 + half
                    q = ((qs[:, n, 16 * half:16 * half + 16] >> (2 * j)) & 3).astype(np.float32)
                    out[:, i] = (d[:, 0] * (sc[:, i] & 0xF))[:, None] * q - (dmin[:, 0] * (sc[:, i] >> 4))[:, None]
        return out.reshape(-1)
    if name == "Q3_K":
        hm, qs = b[:, 0:32], b[:, 32:96].reshape(nb, 2, 32)
        aux = b[:, 96:108].copy().view(np.uint32)                         # [nb, 3]
        d = _f16(b[:, 108:110])
        k1, k2 = np.uint32(0x03030303), np.uint32(0x0F0F0F0F)
        a0, a1, tmp = aux[:, 0], aux[:, 1], aux[:, 2]
        sc = np.stack([(a0 & k2) | (((tmp >> 0) & k1) << 4), (a1 & k2) | (((tmp >> 2) & k1) << 4),
                       ((a0 >> 4) & k2) | (((tmp >> 4) & k1) << 4), ((a1 >> 4) & k2) | (((tmp >> 6) & k1) << 4)], 1)
        sc = np.ascontiguousarray(sc).view(np.int8).astype(np.float32) - 32.0             # [nb, 16]
        out = np.empty((nb, 16, 16), np.float32)
        for n in range(2):
            for j in range(4):
                bit = np.uint8(1 << (n * 4 + j))
                for half in range(2):
                    i = n * 8 + j * 2 + half
                    q = ((qs[:, n, 16 * half:16 * half + 16] >> (2 * j)) & 3).astype(np.float32)
                    q = q - np.where(hm[:, 16 * half:16 * half + 16] & bit, 0.0, 4.0).astype(np.float32)
                    out[:, i] = (d[:, 0] * sc[:, i])[:, None] * q
        return out.reshape(-1)
    if name in ("IQ2_XXS", "IQ2_XS", "IQ2_S", "IQ3_XXS", "IQ3_S", "IQ1_S", "IQ1_M"):
        return _dequantize_iq(b, name)
    raise NotImplementedError(f"ggml type {name} has no decoder here")


def _signs(mask: np.ndarray) -> np.ndarray:
    """8-bit sign masks [...] -> [..., 8] of +1 / -1 (bit j set = value j negative)."""
    return np.where((mask[..., None] >> np.arange(8, dtype=np.uint8)) & 1, np.float32(-1), np.float32(1))


def _dequantize_iq(b: np.ndarray, name: str) -> np.ndarray:
    """The codebook ("IQ") super-blocks of 256 values: grid entries picked by index bits, signs, and sub-block scales."""
    from .gguf_tables import GRID, KSIGNS
    nb = b.shape[0]
    d = _f16(b[:, 0:2])[:, 0] if name != "IQ1_M" else None
    if name == "IQ2_XXS":
        q32 = b[:, 2:66].copy().view(np.uint32).reshape(nb, 8, 2)
        idx = b[:, 2:66].reshape(nb, 8, 8)[:, :, :4]                                   # the 4 grid indices of a group
        db = d[:, None] * (np.float32(0.5) + (q32[:, :, 1] >> 28).astype(np.float32)) * np.float32(0.25)
        sg = KSIGNS[(q32[:, :, 1, None] >> (7 * np.arange(4, dtype=np.uint32))) & 127]  # [nb, 8, 4]
        g = GRID["iq2xxs"][idx].astype(np.float32)                                     # [nb, 8, 4, 8]
        return (db[:, :, None, None] * g * _signs(sg)).reshape(-1)
    if name == "IQ2_XS":
        qs = b[:, 2:66].copy().view(np.uint16).reshape(nb, 8, 4)
        sc = b[:, 66:74]
        db = np.stack([sc & 0xF, sc >> 4], -1).astype(np.float32)                       # [nb, 8, 2]
        db = d[:, None, None] * (np.float32(0.5) + db) * np.float32(0.25)
        g = GRID["iq2xs"][qs & 511].astype(np.float32)
        return (np.repeat(db, 2, -1)[..., None] * g * _signs(KSIGNS[qs >> 9])).reshape(-1)
    if name == "IQ2_S":
        qs, sg = b[:, 2:34].reshape(nb, 8, 4), b[:, 34:66].reshape(nb, 8, 4)
        qh, sc = b[:, 66:74], b[:, 74:82]
        db = np.stack([sc & 0xF, sc >> 4], -1).astype(np.float32)
        db = d[:, None, None] * (np.float32(0.5) + db) * np.float32(0.25)
        hi = (qh[:, :, None].astype(np.uint16) << (8 - 2 * np.arange(4, dtype=np.uint16))) & 0x300
        g = GRID["iq2s"][qs.astype(np.uint16) | hi].astype(np.float32)
        return (np.repeat(db, 2, -1)[..., None] * g * _signs(sg)).reshape(-1)
    if name == "IQ3_XXS":
        qs = b[:, 2:66].reshape(nb, 8, 8)
        aux = b[:, 66:98].copy().view(np.uint32)                                        # [nb, 8]
        db = d[:, None] * (np.float32(0.5) + (aux >> 28).astype(np.float32)) * np.float32(0.5)
        sg = _signs(KSIGNS[(aux[:, :, None] >> (7 * np.arange(4, dtype=np.uint32))) & 127])   # [nb, 8, 4, 8]
        g = GRID["iq3xxs"][qs].astype(np.float32).reshape(nb, 8, 4, 8)                  # two 4-value entries per 8 signs
        return (db[:, :, None, None] * g * sg).reshape(-1)
    if name == "IQ3_S":
        qs, qh = b[:, 2:66].reshape(nb, 8, 8), b[:, 66:74]
        sg, sc = b[:, 74:106].reshape(nb, 8, 4), b[:, 106:110]
        db = np.stack([sc & 0xF, sc >> 4], -1).reshape(nb, 8).astype(np.float32)
        db = d[:, None] * (np.float32(1) + np.float32(2) * db)
        hi = ((qh[:, :, None].astype(np.uint16) << 8) >> np.arange(8, dtype=np.uint16)) & 256   # bit l of qh -> bit 8
        g = GRID["iq3s"][qs.astype(np.uint16) | hi].astype(np.float32).reshape(nb, 8, 4, 8)
        return (db[:, :, None, None] * g * _signs(sg)).reshape(-1)
    delta = np.float32(0.125)
    if name == "IQ1_S":
        qs = b[:, 2:34].reshape(nb, 8, 4)
        qh = b[:, 34:50].copy().view(np.uint16)                                         # [nb, 8]
        dl = d[:, None] * (2 * ((qh >> 12) & 7) + 1).astype(np.float32)
        dlt = np.where(qh & 0x8000, -delta, delta).astype(np.float32)
        idx = qs.astype(np.uint16) | (((qh[:, :, None] >> (3 * np.arange(4, dtype=np.uint16))) & 7) << 8)
        g = GRID["iq1s"][idx].astype(np.float32)                                        # [nb, 8, 4, 8]
        return (dl[:, :, None, None] * (g + dlt[:, :, None, None])).reshape(-1)
    # IQ1_M: the fp16 super-block scale is spread over the top nibbles of the four 16-bit scale words
    qs, qh = b[:, 0:32].reshape(nb, 8, 4), b[:, 32:48].reshape(nb, 8, 2)
    sc = b[:, 48:56].copy().view(np.uint16)                                             # [nb, 4]
    dbits = (sc[:, 0] >> 12) | ((sc[:, 1] >> 8) & 0x00F0) | ((sc[:, 2] >> 4) & 0x0F00) | (sc[:, 3] & 0xF000)
    d = dbits.astype(np.uint16).view(np.float16).astype(np.float32)
    ib = np.arange(8)
    w = sc[:, ib // 2]                                                                  # [nb, 8]
    dl1 = d[:, None] * (2 * ((w >> (6 * (ib % 2))) & 7) + 1).astype(np.float32)
    dl2 = d[:, None] * (2 * ((w >> (6 * (ib % 2) + 3)) & 7) + 1).astype(np.float32)
    dl = np.stack([dl1, dl1, dl2, dl2], -1)                                             # [nb, 8, 4]
    h = np.stack([qh[:, :, 0], qh[:, :, 0] >> 4, qh[:, :, 1], qh[:, :, 1] >> 4], -1).astype(np.uint16)   # 4 nibbles
    idx = qs.astype(np.uint16) | ((h & 7) << 8)
    dlt = np.where(h & 8, -delta, delta).astype(np.float32)
    g = GRID["iq1s"][idx].astype(np.float32)
    return (dl[..., None] * (g + dlt[..., None])).reshape(-1)


# ---- encoders (tests, synthetic checkpoints) and writer -------------------------------------------------------

def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.float32).reshape(-1, 32)
    d = np.abs(x).max(1, keepdims=True) / 127.0
    q = np.where(d > 0, np.round(x / np.where(d > 0, d, 1)), 0).astype(np.int8)
    out = np.empty((x.shape[0], 34), np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.float32).reshape(-1, 32)
    idx = np.abs(x).argmax(1)
    mx = x[np.arange(x.shape[0]), idx]
    d = mx / -8.0
    inv = np.where(d != 0, 1.0 / np.where(d != 0, d, 1), 0)
    q = np.clip(np.floor(x * inv[:, None] + 8.5), 0, 15).astype(np.uint8)
    out = np.empty((x.shape[0], 18), np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


def write_gguf(path: str, meta: Dict[str, Any], tensors: Dict[str, Tuple[np.ndarray, int, List[int]]], align: int = 32) -> None:
    """tensors: name -> (raw block bytes, ggml type id, row-major shape)."""
    def s(x: str) -> bytes:
        b = x.encode()
        return struct.pack("<Q", len(b)) + b

    def kv(k, v) -> bytes:
        if isinstance(v, bool):
            return s(k) + struct.pack("<I?", 7, v)
        if isinstance(v, int):
            return s(k) + struct.pack("<Iq", 11, v) if v < 0 else s(k) + struct.pack("<II", 4, v) if v < 2 ** 32 else s(k) + struct.pack("<IQ", 10, v)
        if isinstance(v, float):
            return s(k) + struct.pack("<If", 6, v)
        if isinstance(v, str):
            return s(k) + struct.pack("<I", 8) + s(v)
        if isinstance(v, list):
            if v and isinstance(v[0], str):
                return s(k) + struct.pack("<IIQ", 9, 8, len(v)) + b"".join(s(x) for x in v)
            return s(k) + struct.pack("<IIQ", 9, 5, len(v)) + struct.pack(f"<{len(v)}i", *v)
        raise TypeError(type(v))

    meta = dict(meta)
    meta.setdefault("general.alignment", align)
    head = struct.pack("<IIQQ", GGUF_MAGIC, 3, len(tensors), len(meta)) + b"".join(kv(k, v) for k, v in meta.items())
    infos, blobs, off = b"", [], 0
    for name, (raw, tid, shape) in tensors.items():
        dims = list(reversed(shape))
        infos += s(name) + struct.pack("<I", len(dims)) + struct.pack(f"<{len(dims)}Q", *dims) + struct.pack("<IQ", tid, off)
        pad = (align - len(raw) % align) % align
        blobs.append(bytes(raw) + b"\0" * pad)
        off += len(raw) + pad
    pos = len(head) + len(infos)
    with open(path, "wb") as f:
        f.write(head + infos + b"\0" * ((align - pos % align) % align))
        for b in blobs:
            f.write(b)
