"""Quantised linears as they sit in a checkpoint, kept packed from the file to the kernels.

A `Packed*` object stands where a dense `[out, in]` weight would: it knows its shape, can be cut by output rows and by
input columns (the two cuts tensor parallelism needs), concatenated along the output rows (fused projections such as
q|k|v or gate|up) and dequantised for the fp32 oracle. Nothing here re-quantises: cuts and concatenations move code
bytes and scale bytes only, so what the kernels multiply is what the checkpoint holds.

Reference: the NVFP4 / FP8 side is `HostLinear::load_sliced` (`crates/fe-fp4/src/lib.rs:305-386`: parts fused along N,
one `alpha` per output column because every part brings its own tensor scale, `Slice` = row ranges + a k range), the
EXL3 side `slice_cols` / `slice_rows` and the split table (`crates/fe-exl3/src/format.rs`, `crates/fe-exl3/src/tp.rs`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from . import nvfp4
from .exl3 import Exl3Tensor


def _slice_idx(idx, n: int):
    """Normalise `t[a:b]` / `t[:, a:b]` to ((row lo, row hi) or None, (col lo, col hi) or None)."""
    rows = cols = None
    if isinstance(idx, tuple):
        assert len(idx) == 2 and isinstance(idx[0], slice) and isinstance(idx[1], slice)
        r, c = idx
    else:
        assert isinstance(idx, slice)
        r, c = idx, slice(None)
    assert r.step in (None, 1) and c.step in (None, 1)
    if r != slice(None):
        rows = r
    if c != slice(None):
        cols = c
    return rows, cols


class PackedLinear:
    """Common surface: `.shape == (out, in)`, `t[a:b]` (output rows), `t[:, a:b]` (input columns), `.contiguous()`,
    `.dequantize(dtype)`, `cat(parts)`."""

    kind = "packed"
    rows: int
    cols: int

    @property
    def shape(self):
        return (self.rows, self.cols)

    def dim(self) -> int:
        return 2

    def contiguous(self):
        return self

    def to(self, *a, **k):           # device / dtype moves happen when the engine turns it into a kernel weight
        return self

    def __getitem__(self, idx):
        r, c = _slice_idx(idx, self.rows)
        out = self
        if r is not None:
            lo, hi, _ = r.indices(self.rows)
            out = out.take_rows(lo, hi)
        if c is not None:
            lo, hi, _ = c.indices(self.cols)
            out = out.take_cols(lo, hi)
        return out


@dataclass
class PackedNVFP4(PackedLinear):
    """ModelOpt NVFP4: `packed` uint8 [out, in/2] (element 2i in the low nibble), `scales` uint8 [out, in/16] holding
    e4m3 bits, `alpha` fp32 [out] = the tensor scale (`weight_scale_2`) of the part each row came from, `input_scale`
    the largest static activation scale of the parts (kept for W4A4 consumers that want a static scale; this engine
    quantises activations per row on the fly)."""
    packed: torch.Tensor
    scales: torch.Tensor
    alpha: torch.Tensor
    input_scale: float = 0.0
    kind = "nvfp4"

    @property
    def rows(self):
        return self.packed.shape[0]

    @property
    def cols(self):
        return self.packed.shape[1] * 2

    def take_rows(self, lo, hi):
        return PackedNVFP4(self.packed[lo:hi], self.scales[lo:hi], self.alpha[lo:hi], self.input_scale)

    def take_cols(self, lo, hi):
        assert lo % nvfp4.BLOCK == 0 and hi % nvfp4.BLOCK == 0, "NVFP4 column cuts fall on 16-element blocks"
        return PackedNVFP4(self.packed[:, lo // 2:hi // 2], self.scales[:, lo // nvfp4.BLOCK:hi // nvfp4.BLOCK], self.alpha,
                           self.input_scale)

    def take(self, index: torch.Tensor):
        """Rows in any order (regrouping of fused checkpoints)."""
        return PackedNVFP4(self.packed[index], self.scales[index], self.alpha[index], self.input_scale)

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        lo = nvfp4.e2m1_to_float(self.packed & 0xF)
        hi = nvfp4.e2m1_to_float(self.packed >> 4)
        w = torch.stack([lo, hi], -1).reshape(self.rows, self.cols)
        sc = self.scales.contiguous().view(torch.float8_e4m3fn).float().repeat_interleave(nvfp4.BLOCK, 1)
        return (w * sc * self.alpha.float()[:, None]).to(dtype)


@dataclass
class PackedFP8(PackedLinear):
    """ModelOpt FP8: e4m3 codes uint8 [out, in] with a per-tensor scale, carried per output row after fusing."""
    codes: torch.Tensor
    alpha: torch.Tensor
    input_scale: float = 0.0
    kind = "fp8"

    @property
    def rows(self):
        return self.codes.shape[0]

    @property
    def cols(self):
        return self.codes.shape[1]

    def take_rows(self, lo, hi):
        return PackedFP8(self.codes[lo:hi], self.alpha[lo:hi], self.input_scale)

    def take_cols(self, lo, hi):
        return PackedFP8(self.codes[:, lo:hi], self.alpha, self.input_scale)

    def take(self, index):
        return PackedFP8(self.codes[index], self.alpha[index], self.input_scale)

    def dequantize(self, dtype=torch.float32):
        return (self.codes.contiguous().view(torch.float8_e4m3fn).float() * self.alpha.float()[:, None]).to(dtype)


class PackedEXL3(PackedLinear):
    """EXL3 trellis tensor (stored [in, out]) behind the [out, in] surface. Cuts fall on the 128-point Hadamard blocks."""
    kind = "exl3"

    def __init__(self, t: Exl3Tensor):
        self.t = t

    @property
    def rows(self):
        return self.t.n

    @property
    def cols(self):
        return self.t.k

    def take_rows(self, lo, hi):
        return PackedEXL3(self.t.slice_cols(lo, hi))

    def take_cols(self, lo, hi):
        return PackedEXL3(self.t.slice_rows(lo, hi))

    def dequantize(self, dtype=torch.float32):
        return self.t.weight(torch.float32).t().contiguous().to(dtype)


class PackedGGUF(PackedLinear):
    """A GGUF tensor in its own block format: `raw` uint8 [out, in / block values * block bytes], every output row a run
    of whole blocks. Row cuts are free; column cuts fall on block boundaries (256 values for the K and IQ types)."""
    kind = "gguf"

    def __init__(self, raw: torch.Tensor, type_id: int, cols: int):
        from .gguf import TYPES
        self.raw, self.type_id, self._cols = raw, int(type_id), int(cols)
        self.bv, self.bb = TYPES[self.type_id][1], TYPES[self.type_id][2]
        assert raw.dim() == 2 and raw.shape[1] == cols // self.bv * self.bb

    @property
    def rows(self):
        return self.raw.shape[0]

    @property
    def cols(self):
        return self._cols

    def take_rows(self, lo, hi):
        return PackedGGUF(self.raw[lo:hi], self.type_id, self._cols)

    def take_cols(self, lo, hi):
        assert lo % self.bv == 0 and hi % self.bv == 0, f"GGUF column cuts fall on {self.bv}-value blocks"
        return PackedGGUF(self.raw[:, lo // self.bv * self.bb:hi // self.bv * self.bb], self.type_id, hi - lo)

    def take(self, index):
        return PackedGGUF(self.raw[index], self.type_id, self._cols)

    def dequantize(self, dtype=torch.float32):
        from .gguf import dequantize
        flat = self.raw.contiguous().numpy().reshape(-1)
        return torch.from_numpy(dequantize(flat, self.type_id)).reshape(self.rows, self._cols).to(dtype)


class PackedStack(PackedLinear):
    """Parts of different storage (for instance an EXL3 q|k|v|z block and the small dense b|a rows of a Gated DeltaNet
    input projection) concatenated along the output rows. The kernels run part by part into column ranges of the
    output; rows are never moved across parts."""
    kind = "stack"

    def __init__(self, parts: Sequence):
        self.parts = [p for p in parts if p.shape[0] > 0]
        assert self.parts and all(p.shape[1] == self.parts[0].shape[1] for p in self.parts)

    @property
    def rows(self):
        return sum(p.shape[0] for p in self.parts)

    @property
    def cols(self):
        return self.parts[0].shape[1]

    def take_rows(self, lo, hi):
        out, o = [], 0
        for p in self.parts:
            n = p.shape[0]
            a, b = max(lo, o), min(hi, o + n)
            if a < b:
                out.append(p[a - o:b - o])
            o += n
        return out[0] if len(out) == 1 else PackedStack(out)

    def take_cols(self, lo, hi):
        return PackedStack([p[:, lo:hi] for p in self.parts])

    def dequantize(self, dtype=torch.float32):
        return torch.cat([p.dequantize(dtype) if isinstance(p, PackedLinear) else p.to(dtype) for p in self.parts], 0)


def is_packed(w) -> bool:
    return isinstance(w, PackedLinear)


def cat_rows(parts: List):
    """Concatenate along the output rows: tensors with tensors, same-kind packed parts by bytes, anything else as a
    `PackedStack`."""
    parts = [p for p in parts if p.shape[0] > 0]
    if all(isinstance(p, torch.Tensor) for p in parts):
        return torch.cat(parts, 0).contiguous()
    flat = []
    for p in parts:
        flat.extend(p.parts if isinstance(p, PackedStack) else [p])
    merged = []
    for p in flat:                                   # neighbours of one kind merge into one part
        q = merged[-1] if merged else None
        if isinstance(p, PackedNVFP4) and isinstance(q, PackedNVFP4):
            merged[-1] = PackedNVFP4(torch.cat([q.packed, p.packed]), torch.cat([q.scales, p.scales]),
                                     torch.cat([q.alpha, p.alpha]), max(q.input_scale, p.input_scale))
        elif isinstance(p, PackedFP8) and isinstance(q, PackedFP8):
            merged[-1] = PackedFP8(torch.cat([q.codes, p.codes]), torch.cat([q.alpha, p.alpha]),
                                   max(q.input_scale, p.input_scale))
        elif isinstance(p, torch.Tensor) and isinstance(q, torch.Tensor):
            merged[-1] = torch.cat([q, p], 0)
        elif isinstance(p, PackedGGUF) and isinstance(q, PackedGGUF) and p.type_id == q.type_id:
            merged[-1] = PackedGGUF(torch.cat([q.raw, p.raw]), p.type_id, p.cols)
        elif isinstance(p, PackedEXL3) and isinstance(q, PackedEXL3) and p.t.bits == q.t.bits and (p.t.suh == q.t.suh).all():
            import numpy as np
            merged[-1] = PackedEXL3(Exl3Tensor(q.t.k, q.t.n + p.t.n, q.t.bits, np.concatenate([q.t.trellis, p.t.trellis], 1),
                                               q.t.suh, np.concatenate([q.t.svh, p.t.svh])))
        else:
            merged.append(p)
    return merged[0] if len(merged) == 1 else PackedStack(merged)


def dense_of(w, dtype=torch.float32) -> torch.Tensor:
    return w.dequantize(dtype) if isinstance(w, PackedLinear) else w.to(dtype)
