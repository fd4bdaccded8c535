"""NVFP4 (ModelOpt): e2m1 values in blocks of 16 with an e4m3 scale per block and an fp32 scale per tensor.

    w ~= e2m1(code) * e4m3(block_scale) * global_scale

Host-side codecs, packing and the scale tilings the kernels read. Counterpart of the reference's
`crates/fe-fp4/src/format.rs` (`quant_fp4_row`, `tile_scales`, `ref_gemm`) and checkpoint reader `st.rs`.
Packing follows ModelOpt: two codes per byte, element 2i in the low nibble.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
BLOCK = 16
GEMV_SPAN = 1024          # weights a warp covers per load in the NVFP4 GEMV (32 lanes x 32 codes)
GEMV_GROUP = 4            # spans whose scales one lane reads with a single 8-byte load


def _e2m1_codes(x: torch.Tensor) -> torch.Tensor:
    """Round |x| (already divided by its scale) to the nearest e2m1 magnitude, ties to even code; returns 4-bit codes."""
    vals = E2M1_VALUES.to(x.device)
    mag = x.abs().clamp(max=6.0)
    # midpoints between representable magnitudes; ties go to the even mantissa (codes 0,2,4,6 at .25,.75? no:
    # follow round-to-nearest-even on the e2m1 grid)
    mids = (vals[1:] + vals[:-1]) / 2
    idx = torch.bucketize(mag, mids, right=False)          # mag == mid -> lower index
    tie = torch.zeros_like(idx, dtype=torch.bool)
    for i in range(7):
        tie |= (mag == mids[i]) & (idx == i)
    # at a tie pick the code with even mantissa bit (even index)
    idx = torch.where(tie & (idx % 2 == 1), idx + 1, idx)
    sign = (x < 0) | ((x == 0) & (torch.signbit(x)))
    return (idx | (sign.to(idx.dtype) << 3)).to(torch.uint8)


def e2m1_to_float(codes: torch.Tensor) -> torch.Tensor:
    vals = E2M1_VALUES.to(codes.device)
    mag = vals[(codes & 7).long()]
    return torch.where((codes & 8) != 0, -mag, mag)


@dataclass
class NVFP4Tensor:
    """A quantised [rows, cols] matrix. `packed` uint8 [rows, cols/2]; `scales` float8_e4m3fn [rows, cols/16];
    `global_scale` python float. `gemv_scales` / `mma_scales` are kernel-side tilings of `scales`."""

    packed: torch.Tensor
    scales: torch.Tensor
    global_scale: float
    rows: int
    cols: int
    gemv_scales: Optional[torch.Tensor] = None
    mma_scales: Optional[torch.Tensor] = None

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        lo = e2m1_to_float(self.packed & 0xF)
        hi = e2m1_to_float(self.packed >> 4)
        w = torch.stack([lo, hi], -1).reshape(self.rows, self.cols)
        s = self.scales.float().repeat_interleave(BLOCK, 1)
        return (w * s * self.global_scale).to(dtype)

    def to(self, device) -> "NVFP4Tensor":
        mv = lambda t: None if t is None else t.to(device)
        return NVFP4Tensor(self.packed.to(device), self.scales.to(device), self.global_scale, self.rows, self.cols,
                           mv(self.gemv_scales), mv(self.mma_scales))

    @property
    def nbytes(self) -> int:
        return self.packed.numel() + self.scales.numel()


def quantize(w: torch.Tensor, global_scale: Optional[float] = None) -> NVFP4Tensor:
    """Quantise a [rows, cols] matrix (cols a multiple of 16). global_scale defaults to amax / (6 * 448)."""
    rows, cols = w.shape
    assert cols % BLOCK == 0
    wf = w.float()
    if global_scale is None:
        amax = float(wf.abs().max())
        global_scale = amax / (6.0 * 448.0) if amax > 0 else 1.0
    blk = wf.view(rows, cols // BLOCK, BLOCK)
    bmax = blk.abs().amax(-1)
    sc = (bmax / (6.0 * global_scale)).clamp(max=448.0).to(torch.float8_e4m3fn)
    scf = sc.float()
    denom = torch.where(scf > 0, scf * global_scale, torch.ones_like(scf))
    codes = _e2m1_codes(blk / denom[..., None]).view(rows, cols)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    return NVFP4Tensor(packed, sc.contiguous(), float(global_scale), rows, cols)


def tile_scales_gemv(scales: torch.Tensor) -> torch.Tensor:
    """Re-tile block scales for the GEMV: per row, groups of GEMV_GROUP spans of 1024 weights; inside a group the
    order is [lane 32][span 4][2 blocks], so one lane fetches the 8 scale bytes of its 4 x 32 codes with one load.
    Output uint8 [rows, ceil(cols/4096) * 256] (padding scales are 0)."""
    rows, nblk = scales.shape
    per_span = GEMV_SPAN // BLOCK                     # 64 blocks
    grp = per_span * GEMV_GROUP                        # 256 blocks
    ngrp = (nblk + grp - 1) // grp
    raw = scales.view(torch.uint8)
    pad = torch.zeros(rows, ngrp * grp, dtype=torch.uint8, device=scales.device)
    pad[:, :nblk] = raw
    t = pad.view(rows, ngrp, GEMV_GROUP, 32, 2)        # [row][group][span][lane][blk]
    return t.permute(0, 1, 3, 2, 4).contiguous().view(rows, ngrp * grp)


def tile_scales_mma(scales: torch.Tensor) -> torch.Tensor:
    """Scale-factor layout of the block-scaled tensor-core GEMM: tiles of 128 rows x 4 k-blocks stored as
    [rows/128][kblocks/4][32][4][4] bytes (row r of a tile at [r % 32][r / 32], then the 4 k-blocks), the
    arrangement `tcgen05.cp` copies into TMEM 32 lanes x 16 bytes at a time. Rows and k-blocks are zero-padded."""
    rows, nblk = scales.shape
    rt, kt = (rows + 127) // 128, (nblk + 3) // 4
    pad = torch.zeros(rt * 128, kt * 4, dtype=torch.uint8, device=scales.device)
    pad[:rows, :nblk] = scales.view(torch.uint8)
    t = pad.view(rt, 4, 32, kt, 4)                     # [rt][r/32][r%32][kt][kb]
    return t.permute(0, 3, 2, 1, 4).contiguous().view(rt, kt, 512)


def prepare(w: torch.Tensor, device=None, mma: bool = False) -> NVFP4Tensor:
    q = quantize(w)
    q.gemv_scales = tile_scales_gemv(q.scales)
    if mma:
        q.mma_scales = tile_scales_mma(q.scales)
    return q.to(device) if device is not None else q


def ref_linear(x: torch.Tensor, q: NVFP4Tensor) -> torch.Tensor:
    """fp32 reference: x [M, K] times dequantised weights [N, K]^T."""
    return x.float() @ q.dequantize(torch.float32).t()
