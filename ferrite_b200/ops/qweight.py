"""Quantised weight holder the linear ops accept in place of a bf16 matrix.

A `QWeight` carries the packed low-bit form the small-row kernels stream (NVFP4 GEMV) and, until the block-scaled
tensor-core GEMM takes the many-row path, the same weights dequantised to bf16 for prompt-sized launches. Both
paths therefore multiply by identical effective weights. The reference routes rows the same way: low-bit GEMV for
decode rows, a second copy of the weights for prompt rows (`Linear::forward`, `crates/fe-model/src/model.rs:275-346`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..formats import nvfp4


@dataclass
class QWeight:
    kind: str                      # "nvfp4"
    rows: int
    cols: int
    packed: torch.Tensor           # uint8 [rows, cols/2]
    gemv_scales: torch.Tensor      # uint8 tiled for the GEMV
    global_scale: float
    dense: Optional[torch.Tensor]  # dequantised copy (activation dtype) for the many-row path
    mma_scales: Optional[torch.Tensor] = None

    @property
    def shape(self):
        return (self.rows, self.cols)

    def __getitem__(self, idx):
        raise TypeError("slice a QWeight before quantising it")


def quantize_weight(w: torch.Tensor, kind: str = "nvfp4", keep_dense: bool = True, dense_dtype=None,
                    mma: bool = True) -> QWeight:
    assert kind == "nvfp4"
    rows, cols = w.shape
    # quantise in row slabs to bound the fp32 temporaries
    slab = max(1, (64 << 20) // max(1, cols))
    amax = float(w.abs().max())
    gs = amax / (6.0 * 448.0) if amax > 0 else 1.0
    packed, scales, dense = [], [], []
    for r0 in range(0, rows, slab):
        q = nvfp4.quantize(w[r0:r0 + slab], global_scale=gs)
        packed.append(q.packed)
        scales.append(q.scales)
        if keep_dense:
            dense.append(q.dequantize(dense_dtype or w.dtype))
    sc = torch.cat(scales, 0)
    return QWeight(kind, rows, cols, torch.cat(packed, 0).contiguous(), nvfp4.tile_scales_gemv(sc), gs,
                   torch.cat(dense, 0).contiguous() if keep_dense else None,
                   nvfp4.tile_scales_mma(sc).contiguous() if mma and cols % 64 == 0 else None)
