"""Quantised weight holder the linear ops accept in place of a bf16 matrix.

A `QWeight` carries the packed low-bit form the small-row kernels stream (NVFP4 GEMV) and, until the block-scaled
tensor-core GEMM takes the many-row path, the same weights dequantised to bf16 for prompt-sized launches. Both
paths therefore multiply by identical effective weights. The reference routes rows the same way: low-bit GEMV for
decode rows, a second copy of the weights for prompt rows (`Linear::forward`, `crates/fe-model/src/model.rs:275-346`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ..formats import nvfp4


@dataclass
class QWeight:
    kind: str                      # "nvfp4" | "fp8b" (e4m3, 128 x 128 blocks)
    rows: int
    cols: int
    packed: torch.Tensor           # uint8 [rows, cols/2]
    gemv_scales: torch.Tensor      # uint8 tiled for the GEMV
    global_scale: float
    dense: Optional[torch.Tensor]  # dequantised copy (activation dtype) for the many-row path
    mma_scales: Optional[torch.Tensor] = None
    fp8_codes: Optional[torch.Tensor] = None     # "fp8b": uint8 [rows, ceil(cols/128)*128]; "fp8": uint8 [rows, cols]
    fp8_scales: Optional[torch.Tensor] = None    # "fp8b": fp32 [ceil(rows/128), ceil(cols/128)]; "fp8": fp32 [rows]
    row_alpha: Optional[torch.Tensor] = None     # "nvfp4": fp32 [rows] tensor scale per output row (fused checkpoint parts
                                                 # bring their own `weight_scale_2`); global_scale is 1 when set
    pair: bool = False                           # rows are gate | up halves consumed with the SwiGLU epilogue
    # the NVFP4 weight the step multiplies next (set by the engine, in execution order, the last one pointing at the
    # first): the few-row tensor-core kernel asks L2 for its head while it drains
    next: Optional["QWeight"] = field(default=None, repr=False, compare=False)

    @property
    def shape(self):
        return (self.rows, self.cols)

    def __getitem__(self, idx):
        raise TypeError("slice a QWeight before quantising it")


def quantize_weight(w: torch.Tensor, kind: str = "nvfp4", keep_dense: bool = True, dense_dtype=None,
                    mma: bool = True) -> QWeight:
    rows, cols = w.shape
    if kind == "fp8b":
        # e4m3 codes with one scale per 128 x 128 block (the form block-scaled FP8 checkpoints ship); the dense copy
        # holds the dequantised values for few-row steps and for the oracle
        nb, kb = (rows + 127) // 128, (cols + 127) // 128
        wf = torch.zeros(nb * 128, kb * 128, dtype=torch.float32, device=w.device)
        wf[:rows, :cols] = w.float()
        blocks = wf.view(nb, 128, kb, 128)
        sc = (blocks.abs().amax((1, 3)) / 448.0).clamp_min(1e-12)
        codes = (blocks / sc[:, None, :, None]).to(torch.float8_e4m3fn)
        dense = None
        if keep_dense:
            dense = (codes.float() * sc[:, None, :, None]).view(nb * 128, kb * 128)[:rows, :cols].to(dense_dtype or w.dtype).contiguous()
        codes = codes.view(torch.uint8).view(nb * 128, kb * 128)[:rows].contiguous()
        empty = torch.empty(0, dtype=torch.uint8, device=w.device)
        return QWeight(kind, rows, cols, empty, empty, 1.0, dense, None, codes, sc.contiguous())
    assert kind == "nvfp4"
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


@dataclass
class ExpertsFP4:
    """Stacked expert matrices [experts, rows, cols] in NVFP4: `packed` uint8 [E, rows, cols/2] (low nibble = even
    element), `scales` uint8 [E, rows, cols/16] holding e4m3 bits, one `global_scale` for the whole stack. Decode rows
    stream this form (`csrc/moe_fp4.cu`); prompt-sized steps dequantise it into a bf16 scratch for the grouped GEMM."""
    packed: torch.Tensor
    scales: torch.Tensor
    global_scale: float

    @property
    def shape(self):
        e, r, kb = self.packed.shape
        return (e, r, kb * 2)

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        e, r, k = self.shape
        lo = nvfp4.e2m1_to_float(self.packed & 0xF)
        hi = nvfp4.e2m1_to_float(self.packed >> 4)
        w = torch.stack([lo, hi], -1).reshape(e, r, k)
        sc = self.scales.view(torch.float8_e4m3fn).float().repeat_interleave(nvfp4.BLOCK, 2)
        return (w * sc * self.global_scale).to(dtype)


def quantize_experts(w: torch.Tensor) -> ExpertsFP4:
    """[experts, rows, cols] -> NVFP4 with one tensor scale shared by all experts (expert by expert, to bound the
    fp32 temporaries)."""
    e, r, k = w.shape
    amax = float(w.abs().max())
    gs = amax / (6.0 * 448.0) if amax > 0 else 1.0
    packed = torch.empty(e, r, k // 2, dtype=torch.uint8, device=w.device)
    scales = torch.empty(e, r, k // nvfp4.BLOCK, dtype=torch.uint8, device=w.device)
    for i in range(e):
        q = nvfp4.quantize(w[i], global_scale=gs)
        packed[i] = q.packed
        scales[i] = q.scales.view(torch.uint8)
    return ExpertsFP4(packed, scales, gs)


class Exl3Weight:
    """An EXL3 linear ready for the kernels (`ops/exl3_linear.py`), behind the [out, in] weight surface."""
    kind = "exl3"

    def __init__(self, lin, rows: int, cols: int, host=None):
        self.lin, self.rows, self.cols = lin, rows, cols
        self.host = host                  # the checkpoint tensor (`formats.exl3.Exl3Tensor`), for the oracle

    @property
    def shape(self):
        return (self.rows, self.cols)

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        return self.host.weight(torch.float32).t().contiguous().to(dtype)


class GgufWeight:
    """A GGUF tensor on the device in its checkpoint block format (`formats.packed.PackedGGUF`): decode rows run the
    dequantising GEMV on these blocks, prompt-sized steps dequantise into a scratch for the tensor-core GEMM."""
    kind = "gguf"

    def __init__(self, raw: torch.Tensor, type_id: int, rows: int, cols: int, host=None):
        self.raw, self.type_id, self.rows, self.cols, self.host = raw, type_id, rows, cols, host

    @property
    def shape(self):
        return (self.rows, self.cols)

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        return self.host.dequantize(dtype)


class StackWeight:
    """Weights of different storage sharing one input, concatenated along the output rows (`formats.packed.PackedStack`
    after conversion): the linear runs part by part into column ranges of one output."""
    kind = "stack"

    def __init__(self, parts):
        self.parts = list(parts)
        self.rows = sum(p.shape[0] for p in self.parts)
        self.cols = self.parts[0].shape[1]

    @property
    def shape(self):
        return (self.rows, self.cols)

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        return torch.cat([(p.to(dtype) if isinstance(p, torch.Tensor) else
                           p.dequantize(dtype) if hasattr(p, "dequantize") else p.dense.to(dtype)).cpu() for p in self.parts], 0)


def from_packed(p, device, dtype, on_gpu: bool, keep_dense: bool = True):
    """A checkpoint's packed linear (`formats/packed.py`) as the object the linear ops accept. On the CPU (fp32 oracle)
    that is the dequantised matrix; on the GPU the codes and scales go to the device in the kernels' layouts:
    NVFP4 -> `QWeight` (GEMV tiling + tensor-core tiling of the block scales, per-row tensor scales when fused parts
    differ), FP8 -> `QWeight` kind "fp8" (codes + per-row scales for the e4m3 GEMM), EXL3 -> `Exl3Weight`."""
    from ..formats.packed import PackedEXL3, PackedFP8, PackedGGUF, PackedNVFP4, PackedStack
    if isinstance(p, torch.Tensor):
        return p.to(device, dtype)
    if not on_gpu:
        return p.dequantize(torch.float32).to(device, dtype)
    if isinstance(p, PackedNVFP4):
        rows, cols = p.shape
        sc = p.scales.contiguous()
        alpha = p.alpha.float()
        uniform = bool((alpha == alpha[0]).all())
        dense = p.dequantize(torch.float32).to(device, dtype) if keep_dense else None
        return QWeight("nvfp4", rows, cols, p.packed.contiguous().to(device), nvfp4.tile_scales_gemv(sc).to(device),
                       float(alpha[0]) if uniform else 1.0, dense,
                       nvfp4.tile_scales_mma(sc).contiguous().to(device) if cols % 64 == 0 else None,
                       row_alpha=None if uniform else alpha.contiguous().to(device))
    if isinstance(p, PackedFP8):
        rows, cols = p.shape
        dense = p.dequantize(torch.float32).to(device, dtype)
        empty = torch.empty(0, dtype=torch.uint8, device=device)
        return QWeight("fp8", rows, cols, empty, empty, 1.0, dense, None, p.codes.contiguous().to(device),
                       p.alpha.float().contiguous().to(device))
    if isinstance(p, PackedEXL3):
        from .exl3_linear import Exl3Linear
        return Exl3Weight(Exl3Linear(p.t, device), p.shape[0], p.shape[1], host=p.t)
    if isinstance(p, PackedGGUF):
        return GgufWeight(p.raw.contiguous().view(-1).to(device), p.type_id, p.shape[0], p.shape[1], host=p)
    if isinstance(p, PackedStack):
        return StackWeight([from_packed(q, device, dtype, on_gpu, keep_dense) for q in p.parts])
    raise TypeError(type(p).__name__)
