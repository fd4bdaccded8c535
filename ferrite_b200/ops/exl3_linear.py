"""EXL3 linear on the GPU: y = H(H(x * suh) @ W_hat) * svh / 128 with the trellis tiles decoded on the fly for decode
rows and, for prompt-sized steps, W_hat decoded into a scratch shared by all linears and multiplied on the tensor-core
GEMM. The trellis stays packed from load to kernel: no dense copy of a weight outlives the step that needed it.
Counterpart of the reference's `Linear::forward` (`crates/fe-exl3/src/linear.rs:274-301`: `rotate_input` +
`gemv_rotated`) and of its load-time `reconstruct_bf16` (`kernels/k-exl3/src/recon.rs`), which here runs per use."""
from __future__ import annotations

import numpy as np
import torch

from ..formats.exl3 import Exl3Tensor

HAD = 1.0 / np.sqrt(128.0)
GEMV_ROWS = 8             # rows one trellis GEMV launch takes


class Exl3Linear:
    def __init__(self, t: Exl3Tensor, device):
        self.k, self.n, self.bits = t.k, t.n, t.bits
        self.trellis = torch.from_numpy(t.trellis.view(np.int16).copy()).to(device)      # [k/16, n/16, 16*bits] 16-bit words
        self.suh = torch.from_numpy(t.suh.copy()).to(device)
        self.svh = torch.from_numpy(t.svh.copy()).to(device)

    def nbytes(self) -> int:
        return self.trellis.numel() * 2 + (self.k + self.n) * 2

    def forward(self, ops, x: torch.Tensor, res=None, gemv_max_rows: int = 32) -> torch.Tensor:
        M = x.shape[0]
        C = ops.C
        y = torch.empty(M, self.n, dtype=torch.bfloat16, device=x.device)
        if M <= gemv_max_rows:
            xh = torch.empty(M, self.k, dtype=torch.float32, device=x.device)
            C.exl3_had(xh, x.contiguous(), self.suh, None, None, HAD)
            z = torch.empty(M, self.n, dtype=torch.float32, device=x.device)
            for r0 in range(0, M, GEMV_ROWS):
                C.exl3_gemv(z[r0:r0 + GEMV_ROWS], xh[r0:r0 + GEMV_ROWS], self.trellis, self.bits)
            C.exl3_had(y, z, None, self.svh, res, HAD)
            ops.launches += 2 + (M + GEMV_ROWS - 1) // GEMV_ROWS
            return y
        xh = torch.empty(M, self.k, dtype=torch.bfloat16, device=x.device)
        C.exl3_had(xh, x.contiguous(), self.suh, None, None, HAD)
        w_hat_t = ops.scratch("exl3_w_hat", self.n * self.k).view(self.n, self.k)
        C.exl3_decode(w_hat_t, self.trellis, self.bits)
        z = ops.linear(xh, w_hat_t)
        C.exl3_had(y, z, None, self.svh, res, HAD)
        ops.launches += 3
        return y
