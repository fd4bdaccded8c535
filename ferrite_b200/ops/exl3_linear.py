"""EXL3 linear on the GPU: y = H(H(x * suh) @ W_hat) * svh / 128 with the trellis tiles decoded on the fly for decode
rows and through a cached bf16 copy of W_hat on the tensor-core GEMM for prompt rows. Counterpart of the reference's
`Linear::forward` (`crates/fe-exl3/src/linear.rs:274-301`: `rotate_input` + `gemv_rotated`)."""
from __future__ import annotations

import numpy as np
import torch

from ..formats.exl3 import Exl3Tensor

HAD = 1.0 / np.sqrt(128.0)


class Exl3Linear:
    def __init__(self, t: Exl3Tensor, ops, keep_prompt_copy: bool = True):
        self.k, self.n, self.bits = t.k, t.n, t.bits
        self.ops, self.C, dev = ops, ops.C, ops.device
        self.trellis = torch.from_numpy(t.trellis.view(np.int16).copy()).to(dev)      # [k/16, n/16, 16*bits] 16-bit words
        self.suh = torch.from_numpy(t.suh.copy()).to(dev)
        self.svh = torch.from_numpy(t.svh.copy()).to(dev)
        self.w_hat_t = None
        if keep_prompt_copy:
            self.w_hat_t = torch.empty(self.n, self.k, dtype=torch.bfloat16, device=dev)
            self.C.exl3_decode(self.w_hat_t, self.trellis, self.bits)
            ops.launches += 1

    def forward(self, x: torch.Tensor, res=None) -> torch.Tensor:
        M = x.shape[0]
        ops = self.ops
        y = torch.empty(M, self.n, dtype=torch.bfloat16, device=x.device)
        if M <= 8 or self.w_hat_t is None:
            xh = torch.empty(M, self.k, dtype=torch.float32, device=x.device)
            self.C.exl3_had(xh, x.contiguous(), self.suh, None, None, HAD)
            z = torch.empty(M, self.n, dtype=torch.float32, device=x.device)
            for r0 in range(0, M, 8):
                self.C.exl3_gemv(z[r0:r0 + 8], xh[r0:r0 + 8], self.trellis, self.bits)
            self.C.exl3_had(y, z, None, self.svh, res, HAD)
            ops.launches += 2 + (M + 7) // 8
            return y
        xh = torch.empty(M, self.k, dtype=torch.bfloat16, device=x.device)
        self.C.exl3_had(xh, x.contiguous(), self.suh, None, None, HAD)
        z = ops.linear(xh, self.w_hat_t)
        self.C.exl3_had(y, z, None, self.svh, res, HAD)
        ops.launches += 2
        return y
