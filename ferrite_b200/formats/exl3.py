"""EXL3 (exllamav3) trellis-quantised tensors: format, decoding, reconstruction and the factored linear.

A weight W [k, n] (y = x @ W) is stored in a rotated basis: W = diag(suh) H_k W_hat H_n diag(svh) / 128 with 128-point
Hadamard blocks H. W_hat is cut into 16x16 tiles; a tile is a cyclic bit stream of 256*bits bits in which position t
owns the 16-bit window ending at bit (t+1)*bits; the window value ("state") is decoded by the `mul1` codebook:
x = state * 0x83DCD12D (mod 2^32); s = sum of the 4 bytes of x; value = fp16(1024 + s) * fp16(1/147.7) + fp16(-10.39)
(one fp16 fma). Position t = lane*8 + j sits at row 2*(lane&3) + (j&1) + 8*((j>>1)&1), column (lane>>2) + 8*(j>>2) of
the tile (the fragment order of a 16x8x16 tensor-core tile).

Behavioural reference: `crates/fe-exl3/src/format.rs` (tensor names, `value_row/col`, slicing), `cpu.rs` (`tile_state`,
`decode_mul1`, `fwht128`, `weight_block_f64`, `linear_f64`) and `tp.rs` (column / row slices per rank).
Tensors of a checkpoint: `<base>.trellis` int16 [k/16, n/16, 16*bits], `<base>.suh` f16 [k], `<base>.svh` f16 [n],
optional `<base>.mcg` / `<base>.mul1` marker naming the codebook.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

MUL1 = 0x83DCD12D
HAD_SCALE = 1.0 / np.sqrt(128.0)


def _value_row(lane, j):
    return 2 * (lane & 3) + (j & 1) + 8 * ((j >> 1) & 1)


def _value_col(lane, j):
    return (lane >> 2) + 8 * (j >> 2)


_T = np.arange(256)
_ROW = _value_row(_T // 8, _T % 8)
_COL = _value_col(_T // 8, _T % 8)


def _mul1_table() -> np.ndarray:
    s = np.arange(1021, dtype=np.float32)
    a = (1024 + s).astype(np.float16)
    m = np.array([0x1EEE], np.uint16).view(np.float16)[0]
    c = np.array([0xC931], np.uint16).view(np.float16)[0]
    # one rounding: the fp16 fma is evaluated in float64 and rounded once
    return (a.astype(np.float64) * float(m) + float(c)).astype(np.float16)


MUL1_TABLE = _mul1_table()


@dataclass
class Exl3Tensor:
    k: int
    n: int
    bits: int
    trellis: np.ndarray        # uint16 [k/16, n/16, 16*bits] (big-endian bit order inside the 32-bit words of the stream)
    suh: np.ndarray            # float16 [k]
    svh: np.ndarray            # float16 [n]

    @staticmethod
    def random(k: int, n: int, bits: int, seed: int = 0) -> "Exl3Tensor":
        """Any bit stream is a valid tensor: random bits give random codebook values (synthetic checkpoints)."""
        r = np.random.default_rng(seed)
        tr = r.integers(0, 1 << 16, size=(k // 16, n // 16, 16 * bits), dtype=np.uint16)
        su = np.where(r.random(k) < 0.5, -1.0, 1.0).astype(np.float16)
        sv = (np.where(r.random(n) < 0.5, -1.0, 1.0) * (0.02 * (0.5 + r.random(n)))).astype(np.float16)
        return Exl3Tensor(k, n, bits, tr, su, sv)

    # ---- decoding ------------------------------------------------------------------------------------
    def states(self) -> np.ndarray:
        """16-bit trellis state of every position: uint32 [k/16, n/16, 256]."""
        kt, nt, _ = self.trellis.shape
        bits = self.bits
        # the stream as 32-bit words, most significant bit first: word w = (u16[2w] | u16[2w+1] << 16) per exllamav3's
        # int16 storage of little-endian uint32 words
        u16 = self.trellis.astype(np.uint32)
        words = u16[..., 0::2] | (u16[..., 1::2] << 16)                 # [kt, nt, 8*bits]
        bitsarr = ((words[..., :, None] >> (31 - np.arange(32))) & 1).reshape(kt, nt, -1).astype(np.uint32)
        length = 256 * bits
        start = ((_T + 1) * bits + length - 16) % length                 # [256]
        idx = (start[:, None] + np.arange(16)[None, :]) % length         # [256, 16]
        win = bitsarr[..., idx]                                          # [kt, nt, 256, 16]
        return (win << (15 - np.arange(16, dtype=np.uint32))).sum(-1).astype(np.uint32)

    def w_hat(self) -> np.ndarray:
        """Rotated-basis weights as float16 [k, n]."""
        st = self.states().astype(np.uint64)
        x = (st * MUL1) & 0xFFFFFFFF
        s = (x & 0xFF) + ((x >> 8) & 0xFF) + ((x >> 16) & 0xFF) + (x >> 24)
        vals = MUL1_TABLE[s.astype(np.int64)]                            # [kt, nt, 256]
        kt, nt = vals.shape[:2]
        tiles = np.empty((kt, nt, 16, 16), np.float16)
        tiles[:, :, _ROW, _COL] = vals
        return tiles.transpose(0, 2, 1, 3).reshape(self.k, self.n)

    def weight(self, dtype=torch.float32) -> torch.Tensor:
        """Original-basis W [k, n] (y = x @ W)."""
        w = torch.from_numpy(self.w_hat().astype(np.float32)).double()
        w = fwht128(w.view(self.k, self.n // 128, 128)).view(self.k, self.n)                 # over n
        w = fwht128(w.t().contiguous().view(self.n, self.k // 128, 128)).view(self.n, self.k).t()   # over k
        su = torch.from_numpy(self.suh.astype(np.float32)).double() * (HAD_SCALE * HAD_SCALE)
        sv = torch.from_numpy(self.svh.astype(np.float32)).double()
        return (w * su[:, None] * sv[None, :]).to(dtype)

    def linear(self, x: torch.Tensor) -> torch.Tensor:
        """y = x @ W through the factored form H(H(x * suh) @ W_hat) * svh / 128 (float64)."""
        xh = x.double() * torch.from_numpy(self.suh.astype(np.float32)).double()
        xh = fwht128(xh.view(x.shape[0], self.k // 128, 128)).view(x.shape[0], self.k)
        z = xh @ torch.from_numpy(self.w_hat().astype(np.float32)).double()
        z = fwht128(z.view(x.shape[0], self.n // 128, 128)).view(x.shape[0], self.n)
        return z * torch.from_numpy(self.svh.astype(np.float32)).double() / 128.0

    # ---- tensor-parallel slices (reference `slice_cols` / `slice_rows`, `crates/fe-exl3/src/tp.rs`) ----------
    def slice_cols(self, n0: int, n1: int) -> "Exl3Tensor":
        assert n0 % 128 == 0 and n1 % 128 == 0
        return Exl3Tensor(self.k, n1 - n0, self.bits, self.trellis[:, n0 // 16:n1 // 16].copy(), self.suh, self.svh[n0:n1])

    def slice_rows(self, k0: int, k1: int) -> "Exl3Tensor":
        assert k0 % 128 == 0 and k1 % 128 == 0
        return Exl3Tensor(k1 - k0, self.n, self.bits, self.trellis[k0 // 16:k1 // 16].copy(), self.suh[k0:k1], self.svh)


def fwht128(v: torch.Tensor) -> torch.Tensor:
    """Unnormalised Sylvester-ordered Walsh-Hadamard transform over the last dimension (128)."""
    shape = v.shape
    v = v.reshape(-1, 128)
    h = 1
    while h < 128:
        v = v.view(-1, 128 // (2 * h), 2, h)
        a, b = v[:, :, 0], v[:, :, 1]
        v = torch.stack([a + b, a - b], 2).reshape(-1, 128)
        h *= 2
    return v.view(shape)


def load_tensor(st, base: str) -> Exl3Tensor:
    """Read `<base>.{trellis,suh,svh}` from a `SafeTensors` folder."""
    tr = st.get(base + ".trellis")
    trn = tr.view(torch.int16).numpy().view(np.uint16) if tr.dtype != torch.uint16 else tr.numpy()
    kt, nt, w = trn.shape
    bits = w // 16
    suh = st.get(base + ".suh").view(torch.float16).numpy()
    svh = st.get(base + ".svh").view(torch.float16).numpy()
    return Exl3Tensor(kt * 16, nt * 16, bits, trn, suh, svh)
