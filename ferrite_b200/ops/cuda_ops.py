"""Device ops backed by the hand-written sm_100a kernels in `csrc/` (loaded from `ferrite_b200/_C.so`).

Same signatures as `torch_ops.TorchOps`. Row counts pick the kernel: up to `GEMV_MAX_ROWS` rows stream the
weights through the SIMT GEMV (fused norm / SwiGLU / residual), more rows go to the tcgen05 GEMM (swapped
orientation with split-K up to 64 rows, normal orientation beyond). There is no PyTorch fallback here: a
missing extension raises.
"""
from __future__ import annotations

import math
from typing import Optional

import os

import torch

from .._ext import load
from .extras import CudaExtras
from .qweight import Exl3Weight, ExpertsFP4, GgufWeight, QWeight, StackWeight

GEMV_MAX_ROWS = 8
MOE_PAIR_ROWS = 64     # up to this many rows (the largest graph-captured step) the experts run as per-pair GEMVs,
                       # beyond as grouped GEMMs, which read the per-expert row counts on the host


class CudaOps(CudaExtras):
    name = "cuda"

    def __init__(self, device, dtype=torch.bfloat16):
        self.C = load()
        self.device = torch.device(device)
        self.dtype = dtype
        assert dtype == torch.bfloat16, "the sm_100a kernels take bf16 activations"
        cap = torch.cuda.get_device_capability(self.device)
        if cap != (10, 0) and not os.environ.get("FB_SKIP_ARCH_CHECK"):
            # the extension holds sm_100a code only: on any other GPU every launch would fail with "no kernel image"
            raise RuntimeError(f"{torch.cuda.get_device_name(self.device)} has compute capability {cap[0]}.{cap[1]}; "
                               "the kernels of this build are sm_100a (B200, 10.0) only")
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.status_word = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._ws: Optional[torch.Tensor] = None
        self._counters = torch.zeros(16384, dtype=torch.int32, device=self.device)
        self.empty = torch.empty            # every output buffer of the ops comes from here (see enable_canaries)
        self._guarded = []
        self._dl_sync = torch.zeros(2, dtype=torch.int32, device=self.device)      # grid-barrier words of the persistent layer kernel
        self._dl_empty = self.empty(0, dtype=self.dtype, device=self.device)
        self.decode_layers_max = int(self.C.decode_layers_max())
        self.C.decode_layers_prepare()      # attributes + residency check now, not inside a graph capture
        self.force_gemv_chunks = False      # debug: run any row count through 8-row GEMV passes
        self.launches = 0                   # kernels launched (or recorded into a graph) through this object
        self.moe_pair_rows = MOE_PAIR_ROWS
        self.mma_gemv_rows = (2, 32)        # row counts routed to the mma.sync weight-streaming kernel
        self.attn_mma = os.environ.get("FB_ATTN_MMA", "1") != "0"   # decode attention on mma.sync (0: SIMT kernel)
        self.attn_tc = os.environ.get("FB_ATTN_TC", "1") != "0"     # prompt attention on tcgen05 (0: mma.sync kernel)
        self._gdn_scratch = None
        self._tree_scratch = None
        self._expert_scratch = {}
        self._kv_scratch = None
        self.fp4_act = False                # NVFP4 weights: quantise activations too and use the tcgen05 GEMM
        self.fp4_prompt = False             # ... for prompt-sized steps too (one NVFP4 rendering per activation row)
        self.fp4_terms = 3                  # few-row NVFP4 steps: NVFP4 renderings per activation row (0 = older fused kernel,
                                            # -1 = the SIMT GEMV with 16-bit activations)
        self.fp4_tc_ctas = int(os.environ.get("FB_FP4_CTAS", "2"))             # ... and CTAs per SM of that kernel
        # prompt-sized FFN blocks: the gate|up GEMM's epilogue re-quantises the SwiGLU output for the down projection;
        # static global scale of that activation (block maxima of 6e-3 .. 168 land on normal e4m3 scales)
        self.fp4_fuse_requant = os.environ.get("FB_FP4_FUSE_REQUANT", "1") != "0"
        self.fp4_act_gscale = 1.0 / 16.0
        self.fp4_prefetch_mb = int(os.environ.get("FB_FP4_PREFETCH_MB", "48"))  # ... and how much of the next weight
                                                                                # (`QWeight.next`) it asks L2 for as it drains
        self._sf_pool = {}
        self._scratch = {}

    # ---- workspace ---------------------------------------------------------------------------------
    def _workspace(self, nbytes: int) -> torch.Tensor:
        if self._ws is None or self._ws.numel() * 4 < nbytes:
            self._ws = self.empty(max(nbytes // 4, 16 << 20), dtype=torch.float32, device=self.device)   # 64 MB up front: graphs keep the pointer
        return self._ws

    # ---- debug: canary-padded output buffers --------------------------------------------------------------
    CANARY_BYTES, CANARY_BYTE = 256, 0xA5

    def enable_canaries(self, on: bool = True) -> None:
        """Debug aid (reference: canary-padded allocations, `crates/fe-cuda/src/lib.rs:299-343`): every output buffer the
        ops allocate gets 256 guard bytes in front and behind, filled with a pattern; `check_canaries()` verifies them, so
        a kernel that writes just past (or before) its output is caught at the step that did it. Eager steps only (the
        guard zones of a captured graph are checked after replays as long as canaries stay enabled)."""
        self.empty = self._empty_guarded if on else torch.empty
        if not on:
            self._guarded = []

    def _empty_guarded(self, *shape, dtype=None, device=None, **kw):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
            shape = tuple(shape[0])
        dtype = dtype or torch.float32
        item = torch.empty(0, dtype=dtype).element_size()
        nbytes = item
        for d in shape:
            nbytes *= int(d)
        body = (nbytes + 255) // 256 * 256
        g = self.CANARY_BYTES
        raw = torch.full((g + body + g,), self.CANARY_BYTE, dtype=torch.uint8, device=device or self.device)
        self._guarded.append((raw, nbytes, tuple(int(d) for d in shape), dtype))
        return raw[g:g + nbytes].view(dtype).view(*shape) if nbytes else torch.empty(*shape, dtype=dtype, device=device or self.device)

    def check_canaries(self) -> int:
        """Raises if any guard byte of a buffer handed out since the last check changed; returns how many were checked."""
        g, n = self.CANARY_BYTES, len(self._guarded)
        for raw, nbytes, shape, dtype in self._guarded:
            front = raw[:g]
            back = raw[g + nbytes:]                      # the round-up slack behind the data is guard too
            if not (bool((front == self.CANARY_BYTE).all()) and bool((back == self.CANARY_BYTE).all())):
                where = "before" if not bool((front == self.CANARY_BYTE).all()) else "behind"
                self._guarded = []
                raise RuntimeError(f"canary: a kernel wrote {where} its output buffer {shape} {dtype}")
        self._guarded = []
        return n

    def status(self) -> int:
        return int(self.status_word.item())

    def scratch(self, name: str, numel: int, dtype=torch.bfloat16) -> torch.Tensor:
        """A named device buffer that only grows (its pointer is stable across the steps of a CUDA graph as long as no
        later call asks for more; callers size it by the largest use up front)."""
        buf = self._scratch.get(name)
        if buf is None or buf.numel() < numel or buf.dtype != dtype:
            buf = self.empty(numel, dtype=dtype, device=self.device)
            self._scratch[name] = buf
        return buf[:numel]

    # ---- rows ------------------------------------------------------------------------------------
    def embed(self, table, ids):
        out = self.empty(ids.numel(), table.shape[1], dtype=self.dtype, device=self.device)
        self.launches += 1
        self.C.embed(out, table, ids)
        return out

    def rmsnorm(self, x, w, eps, centred=True, res=None, out=None):
        out = torch.empty_like(x) if out is None else out
        if res is not None:
            xo = torch.empty_like(x)
            self.launches += 1
            self.C.rmsnorm(out, x, w, eps, centred, res, xo)
            return out, xo
        self.launches += 1
        self.C.rmsnorm(out, x, w, eps, centred, None, None)
        return out, x

    def _split_k(self, M, N, K):
        # work items = weight tiles x k splits, spread persistently over the SMs: aim at >= 4 items per SM so the
        # last wave is nearly full, but keep at least 8 k blocks (512 k) per item
        tiles = (N + 127) // 128
        kblocks = (K + 63) // 64
        want = (self.sm_count + tiles - 1) // tiles
        s = max(1, min(kblocks // 4, want))
        return s

    def linear(self, x, w, norm_w=None, eps=1e-6, res=None, swiglu=False, out_f32=False, out=None):
        if isinstance(w, (Exl3Weight, StackWeight, GgufWeight)):
            # EXL3 / GGUF blocks (and stacks of differently stored parts): the norm runs once, each part fills its column
            # range, the SwiGLU / residual run on the joined output. The trellis kernels rotate their own input.
            if norm_w is not None:
                x, _ = self.rmsnorm(x, norm_w, eps, True)
            if isinstance(w, Exl3Weight):
                y = w.lin.forward(self, x, None if swiglu else res)
            elif isinstance(w, GgufWeight):
                if x.shape[0] <= GEMV_MAX_ROWS and w.cols * 4 * 8 <= 200 * 1024:
                    y = self.gguf_gemv(x, w.raw, w.type_id, w.rows, None if swiglu else res)
                else:
                    dense = self.scratch("gguf_dense", w.rows * w.cols).view(w.rows, w.cols)
                    self.launches += 1
                    self.C.gguf_dequant(dense, w.raw, w.type_id)
                    y = self.linear(x, dense, res=None if swiglu else res)
            else:
                y = torch.cat([self.linear(x, p) for p in w.parts], 1)
                self.launches += 1
                if res is not None and not swiglu:
                    y = y + res
                    self.launches += 1
            if swiglu:
                y = self.silu_mul(y)
            return y.float() if out_f32 else y
        if isinstance(w, QWeight) and w.kind == "fp8":
            # ModelOpt FP8 (per-tensor scales, carried per output row): prompt-sized steps multiply the codes on the
            # f8f6f4 tensor path with rows quantised on the fly; few-row steps stream the dequantised copy
            if x.shape[0] > self.mma_gemv_rows[1] and not out_f32 and out is None and w.cols % 128 == 0:
                return self.linear_fp8(x, w.fp8_codes, w.fp8_scales, norm_w, eps, res, swiglu)
            w = w.dense
        if isinstance(w, QWeight) and w.kind == "fp8b":
            # block-scaled e4m3: prompt-sized steps multiply the codes on the f8f6f4 tensor path (activations quantised
            # per 1 x 128 block on the fly); few-row steps stream the dequantised copy through the bf16 row kernels
            if x.shape[0] > self.mma_gemv_rows[1] and not out_f32 and out is None:
                if norm_w is not None:
                    x, _ = self.rmsnorm(x, norm_w, eps, True)
                if swiglu:
                    return self.silu_mul(self.linear_fp8_block(x, w.fp8_codes, w.fp8_scales))
                return self.linear_fp8_block(x, w.fp8_codes, w.fp8_scales, res=res)
            w = w.dense
        if isinstance(w, QWeight):
            M = x.shape[0]
            N = w.rows // 2 if swiglu else w.rows
            if (self.fp4_act and self.fp4_terms > 0 and M <= 8 and w.mma_scales is not None and w.cols % 256 == 0
                    and (not swiglu or N % 128 == 0) and out is None):
                return self._linear_w4_tc(x, w, norm_w, eps, res, swiglu, M, N, out_f32)
            if (self.fp4_act and (self.fp4_prompt or (M <= 8 and self.fp4_terms == 0)) and w.row_alpha is None
                    and w.mma_scales is not None and w.cols % 256 == 0 and (not out_f32 or M <= 8)
                    and (not swiglu or N % 128 == 0) and (M <= 64 or N % 8 == 0)):
                return self._linear_w4a4(x, w, norm_w, eps, res, swiglu, M, N, out_f32)
            if M <= GEMV_MAX_ROWS and not self.force_gemv_chunks:
                N = w.rows // 2 if swiglu else w.rows
                y = self.empty(M, N, dtype=torch.float32 if out_f32 else self.dtype, device=self.device)
                self.launches += 1
                self.C.gemv_nvfp4(y, x, w.packed, w.gemv_scales, w.global_scale, norm_w, res, eps, 1 if swiglu else 0,
                                  w.row_alpha)
                return y
            w = w.dense
        M, K = x.shape
        N = w.shape[0] // 2 if swiglu else w.shape[0]
        # 2..8 rows always; 9..32 rows unless the matrix is very wide (lm_head), where the swapped tcgen05 GEMM with its
        # TMA pipeline measured faster
        if (self.mma_gemv_rows[0] <= M <= self.mma_gemv_rows[1] and K % 32 == 0 and not self.force_gemv_chunks
                and w.stride(0) == K and (M <= 8 or N < 65536)):
            # a few rows (concurrent decode streams, speculative verify): weights streamed once into mma.sync fragments
            y = out if out is not None else self.empty(M, N, dtype=torch.float32 if out_f32 else self.dtype, device=self.device)
            self.launches += 1
            self.C.gemv_mma(y, x, w, norm_w, res, eps, 1 if swiglu else 0, self._workspace(8 << 20), self._counters)
            return y
        if M <= GEMV_MAX_ROWS or self.force_gemv_chunks:
            y = out if out is not None else self.empty(M, N, dtype=torch.float32 if out_f32 else self.dtype, device=self.device)
            for r0 in range(0, M, GEMV_MAX_ROWS):
                r1 = min(M, r0 + GEMV_MAX_ROWS)
                self.launches += 1
                self.C.gemv(y[r0:r1], x[r0:r1], w, norm_w, None if res is None else res[r0:r1], eps, True,
                            1 if swiglu else 0)
            return y
        if norm_w is not None:
            x, _ = self.rmsnorm(x, norm_w, eps, True)
        # the wide-M epilogue stores 16-byte row pieces: give odd widths a padded leading dimension
        y = out if out is not None else self.empty(M, (N + 7) // 8 * 8, dtype=torch.float32 if out_f32 else self.dtype,
                                                    device=self.device)[:, :N]
        split = self._split_k(M, N, K) if M <= 64 else 1
        ws = cnt = None
        if split > 1:
            nb = self.C.gemm_workspace_bytes(M, N, split)
            ws = self._workspace(nb)
            cnt = self._counters
        self.launches += 1
        self.C.gemm(y, x, w, res, (1 if swiglu else 0) | (2 if out_f32 else 0), split, ws, cnt, self.status_word)
        return y

    # ---- FP8 (e4m3) weights and activations -----------------------------------------------------------
    @staticmethod
    def quantize_weight_fp8(w):
        """Per-output-feature e4m3 quantisation of a [N, K] weight: (codes uint8 [N, K], scales fp32 [N])."""
        wf = w.float()
        sc = (wf.abs().amax(1) / 448.0).clamp_min(1e-12)
        q = (wf / sc[:, None]).to(torch.float8_e4m3fn).view(torch.uint8)
        return q.contiguous(), sc.contiguous()

    def linear_fp8(self, x, wq, w_scale, norm_w=None, eps=1e-6, res=None, swiglu=False):
        """y = x W^T with both operands in e4m3 on the tcgen05 f8f6f4 path: rows are quantised on the fly (optionally
        after RMSNorm) with one scale per row; the epilogue applies row scale x feature scale."""
        M, K = x.shape
        N = wq.shape[0] // 2 if swiglu else wq.shape[0]
        xq = self.empty(M, K, dtype=torch.uint8, device=self.device)
        xs = self.empty(M, dtype=torch.float32, device=self.device)
        self.C.quant_fp8(xq, xs, x, norm_w, eps)
        y = self.empty(M, (N + 7) // 8 * 8, dtype=self.dtype, device=self.device)[:, :N]
        split = self._split_k(M, N, K // 2) if M <= 64 else 1
        ws = cnt = None
        if split > 1:
            ws = self._workspace(self.C.gemm_workspace_bytes(M, N, split))
            cnt = self._counters
        self.launches += 2
        self.C.gemm_fp8(y, xq, wq, xs, w_scale, res, 1 if swiglu else 0, split, ws, cnt, self.status_word)
        return y

    @staticmethod
    def quantize_weight_fp8_block(w):
        """128 x 128 block e4m3 quantisation of a [N, K] weight: (codes uint8 [N, ceil(K/128)*128] zero padded, scales
        fp32 [ceil(N/128), ceil(K/128)]), scale = block amax / 448."""
        N, K = w.shape
        nb, kb = (N + 127) // 128, (K + 127) // 128
        wf = torch.zeros(nb * 128, kb * 128, dtype=torch.float32, device=w.device)
        wf[:N, :K] = w.float()
        blocks = wf.view(nb, 128, kb, 128)
        sc = (blocks.abs().amax((1, 3)) / 448.0).clamp_min(1e-12)
        q = (blocks / sc[:, None, :, None]).to(torch.float8_e4m3fn).view(torch.uint8).view(nb * 128, kb * 128)
        return q[:N].contiguous(), sc.contiguous()

    def quantize_act_fp8_block(self, x):
        """Rows to e4m3 with one scale per (row, 128 columns): (codes [M, ceil(K/128)*128], scales fp32 [M, ceil(K/128)])."""
        M, K = x.shape
        kb = (K + 127) // 128
        q = self.empty(M, kb * 128, dtype=torch.uint8, device=self.device)
        sc = self.empty(M, kb, dtype=torch.float32, device=self.device)
        self.launches += 1
        self.C.quant_fp8_block(q, sc, x)
        return q, sc

    def linear_fp8_block(self, x, wq, w_scale, res=None):
        """y = x W^T with block-scaled e4m3 operands (activations 1 x 128, weights 128 x 128): per k block the tensor
        core's partial product is scaled and added into fp32 registers by the epilogue warps."""
        M, K = x.shape
        N = wq.shape[0]
        xq, xs = self.quantize_act_fp8_block(x)
        y = self.empty(M, (N + 7) // 8 * 8, dtype=self.dtype, device=self.device)[:, :N]
        fused = res is not None and res.stride(0) == y.stride(0)       # the kernel reads res with y's row stride
        self.launches += 1
        self.C.gemm_fp8_block(y, xq, xs, wq, w_scale, res if fused else None, K, self.status_word)
        if res is not None and not fused:
            y += res
        return y

    # ---- NVFP4 weights x NVFP4 activations on the block-scaled tensor-core GEMM -------------------------
    def quant_nvfp4(self, x, norm_w=None, eps=1e-6):
        """Quantise activation rows (optionally after RMSNorm) to e2m1 codes + tiled e4m3 scales + per-row scale."""
        M, K = x.shape
        codes = self.empty(M, K // 2, dtype=torch.uint8, device=self.device)
        key = ((M + 127) // 128, K)
        sf = self._sf_pool.get(key)
        if sf is None:
            # zero-initialised once: rows of the last 128-row tile that no call writes keep a finite (zero) scale
            sf = torch.zeros(int(self.C.nvfp4_sf_bytes(M, K)), dtype=torch.uint8, device=self.device)
            self._sf_pool[key] = sf
        rs = self.empty(M, dtype=torch.float32, device=self.device)
        self.launches += 1
        self.C.quant_nvfp4(codes, sf, rs, x, norm_w, eps)
        return codes, sf, rs

    def _linear_w4_tc(self, x, w, norm_w, eps, res, swiglu, M, N, out_f32=False):
        """Few rows: weights stay packed on the block-scaled tensor cores, every activation row goes in as up to
        `fp4_terms` NVFP4 renderings (value, residual, residual of the residual) that the epilogue sums."""
        K = w.cols
        nb = int(self.C.gemv_nvfp4_tc_workspace_bytes(M, N, K, swiglu, self.fp4_terms, self.fp4_tc_ctas))
        y = self.empty(M, N, dtype=torch.float32 if out_f32 else self.dtype, device=self.device)
        self.launches += 1
        nxt = getattr(w, "next", None) if self.fp4_prefetch_mb > 0 else None
        if nxt is not None and (nxt.mma_scales is None or nxt.cols % 256):
            nxt = None
        self.C.gemv_nvfp4_tc(y, x, norm_w, eps, w.packed, w.mma_scales, w.global_scale, w.row_alpha, res,
                             1 if swiglu else 0, self.fp4_terms, self._workspace(max(nb, 16)), self._counters,
                             self.status_word, self.fp4_tc_ctas, None if nxt is None else nxt.packed,
                             None if nxt is None else nxt.mma_scales, 1 if (nxt is not None and nxt.pair) else 0,
                             self.fp4_prefetch_mb << 20)
        return y

    def _linear_w4a4(self, x, w, norm_w, eps, res, swiglu, M, N, out_f32=False):
        split = self._split_k(M, N, w.cols // 4) if M <= 64 else 1
        ws = cnt = None
        if split > 1:
            ws = self._workspace(int(self.C.gemm_nvfp4_workspace_bytes(M, N, split)))
            cnt = self._counters
        if M <= GEMV_MAX_ROWS:
            # decode rows: RMSNorm + activation quantisation happen inside the GEMM kernel
            y = self.empty(M, N, dtype=torch.float32 if out_f32 else self.dtype, device=self.device)
            self.launches += 1
            self.C.gemm_nvfp4_fused(y, x, norm_w, eps, w.packed, w.mma_scales, w.global_scale, res,
                                    1 if swiglu else 0, split, ws, cnt, self.status_word)
            return y
        xq, xsf, rs = self.quant_nvfp4(x, norm_w, eps)
        y = self.empty(M, N, dtype=self.dtype, device=self.device)
        self.launches += 1
        self.C.gemm_nvfp4(y, xq, xsf, rs, w.packed, w.mma_scales, w.global_scale, res, 1 if swiglu else 0, split, ws,
                          cnt, self.status_word)
        return y

    def ffn(self, x, w_gu, w_down, norm_w, eps, res):
        """Dense FFN block: down(SwiGLU(gate|up(norm(x)))) + res. With NVFP4 weights on the block-scaled GEMMs and a
        prompt-sized step the gate|up kernel's epilogue writes the activation already quantised for the down
        projection (one static global scale, `fp4_act_gscale`): the bf16 activation never exists."""
        M = x.shape[0]
        if (self.fp4_fuse_requant and self.fp4_act and self.fp4_prompt and M > 64 and isinstance(w_gu, QWeight)
                and isinstance(w_down, QWeight) and w_gu.kind == w_down.kind == "nvfp4" and w_gu.row_alpha is None
                and w_down.row_alpha is None and w_gu.mma_scales is not None and w_down.mma_scales is not None
                and w_gu.cols % 256 == 0 and w_down.cols % 256 == 0 and (w_gu.rows // 2) % 128 == 0
                and w_down.rows % 8 == 0):
            inter = w_gu.rows // 2
            xq, xsf, rs = self.quant_nvfp4(x, norm_w, eps)
            codes = self.empty(M, inter // 2, dtype=torch.uint8, device=self.device)
            key = ((M + 127) // 128, inter, "act")
            sf = self._sf_pool.get(key)
            if sf is None:
                sf = torch.zeros(int(self.C.nvfp4_sf_bytes(M, inter)), dtype=torch.uint8, device=self.device)
                self._sf_pool[key] = sf
            ars = self.empty(M, dtype=torch.float32, device=self.device)
            gs = self.fp4_act_gscale
            self.launches += 2
            self.C.gemm_nvfp4_swiglu_q(codes, sf, ars, float(gs), xq, xsf, rs, w_gu.packed, w_gu.mma_scales, w_gu.global_scale,
                                       self.status_word)
            y = self.empty(M, w_down.rows, dtype=self.dtype, device=self.device)
            self.C.gemm_nvfp4(y, codes, sf, ars, w_down.packed, w_down.mma_scales, w_down.global_scale, res, 0, 1, None,
                              None, self.status_word)
            return y
        return self.linear(self.linear(x, w_gu, norm_w=norm_w, eps=eps, swiglu=True), w_down, res=res)

    def kv_move_rows(self, k_cache, v_cache, kv_scale, src, dst, seg_off):
        """Cache rows src[i] -> dst[i] (flat row ids, grouped per segment by `seg_off`) in K, V and the scales."""
        self.launches += 1
        self.C.kv_move_rows(k_cache, v_cache, kv_scale, src, dst, seg_off)

    def silu_mul(self, gu):
        out = self.empty(gu.shape[0], gu.shape[1] // 2, dtype=self.dtype, device=self.device)
        self.launches += 1
        self.C.silu_mul(out, gu, 0.0)
        return out

    def gated_norm(self, y, proj, z_off, w, heads, dv, eps):
        out = self.empty(y.shape[0], heads * dv, dtype=self.dtype, device=self.device)
        self.launches += 1
        self.C.gated_norm(out, y, proj, z_off, proj.stride(0), w, heads, dv, eps)
        return out

    # ---- mixture of experts ---------------------------------------------------------------------------
    def moe_route(self, logits, bias, mode, top_k, n_groups, topk_groups, scale, n_exp=0, shared_col=-1, shared_id=-1):
        """Top-k routing. `shared_id` >= 0 appends the shared expert (entry shared_id of the expert stacks) as an extra
        pick weighted by sigmoid(logits[:, shared_col]) (1 when shared_col < 0); `n_exp`: expert columns of `logits`."""
        T = logits.shape[0]
        kout = top_k + (1 if shared_id >= 0 else 0)
        ids = self.empty(T, kout, dtype=torch.int32, device=self.device)
        wts = self.empty(T, kout, dtype=torch.float32, device=self.device)
        self.launches += 1
        self.C.moe_route(ids, wts, logits, bias, mode, n_groups, topk_groups, scale, n_exp, shared_col, shared_id)
        return ids, wts

    def moe_experts(self, h, ids, wts, w_gu, w_down, e_lo, e_hi, shared=None, shared_gate=None, res=None, out_f32=False):
        T, K = ids.shape
        H, inter = h.shape[1], w_down.shape[2]
        if isinstance(w_gu, ExpertsFP4):
            if T > self.moe_pair_rows:
                w_gu, w_down = self.experts_dense(w_gu, 0), self.experts_dense(w_down, 1)
            else:
                # decode rows stream the 4-bit expert rows directly
                act = self.empty(T * K, inter, dtype=self.dtype, device=self.device)
                yp = self.empty(T * K, H, dtype=torch.float32, device=self.device)
                out = self.empty(T, H, dtype=torch.float32 if out_f32 else self.dtype, device=self.device)
                self.launches += 3
                self.C.moe_experts_fp4(out, act, yp, h, w_gu.packed, w_gu.scales, w_gu.global_scale, w_down.packed,
                                       w_down.scales, w_down.global_scale, ids, wts, e_lo, e_hi, shared,
                                       None if shared_gate is None else shared_gate.reshape(-1).float().contiguous(), res)
                return out
        if T > self.moe_pair_rows:
            return self._moe_grouped(h, ids, wts, w_gu, w_down, e_lo, e_hi, shared, shared_gate, res, out_f32)
        act = self.empty(T * K, inter, dtype=self.dtype, device=self.device)
        yp = self.empty(T * K, H, dtype=torch.float32, device=self.device)
        out = self.empty(T, H, dtype=torch.float32 if out_f32 else self.dtype, device=self.device)
        self.launches += 3
        self.C.moe_experts(out, act, yp, h, w_gu, w_down, ids, wts, e_lo, e_hi, shared,
                           None if shared_gate is None else shared_gate.reshape(-1).float().contiguous(), res)
        return out

    def experts_dense(self, w, which: int):
        """bf16 copy of an NVFP4 expert stack in a scratch that all layers share (`which`: 0 gate/up, 1 down): the
        grouped tensor-core GEMM of prompt-sized steps reads it; the next layer's call overwrites it."""
        if not isinstance(w, ExpertsFP4):
            return w
        e, r, k = w.shape
        buf = self._expert_scratch.get(which)
        if buf is None or buf.numel() < e * r * k:
            buf = self.empty(e * r * k, dtype=self.dtype, device=self.device)
            self._expert_scratch[which] = buf
        out = buf[:e * r * k].view(e, r, k)
        self.launches += 1
        self.C.nvfp4_dequant(out, w.packed, w.scales, w.global_scale)
        return out

    def _moe_grouped(self, h, ids, wts, w_gu, w_down, e_lo, e_hi, shared, shared_gate, res, out_f32):
        """Prompt-sized batches: sort the (token, expert) pairs by expert and run one tcgen05 GEMM pair per expert that
        received rows (reference: sorted pair list + segmented GEMM, `kernels/k-gguf/src/sort.rs`, `mmq.rs:522`)."""
        T, K = ids.shape
        flat = ids.reshape(-1).long()
        order = torch.argsort(flat, stable=True)
        tok = (order // K)
        counts = torch.bincount(flat, minlength=e_hi)[e_lo:e_hi].tolist()
        start = int((flat < e_lo).sum())
        out = torch.zeros(T, h.shape[1], dtype=torch.float32, device=self.device)
        wflat = wts.reshape(-1)
        for j, n in enumerate(counts):
            if n == 0:
                continue
            sel = order[start:start + n]
            rows = tok[start:start + n]
            xe = h[rows].contiguous()
            a = self.linear(xe, w_gu[j], swiglu=True)
            y = self.linear(a, w_down[j])
            out.index_add_(0, rows, y.float() * wflat[sel][:, None])
            start += n
        if shared is not None:
            g = torch.sigmoid(shared_gate.float()).reshape(-1, 1) if shared_gate is not None else 1.0
            out += shared.float() * g
        if res is not None:
            out += res.float()
        return out if out_f32 else out.to(self.dtype)

    # ---- attention ---------------------------------------------------------------------------------
    def attn_prep(self, proj, q_norm, k_norm, inv_freq, row_slot, row_pos, block_table, k_cache, v_cache, kv_block,
                  nq, nkv, hd, rot, gated, eps, kv_scale=None, row_cpos=None, hrot=False, kv_bits=None):
        """q/k RMSNorm + partial RoPE, K/V rows into the paged cache (bf16, or e4m3 / 6-bit / 4-bit codes + scales when
        `kv_scale` is given; the byte width of the cache rows tells the form). `row_cpos`: cache row of each row when it
        differs from its rotary position (trees). `hrot`: queries and keys leave in a Walsh-Hadamard rotated basis."""
        q = self.empty(proj.shape[0], nq, hd, dtype=self.dtype, device=self.device)
        self.launches += 1
        self.C.attn_prep(q, k_cache, v_cache, proj, q_norm, k_norm, inv_freq, row_slot, row_pos, block_table,
                         kv_block, nq, nkv, hd, rot, gated, eps, self.status_word, kv_scale, row_cpos, 1 if hrot else 0)
        return q

    def attention(self, q, proj, k_cache, v_cache, row_slot, row_kvlen, block_table, kv_block, nq, nkv, hd, gated,
                  row_base=None, row_mask=None, nsplit=1, kv_scale=None, segs=None):
        """Split-KV decode / verify / tree attention. With `segs` = (seg_slot, seg_row0, seg_nrows, max rows per
        segment) and a bf16 cache the tensor-core kernel runs: the rows of a segment share one pass over the K/V of
        each kv head (bf16 and e4m3 caches). The 4-bit cache and callers without segment tables take the SIMT kernel."""
        T = q.shape[0]
        out = self.empty(T, nq * hd, dtype=self.dtype, device=self.device)
        o_part = self.empty(T, nq, nsplit, hd, dtype=torch.float32, device=self.device)
        ml_part = self.empty(T, nq, nsplit, 2, dtype=torch.float32, device=self.device)
        self.launches += 2
        fp8_cache = kv_scale is not None and k_cache.shape[-1] == hd           # (the 4-bit cache has hd / 2 bytes per row)
        if segs is not None and (kv_scale is None or fp8_cache) and self.attn_mma and nq // nkv <= 64:
            rc = self.C.attn_decode_mma(out, o_part, ml_part, q, k_cache, v_cache, proj, segs[0], segs[1], segs[2], segs[3],
                                        row_kvlen, row_base, row_mask, block_table, kv_block, nq, nkv, hd, nsplit, gated,
                                        kv_scale if fp8_cache else None)
            if rc == 0:
                return out
        self.C.attn_decode(out, o_part, ml_part, q, k_cache, v_cache, proj, row_slot, row_kvlen, row_base, row_mask,
                           block_table, kv_block, nq, nkv, hd, nsplit, gated, kv_scale)
        return out

    def attention_prefill(self, q, proj, k_cache, v_cache, seg_slot, seg_row0, seg_nrows, seg_pos0, block_table,
                          kv_block, nq, nkv, hd, gated, max_rows, row_slot=None, row_kvlen=None, kv_scale=None,
                          max_kvlen=None):
        """Causal flash attention over prompt segments (their K/V rows are already in the cache). With an e4m3 cache
        the visible rows are first decoded into a per-slot bf16 scratch that the kernel reads through an identity
        block table."""
        out = self.empty(q.shape[0], nq * hd, dtype=self.dtype, device=self.device)
        if kv_scale is not None:
            n_slots, max_blocks = block_table.shape
            toks = max_blocks * kv_block
            key = (n_slots, toks, nkv, hd)
            if self._kv_scratch is None or self._kv_scratch[0] != key:
                # zeros: rows past the decoded ones are masked by causality but still multiplied (0 x value) by the
                # tensor-core kernel, so they must hold finite numbers
                ks = torch.zeros(n_slots * max_blocks, kv_block, nkv, hd, dtype=self.dtype, device=self.device)
                vs = torch.zeros_like(ks)
                ident = torch.arange(n_slots * max_blocks, dtype=torch.int32, device=self.device).view(n_slots, max_blocks)
                self._kv_scratch = (key, ks, vs, ident.contiguous())
            _, ks, vs, ident = self._kv_scratch
            self.launches += 1
            self.C.kv_dequant(ks, vs, k_cache, v_cache, kv_scale, seg_slot, seg_pos0, seg_nrows, block_table, kv_block,
                              toks if max_kvlen is None else max_kvlen, nkv, hd, toks)
            k_cache, v_cache, block_table = ks, vs, ident
        self.launches += 1
        if self.attn_tc and hd in (64, 128, 256) and kv_block % 64 == 0:
            # tcgen05 / TMEM kernel (TMA-fed, 128 query rows per CTA); other shapes take the mma.sync kernel
            rc = self.C.attn_prefill_tc(out, q.view(q.shape[0], nq * hd), k_cache, v_cache, proj, seg_slot, seg_row0,
                                        seg_nrows, seg_pos0, block_table, kv_block, max_rows, nq, nkv, hd, gated,
                                        self.status_word)
            if rc == 0:
                return out
        self.C.attn_prefill(out, q, k_cache, v_cache, proj, seg_slot, seg_row0, seg_nrows, seg_pos0, block_table,
                            kv_block, max_rows, nq, nkv, hd, gated)
        return out

    # ---- gated delta net ---------------------------------------------------------------------------
    def gdn_conv(self, proj, conv_w, conv_state, seg_slot, seg_row0, seg_nrows, conv_dim, max_rows=None):
        out = self.empty(proj.shape[0], conv_dim, dtype=self.dtype, device=self.device)
        self.launches += 1
        self.C.gdn_conv(out, proj, conv_w, conv_state, seg_slot, seg_row0, seg_nrows,
                        proj.shape[0] if max_rows is None else max_rows)
        return out

    def gdn_conv_tree(self, proj, conv_w, conv_state, seg_slot, seg_row0, seg_nrows, conv_dim, row_parent):
        """Conv over verify-tree rows: a row's window is its three nearest ancestors, then the slot's saved tail."""
        out = self.empty(proj.shape[0], conv_dim, dtype=self.dtype, device=self.device)
        self.launches += 1
        self.C.gdn_conv_tree(out, proj, conv_w, conv_state, seg_slot, seg_row0, seg_nrows, row_parent)
        return out

    def gdn_rec_tree(self, qkv, proj, rec_state, A_log, dt_bias, seg_slot, seg_row0, seg_nrows, row_parent, row_flags, nk,
                     nv, dk, dv, eps):
        """Recurrence over verify-tree rows (read-only): every row starts from the state its parent left. Branch-point
        states are parked in a scratch of rows x heads x dk x dv floats that all layers share."""
        T = qkv.shape[0]
        y = self.empty(T, nv * dv, dtype=torch.float32, device=self.device)
        need = T * nv * dk * dv
        if self._tree_scratch is None or self._tree_scratch.numel() < need:
            self._tree_scratch = self.empty(need, dtype=torch.float32, device=self.device)
        self.launches += 1
        self.C.gdn_rec_tree(y, rec_state, qkv, proj, A_log, dt_bias, seg_slot, seg_row0, seg_nrows, row_parent, row_flags,
                            self._tree_scratch, nk, nv, dk, dv, eps)
        return y

    def decode_layers(self, comm, x, layers, seg_slot=None, heads=(0, 0, 0), eps=1e-6):
        """A run of consecutive decoder layers for one-row-per-sequence steps as ONE persistent launch
        (`csrc/decode_layer.cu`). `layers`: dicts with w_out, post_norm, w_gu, w_down and either `o` (the mixer output of a
        layer whose attention already ran; first layer of the run only) or the Gated DeltaNet operands w_in, input_norm,
        rec, conv, conv_w, A_log, dt_bias, gnorm_w. `comm`: the tensor-parallel workspace handle (the sums over ranks
        happen inside the kernel) or None. Returns the output rows of every layer of the run."""
        M, H = x.shape
        e = self._dl_empty
        mk = lambda n: self.empty(M, n, dtype=self.dtype, device=self.device)
        cols = {k: [] for k in ("sp", "x_out", "x_mid", "act", "proj", "o", "w_in", "inorm", "w_out", "pnorm", "w_gu", "w_down",
                                "rec", "conv", "conv_w", "A_log", "dt_bias", "gnorm")}
        for L in layers:
            gdn = "o" not in L
            cols["sp"].append(1 if gdn else 3)
            cols["x_out"].append(mk(H)); cols["x_mid"].append(mk(H)); cols["act"].append(mk(L["w_down"].shape[1]))
            cols["proj"].append(mk(L["w_in"].shape[0]) if gdn else e)
            cols["o"].append(mk(L["w_out"].shape[1]) if gdn else L["o"])
            cols["w_in"].append(L["w_in"] if gdn else e); cols["inorm"].append(L["input_norm"] if gdn else e)
            cols["w_out"].append(L["w_out"]); cols["pnorm"].append(L["post_norm"]); cols["w_gu"].append(L["w_gu"])
            cols["w_down"].append(L["w_down"])
            for k in ("rec", "conv", "conv_w", "A_log", "dt_bias"):
                cols[k].append(L[k] if gdn else e)
            cols["gnorm"].append(L["gnorm_w"] if gdn else e)
        self.launches += 1
        nk, nv, dk = heads
        self.C.decode_layers(comm, cols["sp"], x, cols["x_out"], cols["x_mid"], cols["act"], cols["proj"], cols["o"], cols["w_in"],
                             cols["inorm"], cols["w_out"], cols["pnorm"], cols["w_gu"], cols["w_down"], cols["rec"], cols["conv"],
                             cols["conv_w"], cols["A_log"], cols["dt_bias"], cols["gnorm"], seg_slot, nk, nv, dk, eps,
                             self.status_word, self._dl_sync)
        return cols["x_out"]

    def gdn_step(self, proj, conv_w, rec_state, conv_state, A_log, dt_bias, gnorm_w, seg_slot, seg_row0, seg_nrows, nk, nv,
                 dk, dv, eps, commit=True):
        """Decode rows: conv + recurrence + gated norm in one launch; returns bf16 [rows, nv * dv]."""
        out = self.empty(proj.shape[0], nv * dv, dtype=self.dtype, device=self.device)
        self.launches += 1
        self.C.gdn_step(out, rec_state, conv_state, proj, conv_w, A_log, dt_bias, gnorm_w, seg_slot, seg_row0, seg_nrows, nk,
                        nv, dk, dv, eps, commit)
        return out

    def gdn_rec(self, qkv, proj, rec_state, conv_state, A_log, dt_bias, seg_slot, seg_row0, seg_nrows, nk, nv, dk, dv,
                eps, commit=True, chunked=False, max_rows=None):
        y = self.empty(qkv.shape[0], nv * dv, dtype=torch.float32, device=self.device)
        if chunked and dk == 128 and dv % 16 == 0:
            nb = int(self.C.gdn_chunk_scratch_bytes(qkv.shape[0], seg_slot.numel(), nv, dk))
            if self._gdn_scratch is None or self._gdn_scratch.numel() < nb:
                self._gdn_scratch = self.empty(nb, dtype=torch.uint8, device=self.device)
            self.launches += 2
            self.C.gdn_chunk(y, rec_state, conv_state, self._gdn_scratch, qkv, proj, A_log, dt_bias, seg_slot, seg_row0,
                             seg_nrows, qkv.shape[0] if max_rows is None else max_rows, nk, nv, dk, dv, eps, commit)
            return y
        self.launches += 1
        self.C.gdn_rec(y, rec_state, conv_state, qkv, proj, A_log, dt_bias, seg_slot, seg_row0, seg_nrows, nk, nv,
                       dk, dv, eps, commit)
        return y

    # ---- multi-head latent attention (absorbed form) ----------------------------------------------------
    def mla_prep(self, q, kva, norm_w, w_uk_t, inv_freq, row_slot, row_pos, block_table, cache, kv_block, nq, dn, L, R, eps,
                 absorb=True):
        """Latent rows into the paged cache and the absorbed queries [T, nq, L + R]. `absorb=False` leaves the first L
        columns of every query unwritten (the expanded prompt path only reads the rotated rope tail)."""
        T = q.shape[0]
        qabs = self.empty(T, nq, L + R, dtype=self.dtype, device=self.device)
        self.launches += 1
        self.C.mla_prep(cache, qabs, kva, q, norm_w, inv_freq, row_slot, row_pos, block_table, kv_block, nq, dn, L, R, eps,
                        self.status_word)
        if absorb:
            # key up-projection folded into the query: one small linear per head
            self.head_linear(q.view(T, nq, dn + R)[:, :, :dn], w_uk_t, out=qabs[:, :, :L])
        return qabs

    def mla_attention_prefill(self, q, qabs, cache, kv_b, segs, seg_row0, seg_nrows, seg_pos0, block_table, kv_block,
                              nq, dn, dv, L, R):
        """Latent attention of prompt segments in the expanded form on the tcgen05 flash kernel. `segs`: host list of
        (slot, pos0, rows) per segment; the context's latent rows are gathered through the block table, expanded to
        per-head keys / values by one GEMM with `kv_b` [nq (dn + dv), L], packed (padded to the kernel's head width) into
        a scratch laid out segment after segment, and read through a step-local page table. Returns [T, nq * dv]."""
        T = q.shape[0]
        HP = 64 if max(dn + R, dv) <= 64 else 128 if max(dn + R, dv) <= 128 else 256
        starts, tables, tot = [], [], 0
        for slot, pos0, n in segs:
            nb = (pos0 + n + kv_block - 1) // kv_block
            starts.append((slot, tot, nb))
            tot += nb
        max_nb = max(nb for _, _, nb in starts)
        pages = torch.cat([block_table[slot, :nb] for slot, _, nb in starts]).long()
        lat = cache.view(-1, kv_block, L + R)[pages].view(tot * kv_block, L + R)            # the segments' latent rows
        kvx = self.linear(lat[:, :L].contiguous(), kv_b)                                     # [rows, nq (dn + dv)]
        kp = self.empty(tot, kv_block, nq, HP, dtype=self.dtype, device=self.device)
        vp = self.empty(tot, kv_block, nq, HP, dtype=self.dtype, device=self.device)
        qp = self.empty(T, nq, HP, dtype=self.dtype, device=self.device)
        self.launches += 2
        self.C.mla_expand(kp, vp, kvx, lat, nq, dn, dv, L, R)
        self.C.mla_qpad(qp, q, qabs, nq, dn, L, R, math.sqrt(HP / (dn + R)))
        table = torch.tensor([[s0 + min(j, nb - 1) for j in range(max_nb)] for _, s0, nb in starts], dtype=torch.int32)
        table = table.pin_memory().to(self.device, non_blocking=True)
        own = torch.arange(len(segs), dtype=torch.int32, device=self.device)
        o = self.attention_prefill(qp, qp.view(T, nq * HP), kp, vp, own, seg_row0, seg_nrows, seg_pos0, table, kv_block,
                                   nq, nq, HP, False, max(n for _, _, n in segs))
        return o.view(T, nq, HP)[:, :, :dv].contiguous().view(T, nq * dv)

    def mla_attention(self, qabs, cache, row_slot, row_kvlen, block_table, kv_block, nq, L, R, scale, nsplit=1):
        T = qabs.shape[0]
        out = self.empty(T, nq, L, dtype=self.dtype, device=self.device)
        o_part = self.empty(T * nq * nsplit * L, dtype=torch.float32, device=self.device)
        ml_part = self.empty(T * nq * nsplit * 2, dtype=torch.float32, device=self.device)
        self.launches += 2
        self.C.mla_attn(out, o_part, ml_part, qabs, cache, row_slot, row_kvlen, block_table, kv_block, nq, L, R, nsplit,
                        scale)
        return out

    def mla_out(self, ol, w_uv):
        T, nq, L = ol.shape
        dv = w_uv.shape[1]
        return self.head_linear(ol, w_uv).view(T, nq * dv)

    def head_linear(self, x, W, out=None):
        """y[t, h, :] = W[h] x[t, h, :]: x [T, heads, K] (a view with unit inner stride), W [heads, N, K]. Up to 8 rows:
        one launch of the row kernel streams the stack once; more rows: head-major copies around one batched tcgen05
        GEMM (every head a group of T rows)."""
        T, nh, K = x.shape
        N = W.shape[1]
        y = out if out is not None else self.empty(T, nh, N, dtype=self.dtype, device=self.device)
        if T <= 8 or K % 64 or N % 8 or nh * T < 256 or nh * N < 256:      # the GEMM's 128/256-row boxes fit the operands
            self.launches += 1
            self.C.head_linear(y, x, W)
            return y
        xh = self.empty(nh, T, K, dtype=self.dtype, device=self.device)
        xh.copy_(x.transpose(0, 1))
        yh = self.empty(nh, T, N, dtype=self.dtype, device=self.device)
        self.launches += 3
        self.C.gemm_batched(yh, xh, W, self.status_word)
        y.copy_(yh.transpose(0, 1))
        return y

    # ---- drafter kernels ---------------------------------------------------------------------------
    def w4_gemv(self, x, qweight, scales, biases, res=None):
        """y = x W^T, W affine 4-bit in groups of 64: qweight uint32/int32 [N, K/8], scales / biases bf16 [N, K/64]."""
        y = self.empty(x.shape[0], qweight.shape[0], dtype=self.dtype, device=self.device)
        self.launches += 1
        self.C.w4_gemv(y, x, qweight, scales, biases, res)
        return y

    # ---- hyper-connection streams: res [rows, hc, d] fp32 ------------------------------------------------
    def hc_norm(self, res, w, eps):
        """Per-stream RMSNorm of the residual streams to bf16: returns (y [rows * hc, d], inv [rows * hc]); `w` [ngw, d]
        fp32, stream g uses row g % ngw."""
        rows, hc, d = res.shape
        y = self.empty(rows * hc, d, dtype=self.dtype, device=self.device)
        inv = self.empty(rows * hc, dtype=torch.float32, device=self.device)
        self.launches += 1
        self.C.hc_norm(y, inv, res.view(rows * hc, d), w, eps)
        return y, inv

    def hc_mix(self, res, inv, w, gate):
        """mixed[r] = mean over streams of (normalised stream * w[s]) * sigmoid(gate[r][s]); fp32 [rows, d]."""
        rows, hc, d = res.shape
        mixed = self.empty(rows, d, dtype=torch.float32, device=self.device)
        self.launches += 1
        self.C.hc_mix(mixed, res, inv, w, gate)
        return mixed

    def hc_combine(self, res, out, inj):
        """res[r][s] += out[r] * 2 sigmoid(inj[r][s]) in place (`inj` may be a column slice of a wider projection)."""
        self.launches += 1
        self.C.hc_combine(res, out, inj)
        return res

    def dynconv(self, x, coef, base, group, blk, res=None):
        """Grouped dynamic causal conv over draft blocks of `blk` rows: y[t] = (base[0] + c[t][g]) x[t] + (base[1] +
        c[t][G + g]) x[t-1] (second term only inside a block). `coef` [rows, 2 * H / group] may be a column slice of a
        wider projection. With `res` the result is added into it in place and `res` is returned."""
        out = res if res is not None else torch.empty_like(x)
        self.launches += 1
        self.C.dynconv(out, x, coef, base, res, group, blk)
        return out

    def topk16_merge(self, vals, ids):
        """[W, rows, 16] per-rank top-16 lists (global ids) -> merged ([rows, 16] vals, ids), ties to the lower id."""
        W, rows, _ = vals.shape
        ov = self.empty(rows, 16, dtype=torch.float32, device=self.device)
        oi = self.empty(rows, 16, dtype=torch.int32, device=self.device)
        self.launches += 1
        self.C.topk16_merge(ov, oi, vals.contiguous(), ids.contiguous())
        return ov, oi

    def draft_select(self, vals, ids, gate, a_cb, b_cb, anchor):
        """Candidate selector walk: per drafted row pick argmax_c vals[c] + <A[pred] * gate, B[ids[c]]>, pred chained."""
        out = self.empty(vals.shape[0], dtype=torch.int32, device=self.device)
        self.launches += 1
        self.C.draft_select(out, vals, ids, gate, a_cb, b_cb, int(anchor))
        return out

    def topk16(self, logits):
        ids = self.empty(logits.shape[0], 16, dtype=torch.int32, device=self.device)
        vals = self.empty(logits.shape[0], 16, dtype=torch.float32, device=self.device)
        self.launches += 1
        self.C.topk16(ids, vals, logits)
        return ids, vals

    # ---- GGUF block formats ------------------------------------------------------------------------
    def gguf_dequant(self, raw, type_id, shape):
        """raw: uint8 tensor of GGUF blocks on the device -> bf16 tensor of `shape`."""
        out = self.empty(shape, dtype=torch.bfloat16, device=self.device)
        self.launches += 1
        self.C.gguf_dequant(out, raw, type_id)
        return out

    def gguf_gemv(self, x, raw, type_id, N, res=None):
        """y = x W^T for up to 8 rows with W [N, K] kept in its GGUF blocks."""
        y = self.empty(x.shape[0], N, dtype=torch.bfloat16, device=self.device)
        self.launches += 1
        self.C.gguf_gemv(y, x, raw, type_id, N, res)
        return y

    def q8_1_quant(self, x):
        out = self.empty(x.numel() // 32 * 36, dtype=torch.uint8, device=self.device)
        self.launches += 1
        self.C.q8_1_quant(out, x.contiguous())
        return out

    def sample(self, logits, samplings, seeds, counts=None):
        """One draw per row on the device: temperature, penalties (with `counts` [rows, vocab] int32), top-k, top-p
        inside the top-k set, min-p; `samplings` are `engine.sampler.Sampling` objects, `seeds` one integer per row.
        Same filter order as the host sampler (`engine/sampler.py::dist`)."""
        import numpy as np
        rows, vocab = logits.shape
        rec = np.zeros(rows, dtype=np.dtype([("temperature", "f4"), ("top_p", "f4"), ("min_p", "f4"), ("presence", "f4"),
                                             ("frequency", "f4"), ("repetition", "f4"), ("top_k", "i4"), ("pad", "i4"),
                                             ("seed", "u8")]))
        for i, (sp, seed) in enumerate(zip(samplings, seeds)):
            rec[i] = (sp.temperature, sp.top_p, sp.min_p, sp.presence_penalty, sp.frequency_penalty,
                      sp.repetition_penalty, sp.top_k, 0, int(seed) & 0xFFFFFFFFFFFFFFFF)
        params = torch.from_numpy(rec.view(np.uint8)).to(self.device)
        ids = self.empty(rows, dtype=torch.int32, device=self.device)
        work = self.empty(rows, vocab, dtype=torch.float32, device=self.device)
        self.launches += 1
        self.C.sample(ids, logits, params, counts, work)
        return ids

    def argmax(self, logits):
        ids = self.empty(logits.shape[0], dtype=torch.int32, device=self.device)
        finite = self.empty(logits.shape[0], dtype=torch.int32, device=self.device)
        scratch = self.empty(logits.shape[0] * 64 * 3, dtype=torch.int32, device=self.device)
        self.launches += 2 if logits.shape[1] >= 8192 else 1
        self.C.argmax(ids, logits, None, finite, scratch)
        return ids, finite
