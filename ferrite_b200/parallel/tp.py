"""Tensor parallelism inside one NVSwitch box: one process per GPU, `torch.distributed` for the plumbing, and
hand-written kernels that reduce over NVLink peer memory for the hot paths.

The reference runs TP=2 over RoCE between two boxes: a TCP bootstrap, NCCL for prompt-sized reductions and a
custom one-shot exchange for decode-sized ones (`crates/fe-fabric/src/lib.rs:62-203`, `crates/fe-model/src/tp.rs`,
reduction site `crates/fe-model/src/model.rs:1761-1797`). Here:

* bootstrap / control = the process group the caller built (NCCL on GPUs, gloo on CPU ranks);
* the symmetric workspace (flags + staging slots, mapped on every rank) comes from
  `torch.distributed._symmetric_memory`; kernels get the table of peer base pointers;
* decode-sized reductions (<= 8 rows) are fused into the producing GEMV (`fb_gemv_allreduce`), up to
  `ONESHOT_MAX` elements go through the one-shot P2P all-reduce kernel, larger ones through NCCL (the baseline);
* ranks sum in rank order, so every rank holds identical bits (the reference's rule, `TP2.md:58-71`).

`fused=False` (or a CPU device) keeps every collective on the process group: that is the baseline path and the
one the CPU multi-rank tests run.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

MAX_CTAS = 1024
SLOT_FLOATS = 512 * 1024
ONESHOT_MAX = (SLOT_FLOATS - 1024) // 2     # a slot holds (value, epoch) pairs below the argmax candidates


class TensorParallel:
    def __init__(self, group, device, fused: bool = True, spin_limit: int = 0):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device)
        self.fused = bool(fused) and self.device.type == "cuda" and self.world > 1
        self.comm = None
        self.stats = {"fused_gemv": 0, "oneshot": 0, "nccl": 0}
        self.big = None
        self.sp_max = None
        if self.fused:
            self._setup_symmetric(spin_limit)

    # ---- symmetric workspace ---------------------------------------------------------------------------
    def _setup_symmetric(self, spin_limit: int) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        from .._ext import load
        C = load()
        nbytes = int(C.comm_workspace_bytes(MAX_CTAS, SLOT_FLOATS))
        name = self.group.group_name
        try:
            symm_mem.enable_symm_mem_for_group(name)
        except Exception:
            pass
        self.ws = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.hdl = symm_mem.rendezvous(self.ws, group=name)
        self.ws.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)                       # nobody pushes before every rank has zeroed its flags
        self.epochs = torch.zeros(MAX_CTAS, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        sm = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.max_resident = 2 * sm                     # every CTA of a fused kernel must be resident at once
        ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        self.comm = C.make_comm(ptrs, self.rank, MAX_CTAS, SLOT_FLOATS, self.epochs, self.status, spin_limit,
                                self.max_resident)
        self.C = C
        self.slot_floats = SLOT_FLOATS
        self.data_offset = 2 * 8 * MAX_CTAS * 4                    # bytes of the flag area in front of the data slots

    # ---- sequence-parallel prompt path: all-gather -> GEMM and GEMM -> reduce-scatter ------------------------
    def setup_big(self, max_rows: int, max_cols: int, spin_limit: int = 0) -> None:
        """Allocate the large symmetric workspace (staging slots of the reduce-scatter, the gathered-X buffer, flags)
        for steps of up to `max_rows` rows and row widths up to `max_cols`. Collective: every rank calls it."""
        self.sp_max = (int(max_rows), int(max_cols))
        if not self.fused:
            return
        import torch.distributed._symmetric_memory as symm_mem
        C = self.C
        nbytes = int(C.big_workspace_bytes(self.world, max_rows, max_cols))
        self.big_ws = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.big_hdl = symm_mem.rendezvous(self.big_ws, group=self.group.group_name)
        self.big_ws.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        self.big_ctr = torch.zeros(2 + (max_rows + 127) // 128 + 62, dtype=torch.int32, device=self.device)
        sm = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.big = C.make_big_comm([int(p) for p in self.big_hdl.buffer_ptrs], self.rank, max_rows, max_cols,
                                   self.big_ctr, self.status, spin_limit, sm)
        self.xfull_off = int(C.big_xfull_offset(self.world, max_rows, max_cols))

    def sp_ready(self, T: int) -> bool:
        return self.world > 1 and T > 64 and self.sp_max is not None and T <= self.sp_max[0]

    def shard_rows(self, T: int):
        per = (T + self.world - 1) // self.world
        lo = min(T, self.rank * per)
        return lo, min(T, lo + per)

    def _xfull(self, T: int, K: int) -> torch.Tensor:
        return self.big_ws[self.xfull_off:self.xfull_off + T * K * 2].view(torch.bfloat16).view(T, K)

    def ag_linear(self, ops, x_shard, w, norm_w, eps, T: int, swiglu: bool = False):
        """y[T, N_local] = (all-gather over ranks of norm(x_shard)) W^T, SwiGLU optional."""
        K = x_shard.shape[1]
        lo, hi = self.shard_rows(T)
        if self.fused and self.big is not None and K <= self.sp_max[1]:
            xf = self._xfull(T, K)
            if norm_w is not None:
                ops.rmsnorm(x_shard, norm_w, eps, True, out=xf[lo:hi])
            else:
                xf[lo:hi].copy_(x_shard)
            N = w.shape[0] // 2 if swiglu else w.shape[0]
            y = torch.empty(T, (N + 7) // 8 * 8, dtype=x_shard.dtype, device=x_shard.device)[:, :N]
            self.C.ag_gemm(self.big, y, w, None, K, 1 if swiglu else 0)
            ops.launches += 1
            self.stats["ag_gemm"] = self.stats.get("ag_gemm", 0) + 1
            return y
        h = ops.rmsnorm(x_shard, norm_w, eps, True)[0] if norm_w is not None else x_shard
        return ops.linear(self.gather_rows(h, T), w, swiglu=swiglu)

    def rs_linear(self, ops, act, w, res_shard, T: int):
        """y_shard = rows of this rank of (sum over ranks of act W^T) + res_shard."""
        lo, hi = self.shard_rows(T)
        N = w.shape[0]
        if self.fused and self.big is not None and N <= self.sp_max[1]:
            y = torch.empty(hi - lo, N, dtype=act.dtype, device=act.device)
            self.C.gemm_rs(self.big, y, act, w, res_shard)
            ops.launches += 1
            self.stats["gemm_rs"] = self.stats.get("gemm_rs", 0) + 1
            return y
        part = ops.linear(act, w)
        buf = part.float() if part.device.type == "cpu" else part
        dist.all_reduce(buf, group=self.group)
        out = buf[lo:hi].float()
        return (out + res_shard.float() if res_shard is not None else out).to(act.dtype)

    def gather_rows(self, x_shard, T: int):
        """All-gather of row shards into the full [T, H] tensor (process group; once per step and per tap)."""
        per = (T + self.world - 1) // self.world
        pad = torch.zeros(per, x_shard.shape[1], dtype=x_shard.dtype, device=x_shard.device)
        pad[:x_shard.shape[0]] = x_shard
        out = torch.empty(self.world * per, x_shard.shape[1], dtype=x_shard.dtype, device=x_shard.device)
        dist.all_gather_into_tensor(out, pad, group=self.group)
        return out[:T]

    def selftest(self) -> None:
        """Start-up check of every ordered pair of ranks (see `parallel/selftest.py`); every rank calls it."""
        from .selftest import p2p_selftest
        p2p_selftest(self)

    def check(self) -> None:
        """Raise when a peer wait ran out (the kernel returned normally and left a status code)."""
        if self.fused and int(self.status.item()) != 0:
            raise RuntimeError(f"tensor-parallel rank {self.rank}: peer wait timed out (status {int(self.status.item())})")

    # ---- row-parallel projection + all-reduce + residual --------------------------------------------------
    def linear_allreduce(self, ops, x, w, res):
        M, N = x.shape[0], w.shape[0]
        kind = getattr(w, "kind", None)
        fp4 = kind == "nvfp4"
        if kind in ("fp8b", "fp8") and M <= 8:
            w, kind = w.dense, None                      # few rows: the dequantised copy through the bf16 row kernels
        if self.fused and M <= 8 and kind in (None, "nvfp4") and not (fp4 and getattr(ops, "fp4_act", False) and getattr(ops, "fp4_terms", 0) >= 0 and w.row_alpha is None):
            y = torch.empty(M, N, dtype=x.dtype, device=x.device)
            if fp4:
                self.C.gemv_nvfp4_allreduce(self.comm, y, x, w.packed, w.gemv_scales, w.global_scale, res, w.row_alpha)
            else:
                self.C.gemv_allreduce(self.comm, y, x, w, res)
            ops.launches += 1
            self.stats["fused_gemv"] += 1
            return y
        part = ops.linear(x, w)
        if self.fused and M * N <= ONESHOT_MAX:
            y = torch.empty_like(part)
            self.C.allreduce_oneshot(self.comm, y, part, res)
            ops.launches += 1
            self.stats["oneshot"] += 1
            return y
        self.stats["nccl"] += 1
        if part.device.type == "cpu":
            part = part.float()
        dist.all_reduce(part, group=self.group)
        if res is not None:
            part = (part.float() + res.float()).to(res.dtype) if part.device.type == "cpu" else part.add_(res)
        return part.to(x.dtype)

    def allreduce_rows(self, ops, part, res):
        """Sum [rows, n] partials over the ranks (rank order) and add the residual: the combine step of the expert-
        parallel MoE block, where every rank holds the partial output of the experts it owns."""
        if self.fused and part.numel() <= ONESHOT_MAX:
            part = part.contiguous()
            y = torch.empty(part.shape, dtype=torch.bfloat16, device=part.device)     # the kernel rounds the sum to bf16
            self.C.allreduce_oneshot(self.comm, y, part, res)
            ops.launches += 1
            self.stats["oneshot"] += 1
            return y
        self.stats["nccl"] += 1
        buf = part.float() if part.device.type == "cpu" else part.clone()
        dist.all_reduce(buf, group=self.group)
        if res is not None:
            buf = buf.float() + res.float()
        return buf.to(res.dtype if res is not None else part.dtype)

    # ---- vocabulary-parallel head -----------------------------------------------------------------------------
    def gather_logits(self, ops, logits, greedy: bool, vocab_offset: int, vocab: int):
        """logits: this rank's shard [rows, n_local] fp32. greedy: (None, (ids, finite)) with ids merged over ranks
        (only (max, index) pairs cross the link). Otherwise the full [rows, vocab] logits on every rank."""
        rows, n_local = logits.shape
        if greedy and self.fused and rows <= MAX_CTAS:
            ids = torch.empty(rows, dtype=torch.int32, device=logits.device)
            vals = torch.empty(rows, dtype=torch.float32, device=logits.device)
            self.C.argmax_gather(self.comm, ids, logits, vocab_offset, vals)
            ops.launches += 1
            finite = torch.isfinite(vals).to(torch.int32)
            return None, (ids, finite)
        per = (vocab + self.world - 1) // self.world
        pad = torch.full((rows, per), float("-inf"), dtype=torch.float32, device=logits.device)
        pad[:, :n_local] = logits
        full = torch.empty(self.world, rows, per, dtype=torch.float32, device=logits.device)
        dist.all_gather_into_tensor(full, pad, group=self.group) if logits.device.type == "cuda" else \
            dist.all_gather(list(full.unbind(0)), pad, group=self.group)
        full = full.permute(1, 0, 2).reshape(rows, self.world * per)[:, :vocab].contiguous()
        if greedy:
            ids, finite = ops.argmax(full)
            return full, (ids, finite)
        return full, None

    def broadcast_object(self, obj, src: int = 0):
        """Control plane: rank 0's step descriptor to every rank (reference: the follower RPC stream,
        `crates/fe-model/src/follow.rs`)."""
        box = [obj]
        dist.broadcast_object_list(box, src=src, group=self.ctrl_group())
        return box[0]

    def ctrl_group(self):
        """CPU-side (gloo) group for control records, so they neither touch the GPUs nor wait on their streams. Created
        on first use: every rank must reach its first `broadcast_object` together."""
        if getattr(self, "_ctrl", None) is None:
            self._ctrl = self.group if dist.get_backend(self.group) == "gloo" else dist.new_group(backend="gloo")
        return self._ctrl
