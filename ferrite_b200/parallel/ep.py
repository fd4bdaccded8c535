"""Expert parallelism for prompt-sized batches: tokens sharded by rows over the ranks, experts owned in contiguous
blocks, and the two all-to-alls (dispatch of hidden rows to the expert owners, combine of the results back at the
tokens' home rank) done by our own kernels over NVLink peer memory (`csrc/moe_ep.cu`), with the grouped tcgen05 GEMM
in between. Decode-sized steps keep replicated rows and reduce the owners' partial sums instead (`Executor._moe_ffn`).

The reference has two forms of this (`crates/fe-dsc/src/engine.rs:2409-2496`: peer copies of x and ids to the expert
cards and back; `kernels/k-fnext/src/fast.rs:1718`: ownership masks + all-reduce). `fused=False` (CPU ranks) states the
same block with process-group collectives and is what the gloo tests run.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class ExpertParallel:
    def __init__(self, tp, device, n_experts: int, hidden: int, cap_rows: int, spin_limit: int = 0):
        self.tp = tp
        self.world = tp.world if tp is not None else 1
        self.rank = tp.rank if tp is not None else 0
        self.device = torch.device(device)
        self.n_experts, self.hidden, self.cap_rows = int(n_experts), int(hidden), int(cap_rows)
        self.fused = self.device.type == "cuda" and (self.world == 1 or (tp is not None and tp.fused))
        self.calls = 0
        self._act = None
        self._plan = None
        if not self.fused:
            return
        from .._ext import load
        C = self.C = load()
        nbytes = int(C.ep_workspace_bytes(n_experts, hidden, cap_rows))
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.ws = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
            hdl = symm_mem.rendezvous(self.ws, group=tp.group.group_name)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            self._hdl = hdl
        else:
            self.ws = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            ptrs = [self.ws.data_ptr()]
        self.ws.zero_()
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(tp.group)
        self.ctr = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.status = tp.status if (tp is not None and tp.fused) else torch.zeros(1, dtype=torch.int32, device=self.device)
        sm = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.handle = C.make_ep_comm(ptrs, self.rank, n_experts, hidden, cap_rows, self.ctr, self.status, spin_limit, sm)

    def check(self) -> None:
        if self.fused and int(self.status.item()) != 0:
            raise RuntimeError(f"expert-parallel rank {self.rank}: status {int(self.status.item())} "
                               "(2 = a peer wait ran out, 5 = receive buffer capacity exceeded)")

    def moe(self, ops, h, ids, wts, w_gu, w_down, shared=None, shared_gate=None, res=None):
        """out[t] = res[t] + shared[t] * sigmoid(shared_gate[t]) + sum_k wts[t, k] * expert_{ids[t, k]}(h[t]) for this
        rank's token rows; w_gu / w_down hold the experts this rank owns."""
        self.calls += 1
        T, K = ids.shape
        inter = w_down.shape[2]
        if self.fused:
            if self._act is None or self._act.numel() < self.cap_rows * inter:
                self._act = torch.empty(self.cap_rows * inter, dtype=h.dtype, device=self.device)
            need = T * K + 3 * self.n_experts + 8
            if self._plan is None or self._plan.numel() < need:
                self._plan = torch.empty(max(need, 4096), dtype=torch.int32, device=self.device)
            out = torch.empty(T, self.hidden, dtype=h.dtype, device=self.device)
            sg = None if shared_gate is None else shared_gate.reshape(-1).float().contiguous()
            self.C.ep_moe(self.handle, out, h.contiguous(), ids.contiguous(), wts.contiguous(), w_gu, w_down, shared, sg,
                          res, self._act, self._plan)
            ops.launches += 7
            return out
        # process-group statement of the same block
        per = self.n_experts // self.world
        e_lo, e_hi = self.rank * per, (self.rank + 1) * per
        if self.world == 1:
            return ops.moe_experts(h, ids, wts, w_gu, w_down, e_lo, e_hi, shared, shared_gate, res)
        n = torch.tensor([T], dtype=torch.int64, device=h.device)
        ns = [torch.zeros_like(n) for _ in range(self.world)]
        dist.all_gather(ns, n, group=self.tp.group)
        ns = [int(v) for v in ns]
        m = max(ns)

        def gather(t):
            pad = torch.zeros(m, *t.shape[1:], dtype=t.dtype, device=t.device)
            pad[:T] = t
            outs = [torch.empty_like(pad) for _ in range(self.world)]
            dist.all_gather(outs, pad, group=self.tp.group)
            return torch.cat([o[:k] for o, k in zip(outs, ns)])
        hf, idf, wf = gather(h), gather(ids), gather(wts)
        part = ops.moe_experts(hf, idf, wf, w_gu, w_down, e_lo, e_hi, None, None, None, out_f32=True)
        dist.all_reduce(part, group=self.tp.group)
        lo = sum(ns[:self.rank])
        out = part[lo:lo + T].float()
        if shared is not None:
            g = torch.sigmoid(shared_gate.float()).reshape(-1, 1) if shared_gate is not None else 1.0
            out = out + shared.float() * g
        if res is not None:
            out = out + res.float()
        return out.to(h.dtype)
