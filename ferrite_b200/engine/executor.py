"""Model executor: weights, per-slot state and the forward pass over a batch of rows.

Mechanism half of the reference's two-layer engine API (`crates/fe-model/ENGINE_API.md`; `Engine::forward_ex`
`crates/fe-model/src/model.rs:2170`, `enqueue_layer` `:2981-3204`, the CUDA-graph cache `:2648-2684`, cache
primitives `:1846-2141`): rows in, logits out, commit, slot copy / snapshot. Policy lives in `scheduler.py`.

A row is (token, slot, position). Rows of one slot form a segment (contiguous, increasing positions): a decode
row, a chain of verify rows, or a prompt chunk. State per slot: paged KV for the attention layers (a block
table per slot), and for every Gated DeltaNet layer an fp32 recurrent state plus a 3-tap conv tail.
"""
from __future__ import annotations

import os

import contextlib
import gc
import math
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..config import EngineConfig, ModelConfig
from ..models.weights import Weights
from ..ops.qweight import QWeight


@contextlib.contextmanager
def capture(g: "torch.cuda.CUDAGraph"):
    """`torch.cuda.graph(g)` with the garbage collector out of the way. A cycle collection that happens to run while the
    stream is being captured may free CUDA graphs or memory pools of engines that went out of scope earlier, and those
    frees are calls the capture forbids: the capture is invalidated and the next launch fails with "operation failed due to
    a previous error during capture". So unreachable objects are collected before the capture starts and the collector
    stays off until it ends."""
    gc.collect()
    was_on = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(g):
            yield
    finally:
        if was_on:
            gc.enable()


@dataclass
class Segment:
    slot: int
    pos0: int
    tokens: List[int]
    want_logits: str = "last"       # "last" | "all" | "none"
    # verify tree: parent row of every row inside the segment (-1 for row 0, parents before children). A row sits at
    # position pos0 + depth, sees the committed context plus its own ancestors, and is stored at cache row pos0 + index.
    parents: Optional[List[int]] = None


@dataclass
class StepBatch:
    segments: List[Segment]
    commit: bool = True             # False: verify rows (GDN state untouched; KV rows are overwritten later)

    @property
    def n_rows(self) -> int:
        return sum(len(s.tokens) for s in self.segments)

    @property
    def tree(self) -> bool:
        return any(s.parents is not None for s in self.segments)


TREE_MAX_ROWS = 32       # rows of one verify tree (reference TREE_ROWS 32); the ancestor mask has 64 bits


def tree_layout(parents: Sequence[int]):
    """Depth, ancestor-or-self bit mask, and state load/store flags of every row of a verify tree (reference
    `ancestors` / `tree_steps`, `crates/fe-model/src/model.rs:210-256`). Flag bit 0: the row's parent is not the row
    before it (its recurrent state must be reloaded); bit 1: a later row that does not directly follow branches from
    this row (its state must be parked)."""
    n = len(parents)
    assert 0 < n <= TREE_MAX_ROWS, f"a verify tree holds 1..{TREE_MAX_ROWS} rows"
    depth, mask, flags = [0] * n, [0] * n, [0] * n
    for r, p in enumerate(parents):
        assert (p == -1 and r == 0) or (0 <= p < r), "parents come before their children; row 0 is the root"
        depth[r] = 0 if p < 0 else depth[p] + 1
        mask[r] = (1 << r) | (0 if p < 0 else mask[p])
        if p != r - 1:
            flags[r] |= 1
            if p >= 0:
                flags[p] |= 2
    return depth, mask, flags


class BlockPool:
    """Free list of KV pages shared by all slots (and by parked sequences)."""

    def __init__(self, n_blocks: int):
        self.free: List[int] = list(range(n_blocks - 1, -1, -1))
        self.n_blocks = n_blocks

    def alloc(self) -> int:
        if not self.free:
            raise MemoryError("KV block pool exhausted")
        return self.free.pop()

    def release(self, blocks: Sequence[int]) -> None:
        self.free.extend(int(b) for b in blocks if b >= 0)

    @property
    def n_free(self) -> int:
        return len(self.free)


FLASH_MIN_ROWS = 32      # segments longer than this go to the flash prefill kernel (reference FLASH_MIN 17)
GDN_STEP_MAX_ROWS = 32    # decode / verify rows per segment handled by the fused conv + recurrence + norm kernel
GDN_CHUNK_MIN_ROWS = 24  # segments this long go through the chunked GDN scan instead of the row-by-row recurrence


def _bucket(n: int) -> int:
    """Row-count buckets for graph keys: exact up to 8, then powers of two."""
    if n <= 8:
        return n
    return 1 << (n - 1).bit_length()


class Executor:
    def __init__(self, cfg: ModelConfig, weights: Weights, ecfg: EngineConfig, ops, tp=None, full_cfg: Optional[ModelConfig] = None):
        self.cfg = cfg                       # per-rank shapes
        self.full_cfg = full_cfg or cfg
        self.w = weights
        self.ecfg = ecfg
        self.ops = ops
        self.tp = tp
        self.device = ops.device
        self.dtype = ops.dtype
        c = cfg
        self.kinds = c.layer_kinds
        self.max_blocks = (ecfg.max_ctx + ecfg.kv_block - 1) // ecfg.kv_block
        n_blocks = ecfg.n_slots * self.max_blocks + (int(ecfg.park_gb * (1 << 30) / max(1, self.kv_block_bytes())) if ecfg.park_gb > 0 else 0)
        self.pool = BlockPool(n_blocks)
        dev, dt = self.device, self.dtype
        # quantised caches: byte codes + fp32 scales. "fp8": e4m3, one scale per (token, kv head); "int4" / "int6": 4- /
        # 6-bit codes with one scale per 32 elements; a trailing "h" ("int4h", "int6h", "fp8h") keeps the keys (and hands
        # out the queries) in a Walsh-Hadamard rotated basis, which spreads outlier channels before quantisation
        kd = ecfg.kv_dtype
        self.kv_hrot = kd in ("int4h", "int6h", "fp8h")
        kd = kd[:-1] if self.kv_hrot else kd
        assert kd in ("bf16", "fp8", "int4", "int6"), f"kv_dtype {ecfg.kv_dtype!r}"
        self.kv8 = kd in ("fp8", "int4", "int6")
        self.kv_bits = {"fp8": 8, "int4": 4, "int6": 6}.get(kd, 16)
        self.kv4 = kd in ("int4", "int6")                   # group scales (one per 32 elements)
        self.kv_scale: Dict[int, torch.Tensor] = {}
        self.k_cache: Dict[int, torch.Tensor] = {}
        self.v_cache: Dict[int, torch.Tensor] = {}
        self.rec_state: Dict[int, torch.Tensor] = {}
        self.conv_state: Dict[int, torch.Tensor] = {}
        for i, kind in enumerate(self.kinds):
            if kind == "attn":
                # e4m3 cache: byte codes on the GPU (the CPU oracle keeps dequantised values) + K / V scales per row
                kdt = torch.uint8 if (self.kv8 and dev.type == "cuda") else dt
                # int4 on the GPU: two codes per byte, one scale per 32 elements (K groups then V groups)
                hd_store = c.head_dim * self.kv_bits // 8 if (self.kv4 and dev.type == "cuda") else c.head_dim
                self.k_cache[i] = torch.zeros(n_blocks, ecfg.kv_block, c.n_kv, hd_store, dtype=kdt, device=dev)
                self.v_cache[i] = torch.zeros(n_blocks, ecfg.kv_block, c.n_kv, hd_store, dtype=kdt, device=dev)
                if self.kv8:
                    ns = 2 * (c.head_dim // 32) if self.kv4 else 2
                    self.kv_scale[i] = torch.ones(n_blocks, ecfg.kv_block, c.n_kv, ns, dtype=torch.float32, device=dev)
            elif kind == "mla":
                # one latent row [kv_lora | rope] per token; the value cache slot stays empty
                self.k_cache[i] = torch.zeros(n_blocks, ecfg.kv_block, 1, c.kv_lora + c.rope_head_dim, dtype=dt, device=dev)
                self.v_cache[i] = torch.zeros(n_blocks, 0, dtype=dt, device=dev)
            elif kind == "gdn":
                self.rec_state[i] = torch.zeros(ecfg.n_slots, c.lin_v_heads, c.lin_dk, c.lin_dv, dtype=torch.float32, device=dev)
                self.conv_state[i] = torch.zeros(ecfg.n_slots, c.conv_k - 1, c.conv_dim, dtype=dt, device=dev)
        self.block_table_host = torch.full((ecfg.n_slots, self.max_blocks), -1, dtype=torch.int32)
        self.block_table = self.block_table_host.to(dev)
        self.slot_blocks: List[List[int]] = [[] for _ in range(ecfg.n_slots)]
        half = c.rotary_dim // 2
        inv = c.rope_theta ** (-torch.arange(half, dtype=torch.float64) / half)
        self.inv_freq = inv.float().to(dev)
        # MLA: per-head slices of kv_b with the key part transposed for the absorbed query, W_uk^T [nq, L, dn] and
        # W_uv [nq, dv, L] (reference: weight absorption in `crates/fe-dsc/src/engine.rs`)
        self.mla_w: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        if c.kv_lora > 0:
            dn, dvh, L = c.nope_head_dim, c.v_head_dim, c.kv_lora
            hr = c.rope_head_dim // 2
            self.inv_freq_mla = (c.rope_theta ** (-torch.arange(hr, dtype=torch.float64) / hr)).float().to(dev)
            for i, kind in enumerate(self.kinds):
                if kind == "mla":
                    kvb = self.w[f"l{i}.kv_b"].view(c.n_q, dn + dvh, L)
                    self.mla_w[i] = (kvb[:, :dn].transpose(1, 2).contiguous(), kvb[:, dn:].contiguous())
        # static step metadata (graph replays read these buffers)
        R = ecfg.max_step_rows
        S = max(ecfg.n_slots, 1) * 2
        self.meta_i32 = torch.zeros(5 * R + 4 * S, dtype=torch.int32, device=dev)
        # verify-tree metadata, fixed offsets: [ancestor masks (int64 x R) | cache row R | base R | parent R | flags R]
        self.tree_i32 = torch.zeros(6 * R, dtype=torch.int32, device=dev)
        self._tring = [torch.zeros(6 * R, dtype=torch.int32, pin_memory=(dev.type == "cuda")) for _ in range(4)]
        # pinned staging ring: a buffer is rewritten only after the copy that last read it has completed
        self._ring = [torch.zeros(5 * R + 4 * S, dtype=torch.int32, pin_memory=(dev.type == "cuda")) for _ in range(4)]
        self._ring_ev = [None] * 4
        self._ring_i = 0
        self.h2d_bytes = 0
        self._R, self._S = R, S
        self.graphs: "OrderedDict[tuple, tuple]" = OrderedDict()
        self.taps: List[torch.Tensor] = []
        self.last_hidden: Optional[torch.Tensor] = None
        self.commit_graphs: Dict[tuple, tuple] = {}
        self._last_graph_key = None
        self.input_rows = False          # True: forward(x_add=...) replaces the embedded rows instead of adding to them
        self.verify_proj: Dict[int, torch.Tensor] = {}
        self.reclaim = None                          # callable() -> bool: free some pages (set by the scheduler)
        self._last_meta = None
        self.profile = None
        # FE_LOG_DUMP=1: one line per layer and step on stderr with a hash of the residual stream after the layer (steps
        # run eagerly and unfused then): two builds, or two schedules of the same prompt, diverge at the first line that
        # differs (reference `FE_LOG_DUMP` layer taps, `crates/fe-model/src/model.rs`)
        self.dump_layers = os.environ.get("FE_LOG_DUMP", "0") not in ("", "0")
        # FE_EXPERT_HEAT=<file>: count how often every expert of every MoE layer is picked (device-side adds, no host
        # sync on the step path); `expert_heat()` reads them, the engine writes them to the file when it is closed.
        # What expert placement and replication decisions are made from (reference `DSC_HEAT_LOG` / `FNEXT_COUNTS`,
        # `crates/fe-dsc/src/engine.rs:2251-2315`).
        self.heat_path = os.environ.get("FE_EXPERT_HEAT", "")
        self.heat: Dict[int, torch.Tensor] = {}
        if self.heat_path and cfg.n_experts > 0:
            for i in range(cfg.n_layers):
                if cfg.is_moe(i):
                    self.heat[i] = torch.zeros((full_cfg or cfg).n_experts + 1, dtype=torch.int64, device=self.device)
        self.moe_merged: Dict[int, torch.Tensor] = {}
        self._merge_shared_experts()
        self._step_max_kvlen = None
        self._step_segments = None            # host view of an eager step's segments: (slot, pos0, rows)
        self.ep = None                        # ExpertParallel, set by the engine for MoE models under TP

    def _count_experts(self, i: int, ids) -> None:
        h = self.heat.get(i)
        if h is not None:
            flat = ids.reshape(-1).long()
            h.scatter_add_(0, flat, torch.ones_like(flat))

    def expert_heat(self) -> Dict[int, List[int]]:
        """Picks per expert and MoE layer since the engine was built (the last entry counts the shared expert when it
        rides along as a pair)."""
        return {i: h.tolist() for i, h in self.heat.items()}

    def write_expert_heat(self) -> None:
        if self.heat_path and self.heat:
            import json
            with open(self.heat_path, "w", encoding="utf-8") as f:
                json.dump({"layers": {str(i): v for i, v in self.expert_heat().items()}}, f)

    def _dump_layer(self, i: int, x, sp: bool, T: int) -> None:
        import hashlib
        import sys
        xf = (self.tp.gather_rows(x, T) if sp else x).float().cpu().contiguous()
        print(f"layer {i}: rows {xf.shape[0]} sha1 {hashlib.sha1(xf.numpy().tobytes()).hexdigest()[:12]} "
              f"mean {float(xf.mean()):.6f} absmax {float(xf.abs().max()):.4f}", file=sys.stderr)

    def _merge_shared_experts(self) -> None:
        """One GPU, one shared expert of the routed experts' width: append it to the expert stacks (entry n_experts) and
        join the router with the shared-gate row, so a decode step's MoE block is norm, one router product, route, pair
        GEMVs, combine: three launches fewer per layer than with the shared expert as separate linears. The stacks keep
        serving prompt-sized steps (which read entries 0 .. n_experts - 1); the separate shared weights stay for those."""
        c, w = self.cfg, self.w
        if (self.device.type != "cuda" or c.n_experts == 0 or c.n_shared != 1 or (self.tp is not None and self.tp.world > 1)
                or os.environ.get("FB_MOE_MERGE_SHARED", "1") == "0"):
            return
        from ..formats import nvfp4
        from ..ops.qweight import ExpertsFP4
        for i in range(c.n_layers):
            p = f"l{i}."
            if not c.is_moe(i) or p + "shared_gate_up" not in w:
                continue
            sg, sd = w[p + "shared_gate_up"], w[p + "shared_down"]
            sg, sd = getattr(sg, "dense", sg), getattr(sd, "dense", sd)
            gu, dn = w[p + "experts_gate_up"], w[p + "experts_down"]
            if not isinstance(sg, torch.Tensor) or tuple(sg.shape) != tuple(gu.shape[1:]) or tuple(sd.shape) != tuple(dn.shape[1:]):
                continue
            if isinstance(gu, ExpertsFP4):
                # the stack's one tensor scale must cover the shared expert too (else its large values would clip)
                if float(sg.abs().max()) > gu.global_scale * 6 * 448 or float(sd.abs().max()) > dn.global_scale * 6 * 448:
                    continue
                for key, stack, extra in ((p + "experts_gate_up", gu, sg), (p + "experts_down", dn, sd)):
                    q = nvfp4.quantize(extra.float(), global_scale=stack.global_scale)
                    w[key] = ExpertsFP4(torch.cat([stack.packed, q.packed[None].to(stack.packed.device)]),
                                        torch.cat([stack.scales, q.scales.view(torch.uint8)[None].to(stack.scales.device)]),
                                        stack.global_scale)
            elif isinstance(gu, torch.Tensor):
                w[p + "experts_gate_up"] = torch.cat([gu, sg[None].to(gu.dtype)])
                w[p + "experts_down"] = torch.cat([dn, sd[None].to(dn.dtype)])
            else:
                continue
            router = w[p + "router"]
            gate = w.get(p + "shared_gate") if c.router == "softmax" else None
            self.moe_merged[i] = torch.cat([router, gate.to(router.dtype)]).contiguous() if gate is not None else router

    # ---- sizes -----------------------------------------------------------------------------------
    def kv_block_bytes(self) -> int:
        c, e = self.cfg, self.ecfg
        kd = e.kv_dtype[:-1] if e.kv_dtype.endswith("h") else e.kv_dtype
        per = 2 * e.kv_block * c.n_kv * c.head_dim * (1 if kd == "fp8" else 2)
        if kd in ("int4", "int6"):
            per = 2 * e.kv_block * c.n_kv * (c.head_dim * int(kd[3]) // 8 + c.head_dim // 32 * 4)
        if c.kv_lora > 0:
            per = e.kv_block * (c.kv_lora + c.rope_head_dim) * 2
        return per * max(1, self.cfg.n_attn)

    # ---- block tables -----------------------------------------------------------------------------
    def ensure_capacity(self, slot: int, n_tokens: int) -> None:
        need = (n_tokens + self.ecfg.kv_block - 1) // self.ecfg.kv_block
        if need > self.max_blocks:
            raise ValueError(f"sequence of {n_tokens} tokens exceeds max_ctx {self.ecfg.max_ctx}")
        blocks = self.slot_blocks[slot]
        changed = False
        while len(blocks) < need:
            while self.pool.n_free == 0 and self.reclaim is not None and self.reclaim():
                pass                                  # the scheduler evicts parked sequences to free pages
            b = self.pool.alloc()
            self.block_table_host[slot, len(blocks)] = b
            blocks.append(b)
            changed = True
        if changed:
            self.block_table.copy_(self.block_table_host, non_blocking=True)

    def reset_slot(self, slot: int) -> None:
        """Free the slot's pages and zero its recurrent state (reference `reset_slot` `model.rs:2141`)."""
        self.pool.release(self.slot_blocks[slot])
        self.slot_blocks[slot] = []
        self.block_table_host[slot].fill_(-1)
        self.block_table.copy_(self.block_table_host, non_blocking=True)
        for t in self.rec_state.values():
            t[slot].zero_()
        for t in self.conv_state.values():
            t[slot].zero_()

    # ---- snapshots (prompt-cache primitives) ---------------------------------------------------------
    def state_save(self, slot: int) -> Dict[str, torch.Tensor]:
        """Copy of the GDN recurrent + conv state of a slot (a `Snap`, reference `pcache.rs`); KV stays in place."""
        return {
            "rec": torch.stack([t[slot] for t in self.rec_state.values()]).clone() if self.rec_state else torch.empty(0),
            "conv": torch.stack([t[slot] for t in self.conv_state.values()]).clone() if self.conv_state else torch.empty(0),
        }

    def state_restore(self, slot: int, snap: Dict[str, torch.Tensor]) -> None:
        for j, t in enumerate(self.rec_state.values()):
            t[slot].copy_(snap["rec"][j])
        for j, t in enumerate(self.conv_state.values()):
            t[slot].copy_(snap["conv"][j])

    def detach_blocks(self, slot: int, n_tokens: int) -> List[int]:
        """Hand the slot's first pages (covering n_tokens) to the caller (parking is a table move, no copy)."""
        need = (n_tokens + self.ecfg.kv_block - 1) // self.ecfg.kv_block
        blocks = self.slot_blocks[slot]
        keep, extra = blocks[:need], blocks[need:]
        self.pool.release(extra)
        self.slot_blocks[slot] = []
        self.block_table_host[slot].fill_(-1)
        self.block_table.copy_(self.block_table_host, non_blocking=True)
        return keep

    def attach_blocks(self, slot: int, blocks: List[int]) -> None:
        assert not self.slot_blocks[slot]
        self.slot_blocks[slot] = list(blocks)
        for j, b in enumerate(blocks):
            self.block_table_host[slot, j] = b
        self.block_table.copy_(self.block_table_host, non_blocking=True)

    def copy_blocks(self, src_blocks: Sequence[int], dst_blocks: Sequence[int]) -> None:
        """Copy KV pages (every attention layer) from one page list to another (shared-prefix restore, slot fork;
        reference `kv_blocks_copy`, `crates/fe-model/src/model.rs:1846-2138`)."""
        if not len(src_blocks):
            return
        s = torch.tensor(list(src_blocks), device=self.device, dtype=torch.long)
        d = torch.tensor(list(dst_blocks), device=self.device, dtype=torch.long)
        for i in self.k_cache:
            self.k_cache[i][d] = self.k_cache[i][s]
            self.v_cache[i][d] = self.v_cache[i][s]
            if i in self.kv_scale:
                self.kv_scale[i][d] = self.kv_scale[i][s]

    def copy_slot(self, src: int, dst: int, n_tokens: int) -> None:
        """Fork: copy KV pages covering n_tokens and the GDN state from one slot to another
        (reference `copy_slot` `model.rs:2121`)."""
        self.reset_slot(dst)
        self.ensure_capacity(dst, n_tokens)
        nb = (n_tokens + self.ecfg.kv_block - 1) // self.ecfg.kv_block
        if nb:
            s = torch.tensor(self.slot_blocks[src][:nb], device=self.device, dtype=torch.long)
            d = torch.tensor(self.slot_blocks[dst][:nb], device=self.device, dtype=torch.long)
            for i in self.k_cache:
                self.k_cache[i][d] = self.k_cache[i][s]
                self.v_cache[i][d] = self.v_cache[i][s]
                if i in self.kv_scale:
                    self.kv_scale[i][d] = self.kv_scale[i][s]
        for t in self.rec_state.values():
            t[dst].copy_(t[src])
        for t in self.conv_state.values():
            t[dst].copy_(t[src])

    # ---- metadata upload ----------------------------------------------------------------------------
    def _upload(self, batch: StepBatch):
        """Fill the pinned metadata buffer for this step and copy its used prefix to the device. Layout (int32):
        [tok T | slot T | pos T | kvlen T | lrow T | seg_slot S | seg_row0 S | seg_nrows S | seg_pos0 S]."""
        T, S = batch.n_rows, len(batch.segments)
        ri = self._ring_i
        self._ring_i = (ri + 1) % len(self._ring)
        if self._ring_ev[ri] is not None:
            self._ring_ev[ri].synchronize()
        h = self._ring[ri]
        tok, slot, pos, kvl, lrow = (h[i * T:(i + 1) * T] for i in range(5))
        o = 5 * T
        sslot, srow0, snrows, spos0 = (h[o + i * S:o + (i + 1) * S] for i in range(4))
        r = 0
        logit_rows: List[int] = []
        tree = batch.tree
        if tree:
            R = self._R
            th = self._tring[ri]
            tmask = th[:2 * R].view(torch.int64)
            tcpos, tbase, tpar, tflag = (th[(2 + i) * R:(3 + i) * R] for i in range(4))
        from .._ext import host
        hn = host()
        if hn is not None:
            # the whole block is written by one C++ call (`csrc/host_runtime.cpp`); the loop below states the same layout
            for sg in batch.segments:
                self.ensure_capacity(sg.slot, sg.pos0 + len(sg.tokens))
            segs = batch.segments
            logit_rows = list(hn.fill_step_meta(
                h, [[int(t) for t in sg.tokens] for sg in segs], [int(sg.slot) for sg in segs], [int(sg.pos0) for sg in segs],
                [2 if sg.want_logits == "all" else 1 if sg.want_logits == "last" else 0 for sg in segs],
                th if tree else None, self._R,
                [([int(x) for x in sg.parents] if sg.parents is not None else []) for sg in segs] if tree else []))
        for si, sg in enumerate(batch.segments if hn is None else ()):
            n = len(sg.tokens)
            self.ensure_capacity(sg.slot, sg.pos0 + n)
            tok[r:r + n] = torch.tensor(sg.tokens, dtype=torch.int32)
            slot[r:r + n] = sg.slot
            pos[r:r + n] = torch.arange(sg.pos0, sg.pos0 + n, dtype=torch.int32)
            kvl[r:r + n] = torch.arange(sg.pos0 + 1, sg.pos0 + n + 1, dtype=torch.int32)
            if tree:
                par = list(sg.parents) if sg.parents is not None else list(range(-1, n - 1))
                assert len(par) == n
                depth, mask, flags = tree_layout(par)
                pos[r:r + n] = torch.tensor([sg.pos0 + d for d in depth], dtype=torch.int32)
                tmask[r:r + n] = torch.tensor(mask, dtype=torch.int64)
                tcpos[r:r + n] = torch.arange(sg.pos0, sg.pos0 + n, dtype=torch.int32)
                tbase[r:r + n] = sg.pos0
                tpar[r:r + n] = torch.tensor(par, dtype=torch.int32)
                tflag[r:r + n] = torch.tensor(flags, dtype=torch.int32)
            sslot[si], srow0[si], snrows[si], spos0[si] = sg.slot, r, n, sg.pos0
            if sg.want_logits == "all":
                logit_rows.extend(range(r, r + n))
            elif sg.want_logits == "last":
                logit_rows.append(r + n - 1)
            r += n
        nl = len(logit_rows)
        if hn is None:
            lrow[:nl] = torch.tensor(logit_rows, dtype=torch.int32) if nl else lrow[:0]
        used = 5 * T + 4 * S
        self.meta_i32[:used].copy_(h[:used], non_blocking=True)
        if tree:
            self.tree_i32.copy_(th, non_blocking=True)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self._ring_ev[ri] = ev
        self.h2d_bytes = used * 4
        return logit_rows

    def _meta_views(self, T: int, nseg: int, nlog: int):
        m = self.meta_i32
        o = 5 * T
        S = nseg
        return dict(
            tok=m[0:T], slot=m[T:2 * T], pos=m[2 * T:3 * T], kvlen=m[3 * T:4 * T], lrow=m[4 * T:4 * T + nlog],
            sslot=m[o:o + S], srow0=m[o + S:o + 2 * S], snrows=m[o + 2 * S:o + 3 * S], spos0=m[o + 3 * S:o + 4 * S],
        )

    def _tree_views(self, T: int):
        m, R = self.tree_i32, self._R
        return dict(mask=m[:2 * R].view(torch.int64)[:T], cpos=m[2 * R:2 * R + T], base=m[3 * R:3 * R + T],
                    parent=m[4 * R:4 * R + T], flags=m[5 * R:5 * R + T])

    # ---- forward -----------------------------------------------------------------------------------
    def _row_parallel(self, x_in, w, res):
        """Row-parallel projection (o_proj / out_proj / down): partial product, reduction over TP ranks, residual."""
        if self.tp is None or self.tp.world == 1:
            return self.ops.linear(x_in, w, res=res)
        return self.tp.linear_allreduce(self.ops, x_in, w, res)

    def _moe_ffn_sp(self, x, i, col, row):
        """MoE block on a row shard of the tokens (prompt path under tensor/expert parallelism): route the local
        tokens, run the column-sharded shared expert through the gather/reduce-scatter GEMMs, and send the routed
        pairs through the expert-parallel dispatch -> grouped GEMM -> combine kernels."""
        c, w, ops = self.cfg, self.w, self.ops
        p = f"l{i}."
        h, _ = ops.rmsnorm(x, w[p + "post_norm"], c.eps, True)
        # router logits in fp32 for every row count: bf16 logits would reorder near-tied experts between the prompt
        # and the decode path
        logits = ops.linear(h, w[p + "router"], out_f32=True)
        ids, wts = ops.moe_route(logits.contiguous(), w.get(p + "router_bias"), 0 if c.router == "softmax" else 1, c.top_k,
                                 c.n_groups, c.topk_groups, c.route_scale)
        self._count_experts(i, ids)
        shared = sgate = None
        if c.n_shared:
            shared = row(col(x, w[p + "shared_gate_up"], w[p + "post_norm"], swiglu=True), w[p + "shared_down"], None)
            if c.router == "softmax":
                sgate = ops.linear(h, w[p + "shared_gate"], out_f32=True)
        return self.ep.moe(ops, h, ids, wts, ops.experts_dense(w[p + "experts_gate_up"], 0),
                           ops.experts_dense(w[p + "experts_down"], 1), shared, sgate, x)

    def _moe_ffn(self, x, i):
        """Routed experts + shared expert. Under expert parallelism a rank computes the pairs of the experts it owns
        (and its column slice of the shared expert); the partial sums are reduced over ranks with the residual."""
        c, w, ops = self.cfg, self.w, self.ops
        p = f"l{i}."
        h, _ = ops.rmsnorm(x, w[p + "post_norm"], c.eps, True)
        merged = self.moe_merged.get(i)
        if merged is not None and h.shape[0] <= getattr(ops, "moe_pair_rows", 0):
            # few rows on one GPU: the shared expert is entry n_experts of the expert stacks and rides along as one more
            # (token, expert) pair, weighted by the sigmoid of the last column of the merged router | shared-gate product
            n_exp = self.full_cfg.n_experts
            logits = ops.linear(h, merged, out_f32=True)
            ids, wts = ops.moe_route(logits, w.get(p + "router_bias"), 0 if c.router == "softmax" else 1, c.top_k,
                                     c.n_groups, c.topk_groups, c.route_scale, n_exp=n_exp,
                                     shared_col=n_exp if merged.shape[0] > n_exp else -1, shared_id=n_exp)
            self._count_experts(i, ids)
            return ops.moe_experts(h, ids, wts, w[p + "experts_gate_up"], w[p + "experts_down"], 0, n_exp + 1, None, None, x)
        logits = ops.linear(h, w[p + "router"], out_f32=True)
        ids, wts = ops.moe_route(logits.contiguous(), w.get(p + "router_bias"), 0 if c.router == "softmax" else 1, c.top_k,
                                 c.n_groups, c.topk_groups, c.route_scale)
        self._count_experts(i, ids)
        shared = sgate = None
        if c.n_shared:
            shared = ops.linear(ops.linear(h, w[p + "shared_gate_up"], swiglu=True), w[p + "shared_down"])
            if c.router == "softmax":
                sgate = ops.linear(h, w[p + "shared_gate"], out_f32=True)
        world = self.tp.world if self.tp is not None else 1
        rank = self.tp.rank if self.tp is not None else 0
        n_exp = self.full_cfg.n_experts
        per = n_exp // world
        e_lo, e_hi = rank * per, (rank + 1) * per
        if world == 1:
            if self.ep is not None and h.shape[0] > getattr(ops, "moe_pair_rows", 1 << 30):
                return self.ep.moe(ops, h, ids, wts, ops.experts_dense(w[p + "experts_gate_up"], 0),
                                   ops.experts_dense(w[p + "experts_down"], 1), shared, sgate, x)
            return ops.moe_experts(h, ids, wts, w[p + "experts_gate_up"], w[p + "experts_down"], e_lo, e_hi, shared, sgate, x)
        part = ops.moe_experts(h, ids, wts, w[p + "experts_gate_up"], w[p + "experts_down"], e_lo, e_hi, shared, sgate, None)
        return self.tp.allreduce_rows(ops, part, x)

    def _layers(self, x, mv, T, nseg, max_seg_rows, nsplit, commit, tv=None):
        c, w, ops = self.cfg, self.w, self.ops
        eps = c.eps
        self.taps = []
        # Sequence-parallel prompt path under tensor parallelism: the residual stream is sharded by rows between
        # blocks; column-parallel projections gather the rows (all-gather fused into the GEMM), row-parallel ones
        # reduce-scatter them (fused into the GEMM epilogue). Decode-sized steps keep replicated rows.
        sp = (self.tp is not None and self.tp.sp_ready(T) and (c.n_experts == 0 or self.ep is not None)
              and c.kv_lora == 0 and isinstance(w["l0.in_proj"], torch.Tensor))       # packed weights keep replicated rows
        if sp:
            lo, hi = self.tp.shard_rows(T)
            x = x[lo:hi].contiguous()

            def col(xs, wt, norm_w, swiglu=False):
                return self.tp.ag_linear(ops, xs, wt, norm_w, eps, T, swiglu)

            def row(act, wt, xs):
                return self.tp.rs_linear(ops, act, wt, xs, T)
        else:
            def col(xs, wt, norm_w, swiglu=False):
                return ops.linear(xs, wt, norm_w=norm_w, eps=eps, swiglu=swiglu)

            row = self._row_parallel
        # plain decode rows (one per sequence): the layer, or what follows its attention, as one persistent kernel
        fuse = self.ecfg.fused_layers
        if fuse is None:
            fuse = self.tp is not None and self.tp.world > 1
        fuse = (fuse and not self.dump_layers and ops.name == "cuda" and commit and tv is None and not sp and max_seg_rows == 1 and nseg == T and T <= 4
                and c.n_experts == 0 and c.kv_lora == 0 and isinstance(w["l0.out_proj"], torch.Tensor)
                and w["l0.out_proj"].dtype == torch.bfloat16 and (self.tp is None or self.tp.world == 1 or self.tp.fused))
        comm = self.tp.comm if (fuse and self.tp is not None and self.tp.world > 1) else None
        gdn_fusable = fuse and c.lin_dk == c.lin_dv and c.lin_dk in (64, 128) and c.lin_v_heads * T <= ops.sm_count
        run, run_idx = [], []                 # consecutive layers waiting to go out as one persistent launch
        run_max = ops.decode_layers_max if fuse else 0

        def flush():
            nonlocal x, run, run_idx
            if run:
                outs = ops.decode_layers(comm, x, run, mv["sslot"], (c.lin_k_heads, c.lin_v_heads, c.lin_dk), eps)
                self.taps.extend(outs[j] for j, li in enumerate(run_idx) if li in c.tap_layers)
                x, run, run_idx = outs[-1], [], []

        tail = lambda p: {"w_out": w[p + "out_proj"], "post_norm": w[p + "post_norm"], "w_gu": w[p + "gate_up"], "w_down": w[p + "down"]}
        for i, kind in enumerate(self.kinds):
            p = f"l{i}."
            if gdn_fusable and kind == "gdn":
                run.append({"w_in": w[p + "in_proj"], "input_norm": w[p + "input_norm"], "rec": self.rec_state[i],
                            "conv": self.conv_state[i], "conv_w": w[p + "conv_w"], "A_log": w[p + "A_log"],
                            "dt_bias": w[p + "dt_bias"], "gnorm_w": w[p + "gnorm_w"], **tail(p)})
                run_idx.append(i)
                if len(run) == run_max:
                    flush()
                continue
            flush()                                # everything else reads the rows
            if kind == "gdn":
                proj = col(x, w[p + "in_proj"], w[p + "input_norm"])
                if tv is not None:
                    # verify tree: conv windows and recurrent states follow the parent links; nothing is committed
                    self.verify_proj[i] = proj
                    qkv = ops.gdn_conv_tree(proj, w[p + "conv_w"], self.conv_state[i], mv["sslot"], mv["srow0"],
                                            mv["snrows"], c.conv_dim, tv["parent"])
                    y = ops.gdn_rec_tree(qkv, proj, self.rec_state[i], w[p + "A_log"], w[p + "dt_bias"], mv["sslot"],
                                         mv["srow0"], mv["snrows"], tv["parent"], tv["flags"], c.lin_k_heads,
                                         c.lin_v_heads, c.lin_dk, c.lin_dv, eps)
                    o = ops.gated_norm(y, proj, c.conv_dim, w[p + "gnorm_w"], c.lin_v_heads, c.lin_dv, eps)
                    x = row(o, w[p + "out_proj"], x)
                    if c.is_moe(i):
                        x = self._moe_ffn(x, i)
                    else:
                        x = row(col(x, w[p + "gate_up"], w[p + "post_norm"], swiglu=True), w[p + "down"], x)
                    if i in c.tap_layers:
                        self.taps.append(x)
                    if self.dump_layers:
                        self._dump_layer(i, x, False, T)
                    continue
                elif hasattr(ops, "gdn_step") and max_seg_rows <= GDN_STEP_MAX_ROWS and c.lin_dk == c.lin_dv and c.lin_dk in (64, 128):
                    if not commit:
                        self.verify_proj[i] = proj
                    o = ops.gdn_step(proj, w[p + "conv_w"], self.rec_state[i], self.conv_state[i], w[p + "A_log"],
                                     w[p + "dt_bias"], w[p + "gnorm_w"], mv["sslot"], mv["srow0"], mv["snrows"],
                                     c.lin_k_heads, c.lin_v_heads, c.lin_dk, c.lin_dv, eps, commit=commit)
                    x = row(o, w[p + "out_proj"], x)
                    if c.is_moe(i):
                        x = self._moe_ffn_sp(x, i, col, row) if sp else self._moe_ffn(x, i)
                    else:
                        act = col(x, w[p + "gate_up"], w[p + "post_norm"], swiglu=True)
                        x = row(act, w[p + "down"], x)
                    if i in c.tap_layers:
                        self.taps.append(self.tp.gather_rows(x, T) if sp else x)
                    if self.dump_layers:
                        self._dump_layer(i, x, sp, T)
                    continue
                qkv = ops.gdn_conv(proj, w[p + "conv_w"], self.conv_state[i], mv["sslot"], mv["srow0"], mv["snrows"],
                                   c.conv_dim, **({"max_rows": max_seg_rows} if ops.name == "cuda" else {}))
                if not commit:
                    self.verify_proj[i] = proj           # kept so the accepted rows can be replayed into the state
                y = ops.gdn_rec(qkv, proj, self.rec_state[i], self.conv_state[i], w[p + "A_log"], w[p + "dt_bias"],
                                mv["sslot"], mv["srow0"], mv["snrows"], c.lin_k_heads, c.lin_v_heads, c.lin_dk,
                                c.lin_dv, eps, commit=commit, chunked=commit and max_seg_rows >= GDN_CHUNK_MIN_ROWS,
                                max_rows=max_seg_rows)
                o = ops.gated_norm(y, proj, c.conv_dim, w[p + "gnorm_w"], c.lin_v_heads, c.lin_dv, eps)
                x = row(o, w[p + "out_proj"], x)
            elif kind == "mla":
                h, _ = ops.rmsnorm(x, w[p + "input_norm"], eps, True)
                qa, _ = ops.rmsnorm(ops.linear(h, w[p + "q_a"]), w[p + "q_a_norm"], eps, True)
                q = ops.linear(qa, w[p + "q_b"])
                kva = ops.linear(h, w[p + "kv_a"])
                w_uk_t, w_uv = self.mla_w[i]
                L, R = c.kv_lora, c.rope_head_dim
                # prompt segments: per-head keys / values expanded from the latent rows, tcgen05 flash kernel
                expand = (ops.name == "cuda" and max_seg_rows > FLASH_MIN_ROWS and self._step_segments is not None
                          and self.ecfg.kv_block % 64 == 0 and max(c.nope_head_dim + R, c.v_head_dim) <= 256
                          and isinstance(w[p + "kv_b"], torch.Tensor))
                qabs = ops.mla_prep(q, kva, w[p + "kv_a_norm"], w_uk_t, self.inv_freq_mla, mv["slot"], mv["pos"],
                                    self.block_table, self.k_cache[i].view(-1, self.ecfg.kv_block, L + R),
                                    self.ecfg.kv_block, c.n_q, c.nope_head_dim, L, R, eps,
                                    **({"absorb": False} if expand else {}))
                if expand:
                    o = ops.mla_attention_prefill(q, qabs, self.k_cache[i], w[p + "kv_b"], self._step_segments, mv["srow0"],
                                                  mv["snrows"], mv["spos0"], self.block_table, self.ecfg.kv_block, c.n_q,
                                                  c.nope_head_dim, c.v_head_dim, L, R)
                else:
                    ol = ops.mla_attention(qabs, self.k_cache[i].view(-1, self.ecfg.kv_block, L + R), mv["slot"], mv["kvlen"],
                                           self.block_table, self.ecfg.kv_block, c.n_q, L, R,
                                           1.0 / math.sqrt(c.nope_head_dim + R),
                                           nsplit=nsplit if max_seg_rows <= FLASH_MIN_ROWS else 1)
                    o = ops.mla_out(ol, w_uv)
                x = row(o, w[p + "out_proj"], x)
            else:
                proj = col(x, w[p + "in_proj"], w[p + "input_norm"])
                kvs = {"kv_scale": self.kv_scale[i]} if self.kv8 else {}
                q = ops.attn_prep(proj, w[p + "q_norm"], w[p + "k_norm"], self.inv_freq, mv["slot"], mv["pos"],
                                  self.block_table, self.k_cache[i], self.v_cache[i], self.ecfg.kv_block, c.n_q,
                                  c.n_kv, c.head_dim, c.rotary_dim, c.attn_gate, eps,
                                  **({"row_cpos": tv["cpos"]} if tv is not None else {}), **kvs,
                                  **({"hrot": self.kv_hrot, "kv_bits": self.kv_bits} if self.kv8 else {}))
                if tv is not None:
                    # tree rows see the committed context plus their own ancestors (bit mask over the segment's rows)
                    o = ops.attention(q, proj, self.k_cache[i], self.v_cache[i], mv["slot"], mv["kvlen"],
                                      self.block_table, self.ecfg.kv_block, c.n_q, c.n_kv, c.head_dim, c.attn_gate,
                                      row_base=tv["base"], row_mask=tv["mask"], nsplit=nsplit,
                                      segs=(mv["sslot"], mv["srow0"], mv["snrows"], max_seg_rows), **kvs)
                elif max_seg_rows > FLASH_MIN_ROWS:
                    o = ops.attention_prefill(q, proj, self.k_cache[i], self.v_cache[i], mv["sslot"], mv["srow0"],
                                              mv["snrows"], mv["spos0"], self.block_table, self.ecfg.kv_block, c.n_q,
                                              c.n_kv, c.head_dim, c.attn_gate, max_seg_rows, row_slot=mv["slot"],
                                              row_kvlen=mv["kvlen"], **kvs, **({"max_kvlen": self._step_max_kvlen} if kvs else {}))
                else:
                    o = ops.attention(q, proj, self.k_cache[i], self.v_cache[i], mv["slot"], mv["kvlen"],
                                      self.block_table, self.ecfg.kv_block, c.n_q, c.n_kv, c.head_dim, c.attn_gate,
                                      nsplit=nsplit, segs=(mv["sslot"], mv["srow0"], mv["snrows"], max_seg_rows), **kvs)
                if fuse:                             # the rest of this layer opens the next run
                    run.append({"o": o, **tail(p)})
                    run_idx.append(i)
                    continue
                x = row(o, w[p + "out_proj"], x)
            if c.is_moe(i):
                x = self._moe_ffn_sp(x, i, col, row) if sp else self._moe_ffn(x, i)
            elif not sp and (self.tp is None or self.tp.world == 1):
                x = ops.ffn(x, w[p + "gate_up"], w[p + "down"], w[p + "post_norm"], eps, x)
            else:
                act = col(x, w[p + "gate_up"], w[p + "post_norm"], swiglu=True)
                x = row(act, w[p + "down"], x)
            if i in c.tap_layers:
                self.taps.append(self.tp.gather_rows(x, T) if sp else x)
            if self.dump_layers:
                self._dump_layer(i, x, sp, T)
        flush()
        return self.tp.gather_rows(x, T) if sp else x

    def _head(self, x, mv, nlog, greedy):
        c, w, ops = self.cfg, self.w, self.ops
        if nlog == 0:
            return None, None
        rows = x[mv["lrow"].long()] if nlog != x.shape[0] else x
        head = w["embed"] if c.tie_embeddings else w["lm_head"]
        if self.tp is not None and self.tp.world > 1:
            per = (c.vocab + self.tp.world - 1) // self.tp.world
            off = self.tp.rank * per
            if c.tie_embeddings:
                head = head[off:min(c.vocab, off + per)]          # tied head: each rank takes its vocabulary rows
            logits = ops.linear(rows, head, norm_w=w["final_norm"], eps=c.eps, out_f32=True)
            return self.tp.gather_logits(ops, logits, greedy, off, c.vocab)
        logits = ops.linear(rows, head, norm_w=w["final_norm"], eps=c.eps, out_f32=True)
        if greedy:
            ids, finite = ops.argmax(logits)
            return logits, (ids, finite)
        return logits, None

    def _run(self, T, nseg, nlog, max_seg_rows, nsplit, commit, greedy, x_add=None, tree=False):
        mv = self._meta_views(T, nseg, nlog)
        self._last_meta = (mv, max_seg_rows)
        x = self.ops.embed(self.w["embed"], mv["tok"])
        if x_add is not None and self.input_rows:
            x = x_add.to(x.dtype)                            # MTP head: the caller computed the input rows itself
        elif x_add is not None:
            x = (x.float() + x_add.float()).to(x.dtype)      # drafter: target features fused into the input rows
        x = self._layers(x, mv, T, nseg, max_seg_rows, nsplit, commit, self._tree_views(T) if tree else None)
        self.last_hidden = x                                 # rows before the final norm (source of the MTP head)
        return self._head(x, mv, nlog, greedy)

    def attn_splits(self, max_kvlen: int) -> int:
        """Split count of the decode attention: one split per 64 keys (16 per warp), rounded up to a power of two,
        capped at 64 (measured at 32K keys, one decode row: 64 splits 103.7 tok/s, 128 splits 101.0, 256 splits 97.1: past 64
        the merge of the partials costs more than the extra CTAs bring). Short contexts are latency-bound, so the keys
        are spread over many CTAs."""
        if self.ecfg.attn_splits > 0:
            return self.ecfg.attn_splits
        s = max(1, (max_kvlen + 63) // 64)
        s = 1 << (s - 1).bit_length()
        return min(s, 64)

    def _replay_fused(self, max_rows: int) -> bool:
        c = self.cfg
        return (hasattr(self.ops, "gdn_step") and max_rows <= GDN_STEP_MAX_ROWS and c.lin_dk == c.lin_dv
                and c.lin_dk in (64, 128))

    def commit_verified(self, keep: Sequence[int]) -> None:
        """After a verify step (commit=False): advance the Gated DeltaNet state of every segment by its first
        keep[i] rows, replaying the saved projections (reference `commit_rows` / `fe_gdn_replay`,
        `crates/fe-model/src/model.rs:2516-2606`, `kernels/k-core/src/gdn.rs:260`). KV rows past the kept ones are
        simply overwritten by later steps."""
        mv, max_seg_rows = self._last_meta
        c, w, ops = self.cfg, self.w, self.ops
        mv["snrows"].copy_(torch.tensor(list(keep), dtype=torch.int32), non_blocking=False)
        mr = max(max(keep), 1)
        if (self._last_graph_key is not None and self.profile is None and self._replay_fused(mr)
                and any(k == "gdn" for k in self.kinds)):
            # The verify step ran as a CUDA graph, so the projections it saved sit in that graph's buffers: the replay
            # (one fused launch per GDN layer, the kept counts are device data) is captured once per forward graph and
            # replayed with it. Eager verify steps allocate fresh projections every time and replay eagerly.
            key = self._last_graph_key
            g = self.commit_graphs.get(key)
            if g is None:
                g = torch.cuda.CUDAGraph()
                l0 = self.ops.launches
                with capture(g):
                    self._replay_layers(mv, mr)
                self.commit_graphs[key] = (g, self.ops.launches - l0)
                self.ops.launches = l0
                g = self.commit_graphs[key]
            g[0].replay()
            self.ops.launches += g[1]
            return
        self._replay_layers(mv, mr)

    def _replay_layers(self, mv, mr: int) -> None:
        c, w, ops = self.cfg, self.w, self.ops
        for i, kind in enumerate(self.kinds):
            if kind != "gdn":
                continue
            p = f"l{i}."
            proj = self.verify_proj[i]
            if self._replay_fused(mr):
                # one launch per layer: the fused step kernel re-runs the kept rows and commits (its outputs are dropped)
                ops.gdn_step(proj, w[p + "conv_w"], self.rec_state[i], self.conv_state[i], w[p + "A_log"],
                             w[p + "dt_bias"], w[p + "gnorm_w"], mv["sslot"], mv["srow0"], mv["snrows"],
                             c.lin_k_heads, c.lin_v_heads, c.lin_dk, c.lin_dv, c.eps, commit=True)
                continue
            qkv = ops.gdn_conv(proj, w[p + "conv_w"], self.conv_state[i], mv["sslot"], mv["srow0"], mv["snrows"],
                               c.conv_dim, **({"max_rows": mr} if ops.name == "cuda" else {}))
            ops.gdn_rec(qkv, proj, self.rec_state[i], self.conv_state[i], w[p + "A_log"], w[p + "dt_bias"],
                        mv["sslot"], mv["srow0"], mv["snrows"], c.lin_k_heads, c.lin_v_heads, c.lin_dk, c.lin_dv,
                        c.eps, commit=True, chunked=False)

    def commit_tree(self, paths: Sequence[Sequence[int]]) -> None:
        """After a verify step with trees (commit=False): keep, for every segment, the rows of `paths[i]` (row indices
        inside the segment from the root down, `paths[i][0] == 0`; empty keeps nothing). The Gated DeltaNet state is
        advanced by replaying the saved projections of the path rows in order, and the path's K/V rows are moved from
        the cache rows they were stored at (pos0 + row index) to consecutive positions (pos0 + depth). Reference
        `commit_tree` (`crates/fe-model/src/model.rs:2516-2606`: keep the accepted path, replay GDN, compact KV)."""
        batch = self._last_batch
        c, w, ops = self.cfg, self.w, self.ops
        dev = self.device
        rows, row0s, ns, slots = [], [], [], []
        src, dst, seg_off = [], [], [0]
        kvb = self.ecfg.kv_block
        r0 = 0
        for sg, path in zip(batch.segments, paths):
            path = [int(r) for r in path]
            assert not path or path[0] == 0
            row0s.append(len(rows)); ns.append(len(path)); slots.append(sg.slot)
            rows.extend(r0 + r for r in path)
            blocks = self.slot_blocks[sg.slot]
            for j, r in enumerate(path):
                if r != j:
                    a, b = sg.pos0 + r, sg.pos0 + j
                    src.append(blocks[a // kvb] * kvb + a % kvb)
                    dst.append(blocks[b // kvb] * kvb + b % kvb)
            seg_off.append(len(src))
            r0 += len(sg.tokens)
        if rows and any(k == "gdn" for k in self.kinds):
            idx = torch.tensor(rows, dtype=torch.long, device=dev)
            sslot = torch.tensor(slots, dtype=torch.int32, device=dev)
            srow0 = torch.tensor(row0s, dtype=torch.int32, device=dev)
            snrows = torch.tensor(ns, dtype=torch.int32, device=dev)
            mr = max(max(ns), 1)
            for i, kind in enumerate(self.kinds):
                if kind != "gdn":
                    continue
                p = f"l{i}."
                proj = self.verify_proj[i].index_select(0, idx).contiguous()
                if self._replay_fused(mr):
                    ops.gdn_step(proj, w[p + "conv_w"], self.rec_state[i], self.conv_state[i], w[p + "A_log"],
                                 w[p + "dt_bias"], w[p + "gnorm_w"], sslot, srow0, snrows, c.lin_k_heads, c.lin_v_heads,
                                 c.lin_dk, c.lin_dv, c.eps, commit=True)
                    continue
                qkv = ops.gdn_conv(proj, w[p + "conv_w"], self.conv_state[i], sslot, srow0, snrows, c.conv_dim,
                                   **({"max_rows": mr} if ops.name == "cuda" else {}))
                ops.gdn_rec(qkv, proj, self.rec_state[i], self.conv_state[i], w[p + "A_log"], w[p + "dt_bias"], sslot,
                            srow0, snrows, c.lin_k_heads, c.lin_v_heads, c.lin_dk, c.lin_dv, c.eps, commit=True,
                            chunked=False)
        if src and ops.name == "cuda":
            # one launch per layer moves the path's K, V and scale rows; a thread walks a segment's moves root first
            idx = torch.tensor([src, dst], dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
            off = torch.tensor(seg_off, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
            for i in self.k_cache:
                vc = self.v_cache.get(i)
                ops.kv_move_rows(self.k_cache[i], vc, self.kv_scale.get(i), idx[0], idx[1], off)
        elif src:
            s_i = torch.tensor(src, dtype=torch.long, device=dev)
            d_i = torch.tensor(dst, dtype=torch.long, device=dev)
            for i in self.k_cache:
                for cache in (self.k_cache[i], self.v_cache[i]) + ((self.kv_scale[i],) if i in self.kv_scale else ()):
                    if cache.numel() == 0:
                        continue
                    flat = cache.view(cache.shape[0] * cache.shape[1], *cache.shape[2:])
                    flat[d_i] = flat[s_i]            # the gather is materialised first, so overlapping moves are safe

    def forward(self, batch: StepBatch, greedy: bool = True, x_add=None):
        """Run one step. Returns (logits [n_logit_rows, vocab] fp32, (ids, finite) when greedy, logit_rows)."""
        T = batch.n_rows
        assert 0 < T <= self._R, f"{T} rows exceed max_step_rows"
        nseg = len(batch.segments)
        max_seg_rows = max(len(s.tokens) for s in batch.segments)
        max_kvlen = max(s.pos0 + len(s.tokens) for s in batch.segments)
        nsplit = self.attn_splits(max_kvlen) if max_seg_rows <= FLASH_MIN_ROWS else 1
        use_graph = (self.ecfg.use_graphs and self.device.type == "cuda" and T <= self.ecfg.decode_rows_max
                     and self.profile is None and x_add is None and not self.dump_layers)
        tree = batch.tree
        if tree:
            assert not batch.commit and max_seg_rows <= TREE_MAX_ROWS and "mla" not in self.kinds, \
                "verify trees: commit=False, at most TREE_MAX_ROWS rows per segment, attention / GDN layers"
            assert self.tp is None or self.tp.world == 1 or not self.tp.sp_ready(T)
        logit_rows = self._upload(batch)
        nlog = len(logit_rows)
        self._last_batch = batch
        # the e4m3 cache decode before prompt attention sizes its grid by the longest visible context, except inside
        # graphs, whose launches must not depend on the step
        self._step_max_kvlen = None if use_graph else max_kvlen
        self._step_segments = None if use_graph else [(s.slot, s.pos0, len(s.tokens)) for s in batch.segments]
        self._last_graph_key = None
        if not use_graph:
            logits, picks = self._run(T, nseg, nlog, max_seg_rows, nsplit, batch.commit, greedy, x_add, tree)
            return logits, picks, logit_rows
        key = (T, nseg, nlog, max_seg_rows, nsplit, batch.commit, greedy, tree)
        hit = self.graphs.get(key)
        if hit is None:
            # warm up eagerly once (lazy module / attribute setup), then capture
            self._run(T, nseg, nlog, max_seg_rows, nsplit, False, greedy, None, tree)
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            l0 = self.ops.launches
            with capture(g):
                out = self._run(T, nseg, nlog, max_seg_rows, nsplit, batch.commit, greedy, None, tree)
            n_kernels = self.ops.launches - l0
            self.ops.launches = l0
            hit = (g, out, n_kernels, self.taps, self.last_hidden, dict(self.verify_proj))
            self.graphs[key] = hit
            if len(self.graphs) > self.ecfg.graph_max:
                old_key, _ = self.graphs.popitem(last=False)
                self.commit_graphs.pop(old_key, None)
            # capture does not execute: replay below performs the step
        else:
            self.graphs.move_to_end(key)
        # taps / hidden / saved projections: this graph's buffers, not those of whichever graph was captured last
        g, (logits, picks), n_kernels, self.taps, self.last_hidden, vp = hit
        self.verify_proj = dict(vp)
        self._last_graph_key = key
        self._last_meta = (self._meta_views(T, nseg, nlog), max_seg_rows)
        g.replay()
        self.ops.launches += n_kernels
        return logits, picks, logit_rows
