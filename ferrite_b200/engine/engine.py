"""Engine facade: builds the executor for a device (CUDA kernels on a GPU, PyTorch ops on CPU) and offers the
row-level calls the scheduler, the CLI and the benchmarks use.

The public surface mirrors the reference's engine API (`crates/fe-model/ENGINE_API.md`): `forward` over rows
of several slots, `prefill` in chunks cut on a fixed grid, `commit`-style slot bookkeeping, greedy `generate`.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..config import EngineConfig, ModelConfig
from ..models.weights import Weights, init_weights, shard_weights
from .executor import Executor, Segment, StepBatch


def prompt_cuts(n: int, chunk: int, align: int) -> List[int]:
    """Chunk lengths for an n-token prompt: full chunks of `chunk` rows cut on the `align` grid, and no tail of
    16 rows or fewer (it is merged into the previous chunk). Cuts depend only on n, so a resumed prompt is cut
    like a fresh one (reference `prompt_cut`, `crates/fe-model/src/sched.rs:636-719`)."""
    chunk = max(align, chunk // align * align)
    out: List[int] = []
    left = n
    while left > 0:
        take = min(chunk, left)
        if 0 < left - take <= 16:
            take = left
        out.append(take)
        left -= take
    return out


class Engine:
    def __init__(self, cfg: ModelConfig, weights: Optional[Weights] = None, ecfg: Optional[EngineConfig] = None,
                 device: Optional[str] = None, seed: int = 0, tp=None):
        self.full_cfg = cfg
        self.ecfg = ecfg or EngineConfig()
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        on_gpu = self.device.type == "cuda"
        self.dtype = torch.bfloat16 if on_gpu else torch.float32
        world = tp.world if tp is not None else 1
        rank = tp.rank if tp is not None else 0
        if weights is None:
            post = None
            if on_gpu and world == 1 and cfg.n_experts > 0 and self.ecfg.weight_dtype in ("nvfp4", "nvfp4-a16", "nvfp4-w4a4"):
                # seeded MoE weights of a 4-bit engine: every expert stack is packed as soon as it is drawn (an
                # 80B-class model is 160 GB in 16 bits and 45 GB packed)
                from ..ops.qweight import quantize_experts

                def post(name, t):
                    if name.split(".")[-1] in ("experts_gate_up", "experts_down") and t.shape[2] % 16 == 0:
                        return quantize_experts(t)
                    return t
            weights = init_weights(cfg, seed=seed, dtype=self.dtype, device=self.device, post=post)
        if world > 1:
            weights = shard_weights(cfg, weights, rank, world)
        from ..formats.packed import is_packed
        weights = {k: (v if (is_packed(v) or not isinstance(v, torch.Tensor)) else
                       v.to(self.device) if v.dtype == torch.float32 and k.endswith(("A_log", "dt_bias", "router_bias"))
                       else v.to(self.device, self.dtype)) for k, v in weights.items()}
        # linears that arrived packed from a quantised checkpoint (ModelOpt NVFP4 / FP8, EXL3) become the kernels' weight
        # objects here, after the tensor-parallel cut; on the CPU they are dequantised for the fp32 oracle
        if any(is_packed(v) for v in weights.values()):
            from ..ops.qweight import from_packed
            for k in list(weights.keys()):
                if is_packed(weights[k]):
                    weights[k] = from_packed(weights[k], self.device, self.dtype, on_gpu)
        is_t = lambda v: isinstance(v, torch.Tensor)
        if self.ecfg.weight_dtype in ("nvfp4", "nvfp4-a16", "nvfp4-w4a4"):
            from ..ops.qweight import quantize_experts, quantize_weight
            big = ("in_proj", "out_proj", "gate_up", "down", "lm_head")
            for k in list(weights.keys()):
                if not is_t(weights[k]):
                    continue
                if k.split(".")[-1] in big and weights[k].dim() == 2 and weights[k].shape[1] % 32 == 0:
                    weights[k] = quantize_weight(weights[k], "nvfp4", keep_dense=True, dense_dtype=self.dtype)
                elif k.split(".")[-1] in ("experts_gate_up", "experts_down") and weights[k].shape[2] % 16 == 0:
                    # routed experts: 4-bit only (no dense copy: they are most of an MoE model's bytes); decode rows
                    # stream the codes, prompt-sized steps dequantise one layer's stack at a time into a shared scratch
                    weights[k] = quantize_experts(weights[k])
        elif self.ecfg.weight_dtype == "fp8-block":
            from ..ops.qweight import quantize_weight
            big = ("in_proj", "out_proj", "gate_up", "down")
            for k in list(weights.keys()):
                if is_t(weights[k]) and k.split(".")[-1] in big and weights[k].dim() == 2:
                    weights[k] = quantize_weight(weights[k], "fp8b", keep_dense=True, dense_dtype=self.dtype)
        elif self.ecfg.weight_dtype in ("exl3", "exl3-4", "exl3-3", "exl3-5"):
            # synthetic EXL3 weights of the architecture's shapes (random bit streams are valid tensors): what a
            # benchmark of the trellis kernels needs when no checkpoint is at hand
            from ..formats.exl3 import Exl3Tensor
            from ..formats.packed import PackedEXL3
            from ..ops.qweight import from_packed
            bits = int(self.ecfg.weight_dtype.split("-")[1]) if "-" in self.ecfg.weight_dtype else 4
            big = ("in_proj", "out_proj", "gate_up", "down")
            for j, k in enumerate(list(weights.keys())):
                t = weights[k]
                if is_t(t) and k.split(".")[-1] in big and t.dim() == 2 and t.shape[0] >= 128 and t.shape[1] % 128 == 0:
                    main = t.shape[0] // 128 * 128       # rows past the last 128-row block (the b | a rows) stay dense
                    p = PackedEXL3(Exl3Tensor.random(t.shape[1], main, bits, seed=seed * 1000 + j))
                    if main < t.shape[0]:
                        from ..formats.packed import PackedStack
                        p = PackedStack([p, t[main:].cpu()])
                    weights[k] = from_packed(p, self.device, self.dtype, on_gpu)
        elif self.ecfg.weight_dtype != "bf16":
            raise ValueError(f"weight_dtype {self.ecfg.weight_dtype!r}: expected bf16, nvfp4, nvfp4-a16, nvfp4-w4a4, fp8-block or exl3[-bits]")
        self.cfg = cfg.shard(world)
        if on_gpu:
            from ..ops.cuda_ops import CudaOps
            ops = CudaOps(self.device, self.dtype)
        else:
            from ..ops.torch_ops import TorchOps
            ops = TorchOps(self.device, self.dtype)
        # "nvfp4": few-row steps multiply the packed weights on the block-scaled tensor cores with the activations expanded
        #   into residual NVFP4 renderings (16-bit-activation accuracy); prompt-sized steps take the dequantised copy;
        # "nvfp4-w4a4": weights and activations in NVFP4 for every row count (prompt rows: one rendering);
        # "nvfp4-a16": NVFP4 weights against 16-bit activations on the SIMT GEMV for decode rows, dense copy for prompts
        if on_gpu:
            ops.fp4_act = self.ecfg.weight_dtype in ("nvfp4", "nvfp4-w4a4")
            ops.fp4_prompt = self.ecfg.weight_dtype == "nvfp4-w4a4"
            if world > 1:
                # a rank's shard of a projection is too small for the tensor-core kernel's fixed cost to pay: few-row
                # steps take the SIMT GEMV, whose row-parallel form has the sum over ranks fused in
                ops.fp4_terms = -1
        self.ops = ops
        self.tp = tp
        if tp is not None and tp.world > 1 and self.ecfg.seq_parallel and tp.sp_max is None:
            tp.setup_big(self.ecfg.max_step_rows, cfg.hidden)
        if on_gpu and ops.fp4_act and world == 1:
            # execution order of the NVFP4 linears, so that each few-row call can prefetch the next one's weights
            from ..ops.qweight import QWeight
            order = []
            names = [f"l{i}.{n}" for i in range(cfg.n_layers) for n in ("in_proj", "out_proj", "gate_up", "down")]
            for k in names + ["lm_head"]:
                v = weights.get(k)
                if isinstance(v, QWeight) and v.kind == "nvfp4" and v.mma_scales is not None:
                    v.pair = k.endswith("gate_up")
                    order.append(v)
            for a, b in zip(order, order[1:] + order[:1]):
                a.next = b
        self.ex = Executor(self.cfg, weights, self.ecfg, ops, tp=tp, full_cfg=cfg)
        if cfg.n_experts > 0 and ((tp is not None and tp.world > 1 and tp.sp_max is not None) or (world == 1 and on_gpu)):
            # prompt-sized MoE steps go through plan / dispatch / grouped GEMM / combine; with one rank the dispatch
            # is a local sort of the (token, expert) pairs
            from ..parallel.ep import ExpertParallel
            self.ex.ep = ExpertParallel(tp if world > 1 else None, self.device, cfg.n_experts, cfg.hidden,
                                        cap_rows=self.ecfg.max_step_rows * cfg.top_k)
        self.slot_len: List[int] = [0] * self.ecfg.n_slots
        if self.ex.heat:
            import atexit
            atexit.register(self.close)
        import os
        if os.environ.get("FB_DEBUG_BOUNDS", "0") not in ("", "0"):
            # debug mode: index tensors are checked on the host before every op (eager steps, one sync per check)
            from ..utils.boundscheck import BoundsChecker
            self.bounds = BoundsChecker(self)

    # ---- rows ------------------------------------------------------------------------------------
    def forward(self, segments: Sequence[Segment], commit: bool = True, greedy: bool = True, x_add=None):
        """One step over the segments: returns (logits [rows wanted, vocab] or None, picks, row indices). On the GPU the
        returned tensors are the output buffers of the step's CUDA graph: they are overwritten by the next step of
        the same shape, so a caller that keeps them across steps clones them."""
        out = self.ex.forward(StepBatch(list(segments), commit=commit), greedy=greedy, x_add=x_add)
        self._last_segments = list(segments)
        if commit:
            for s in segments:
                self.slot_len[s.slot] = s.pos0 + len(s.tokens)
        return out

    def commit_verified(self, keep: Sequence[int]) -> None:
        """Accept the first keep[i] rows of every segment of the last verify step (forward with commit=False)."""
        self.ex.commit_verified(keep)
        for s, k in zip(self._last_segments, keep):
            self.slot_len[s.slot] = s.pos0 + int(k)

    def commit_tree(self, paths) -> None:
        """Accept one root-to-node path per segment of the last verify step with trees (`Segment.parents`): `paths[i]`
        lists row indices inside segment i starting with 0. The slot then holds pos0 + len(path) tokens."""
        self.ex.commit_tree(paths)
        for s, path in zip(self._last_segments, paths):
            self.slot_len[s.slot] = s.pos0 + len(path)

    @property
    def taps(self):
        """Hidden rows of the tapped layers from the last forward (inputs of the block drafter)."""
        return self.ex.taps

    def check(self) -> None:
        """Raise when a kernel recorded a bounded-wait timeout or a bounds error in the status word."""
        code = self.ops.status()
        if code:
            raise RuntimeError(f"device status {code}: a kernel wait ran out or an index was out of range")

    def expert_heat(self):
        """Picks per expert and MoE layer (counted when FE_EXPERT_HEAT is set)."""
        return self.ex.expert_heat()

    def close(self) -> None:
        """End of the engine's life: write what was asked to be written (expert heat counters)."""
        self.ex.write_expert_heat()

    def reset_slot(self, slot: int) -> None:
        self.ex.reset_slot(slot)
        self.slot_len[slot] = 0

    # ---- prompts ---------------------------------------------------------------------------------
    def prefill(self, slot: int, tokens: Sequence[int], pos0: Optional[int] = None, greedy: bool = True):
        """Run a prompt (or the rest of one) through the slot in chunks; returns the output of the last chunk."""
        pos = self.slot_len[slot] if pos0 is None else pos0
        out = None
        i = 0
        for n in prompt_cuts(len(tokens), self.ecfg.prefill_chunk, self.ecfg.prompt_align):
            last = i + n == len(tokens)
            seg = Segment(slot, pos, list(tokens[i:i + n]), "last" if last else "none")
            out = self.forward([seg], commit=True, greedy=greedy)
            pos += n
            i += n
        return out

    @torch.no_grad()
    def generate(self, prompt: Sequence[int], n_new: int, slot: int = 0) -> List[int]:
        """Greedy decode of n_new tokens after the prompt."""
        self.reset_slot(slot)
        _, picks, _ = self.prefill(slot, prompt)
        tok = int(picks[0][0])
        out: List[int] = []
        for _ in range(n_new):
            out.append(tok)
            _, picks, _ = self.forward([Segment(slot, self.slot_len[slot], [tok], "last")])
            tok = int(picks[0][0])
        return out
