#!/usr/bin/env python
"""Headline benchmark: decode tok/s (1 and 4 streams) and prefill tok/s of the 27B-class dense hybrid on 1-8 B200.

    python bench.py --gpus 1 --steps 64 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

The model is BASELINE config 2 (64 layers 3:1 GDN:GQA, hidden 5120, FFN 17408, vocab 151936) with random-init
weights and synthetic uniform-random prompts. N > 1 runs tensor parallel (strong scaling: the same request
stream on more GPUs). A step is one decode step of every stream. Timed with CUDA events between barriers +
synchronizes, max over ranks. Weights (tens of GB) are streamed every step, far larger than the 126 MB L2.
One JSON line on rank 0. `--impl reference` reports that the Rust/nvptx reference cannot be built here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

BASELINE_DECODE_1 = 33.7      # tok/s, plain decode 1 stream at 2K ctx, 2x GB10 TP2 (reference TP2.md:112-116)
BASELINE_DECODE_4 = 119.1     # tok/s aggregate, 4 streams (reference TP2.md:117)
BASELINE_PREFILL_2K = 3669.0  # tok/s (reference TP2.md:114)
BASELINE_PREFILL_32K = 2880.0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.idx)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass
        sm, mx, reasons = [], 0.0, set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx = max(mx, float(r[2]))
                names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--streams", type=int, default=1)
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (the JSON line says so)")
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--no-extras", action="store_true", help="skip the 4-stream and prefill measurements")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "reference is Rust + nvptx kernels for sm_120a/121a: no cargo/rustc in the image and no "
                          "setup.py/pyproject to pip-install; no sm_100 kernel exists in it"}))
        return 0

    import torch
    import torch.distributed as dist

    from ferrite_b200.config import EngineConfig, hybrid_27b, scaled
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    tp = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        from ferrite_b200.parallel.tp import TensorParallel
        tp = TensorParallel(dist.group.WORLD, dev)
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE {world}: launch with torch.distributed.run"

    cfg = hybrid_27b()
    if args.layers:
        cfg = scaled(cfg, args.layers)
    W = max(3, args.warmup)
    K = args.steps
    n_streams_max = 4
    long_ctx = 0 if args.no_extras else 32768
    ecfg = EngineConfig(n_slots=n_streams_max, max_ctx=max(args.ctx + 2 * (K + W) + 64, long_ctx + 64), prefill_chunk=2048,
                        weight_dtype=args.dtype)
    eng = Engine(cfg, None, ecfg, device=str(dev), seed=0, tp=tp)
    gen = torch.Generator().manual_seed(1234)
    prompts = [torch.randint(0, cfg.vocab, (args.ctx,), generator=gen).tolist() for _ in range(n_streams_max)]
    feed = torch.randint(0, cfg.vocab, (n_streams_max, 4 * (K + W) + 8), generator=gen).tolist()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- prefill (timed as an extra) -------------------------------------------------------------------
    def timed_prefill(slot, prompt):
        eng.reset_slot(slot)
        barrier()
        e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
        e0.record()
        eng.prefill(slot, prompt)
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    timed_prefill(0, prompts[0][:256])            # warm the prompt kernels
    prefill_ms = timed_prefill(0, prompts[0])
    for s in range(1, n_streams_max):
        eng.prefill(s, prompts[s]) if not args.no_extras else None
    eng.check()

    def decode_run(n_streams: int, steps: int, warm: int, e2e: bool):
        """K decode steps of n_streams streams. e2e=False: tokens come from a fixed feed, no host sync inside
        the region. e2e=True: the public call per step, next tokens read back from the device every step."""
        pos = [eng.slot_len[s] for s in range(n_streams)]
        cur = [feed[s][0] for s in range(n_streams)]
        d2h = 0

        def step(i):
            nonlocal cur, d2h
            segs = [Segment(s, pos[s] + i, [cur[s] if e2e else feed[s][i]], "last") for s in range(n_streams)]
            _, picks, _ = eng.forward(segs, commit=True, greedy=True)
            if e2e:
                ids = picks[0].cpu()               # device -> host read of the step's result
                d2h = ids.numel() * ids.element_size()
                cur = ids.tolist()

        for i in range(warm):
            step(i)
        barrier()
        launches0 = eng.ops.launches
        e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
        e0.record()
        for i in range(warm, warm + steps):
            step(i)
        e1.record()
        barrier()
        ms = max_over_ranks(e0.elapsed_time(e1))
        for s in range(n_streams):
            pos[s] += warm + steps
        return ms, eng.ops.launches - launches0, eng.ex.h2d_bytes, d2h

    sampler = ClockSampler(local)
    sampler.start()
    ms1, launches, h2d, _ = decode_run(args.streams, K, W, e2e=False)
    clocks = sampler.stop()
    ms_e2e, _, h2d_e, d2h_e = decode_run(args.streams, K, W, e2e=True)
    extras = {}
    if not args.no_extras and args.streams == 1:
        ms4, _, _, _ = decode_run(4, K, W, e2e=False)
        extras["decode_4streams_tok_s"] = 4 * K / (ms4 / 1e3)
        extras["decode_4streams_vs_baseline"] = extras["decode_4streams_tok_s"] / BASELINE_DECODE_4
    if not args.no_extras and args.streams == 1:
        # speculative verification: one step scores 1 + 16 drafted rows of one stream without committing them; with k
        # accepted drafts per step the stream advances k + 1 tokens in this time
        p0 = eng.slot_len[0]
        rows = feed[0][:17]

        def verify():
            eng.forward([Segment(0, p0, rows, "all")], commit=False, greedy=True)
        for _ in range(W):
            verify()
        barrier()
        e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
        e0.record()
        for _ in range(K):
            verify()
        e1.record()
        barrier()
        vms = max_over_ranks(e0.elapsed_time(e1)) / K
        extras["verify_17rows_ms"] = vms
        extras["spec_tok_s_at_8_accepted"] = 9.0 / (vms / 1e3)
        # the same step with what follows an acceptance of 8 drafts: the GDN state replayed over the 9 kept rows
        st0 = eng.ex.state_save(0)

        def verify_commit():
            eng.forward([Segment(0, p0, rows, "all")], commit=False, greedy=True)
            eng.commit_verified([9])
            eng.slot_len[0] = p0
        for _ in range(W):
            verify_commit()
        barrier()
        e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
        e0.record()
        for _ in range(K):
            verify_commit()
        e1.record()
        barrier()
        vcms = max_over_ranks(e0.elapsed_time(e1)) / K
        eng.ex.state_restore(0, st0)
        extras["verify_commit_ms"] = vcms
        extras["spec_tok_s_at_8_accepted_with_commit"] = 9.0 / (vcms / 1e3)
    if long_ctx:
        # long-context prefill: 32K synthetic tokens through 2048-row chunks on one slot
        long_prompt = torch.randint(0, cfg.vocab, (long_ctx,), generator=gen).tolist()
        ms32 = timed_prefill(3, long_prompt)
        extras["prefill_32k_tok_s"] = long_ctx / (ms32 / 1e3)
        extras["prefill_32k_vs_baseline"] = extras["prefill_32k_tok_s"] / BASELINE_PREFILL_32K
    extras["prefill_tok_s"] = args.ctx / (prefill_ms / 1e3)
    extras["prefill_ctx"] = args.ctx
    extras["prefill_vs_baseline"] = extras["prefill_tok_s"] / BASELINE_PREFILL_2K
    eng.check()

    value = args.streams * K / (ms1 / 1e3)
    base = BASELINE_DECODE_1 if args.streams == 1 else BASELINE_DECODE_4
    out = {
        "metric": f"decode tok/s, {args.streams} stream(s), plain decode at {args.ctx} ctx, 27B hybrid",
        "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms1 / K,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": value / base, "dtype": args.dtype,
        "data": "synthetic uniform-random prompts, random-init weights N(0,0.02)",
        "config": {"model": cfg.name + (f"-{args.layers}layers-DEBUG" if args.layers else ""),
                   "global_batch": args.streams, "seq_len": args.ctx,
                   "parallelism": f"tp{world}", "params": cfg.param_count(),
                   "l2": "inputs larger than L2: every step streams all weights (>40 GB)"},
        "clocks": clocks,
        "e2e": {"value": args.streams * K / (ms_e2e / 1e3), "unit": "tok/s", "h2d_bytes_per_step": h2d_e,
                "d2h_bytes_per_step": d2h_e},
        "gpu_launches": launches,
        "extras": extras,
    }
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
