"""Where the time of the fused GEMV + all-reduce goes, measured on the device.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m ferrite_b200.utils.comm_trace --layers 16 --steps 40

Runs 1-row decode steps of the 27B hybrid (a cut of `--layers` layers) under tensor parallelism inside a CUDA graph,
with CTA 0 of every `gemv_allreduce_kernel` stamping `%globaltimer` at: previous kernel done (after
`griddepcontrol.wait`), GEMV done, pair stores issued,
first peer pair seen, last peer pair seen, kernel end. Prints, per kernel shape (grid size) and as the max over ranks
of the per-rank means: the time from entry to GEMV done, the store fan-out, the wait for the first and for the last
peer, and the epilogue; then the step time with the sources polled together and polled one after the other.
Timestamps of different GPUs are not compared with each other: only differences inside one kernel are used.

The reference measures its exchange the same way from the host side only (`crates/fe-fabric/src/bin/fabric-reduce.rs`:
latency of the reduction after an exact check); device stamps are what separates launch skew between ranks (the wait
for the first peer) from the fan-out and the polls.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _step_ms(eng, feed, pos0, steps, warm, dev):
    from ..engine.executor import Segment
    for i in range(warm):
        eng.forward([Segment(0, pos0 + i, [feed[i]], "last")], commit=True, greedy=True)
    dist.barrier()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
    e0.record()
    for i in range(warm, warm + steps):
        eng.forward([Segment(0, pos0 + i, [feed[i]], "last")], commit=True, greedy=True)
    e1.record()
    dist.barrier()
    torch.cuda.synchronize(dev)
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()), pos0 + warm + steps


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--ctx", type=int, default=512)
    ap.add_argument("--out", default="")
    args = ap.parse_args()

    from .._ext import load
    from ..config import EngineConfig, hybrid_27b, scaled
    from ..engine.engine import Engine
    from ..parallel.tp import TensorParallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world > 1, "launch with torch.distributed.run on 2+ GPUs"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    C = load()
    tp = TensorParallel(dist.group.WORLD, dev)
    cfg = scaled(hybrid_27b(), args.layers)
    eng = Engine(cfg, None, EngineConfig(n_slots=1, max_ctx=args.ctx + 4 * (args.steps + args.warmup) + 64), device=str(dev),
                 seed=0, tp=tp)
    gen = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, cfg.vocab, (args.ctx,), generator=gen).tolist()
    feed = torch.randint(0, cfg.vocab, (8 * (args.steps + args.warmup),), generator=gen).tolist()
    eng.prefill(0, prompt)
    pos = eng.slot_len[0]
    out = {"world": world, "layers": args.layers}

    # 1. stamps (graphs captured with the trace buffer in their kernel arguments)
    recs, words = C.comm_trace_shape()
    trace = torch.zeros(recs * words, dtype=torch.int64, device=dev)
    C.comm_trace_set(trace)
    ms, pos = _step_ms(eng, feed, pos, args.steps, args.warmup, dev)
    out["step_ms_traced"] = ms
    t = trace.view(recs, words).cpu()
    t = t[t[:, 6] > 0]
    table = {}
    for grid in sorted(set(t[:, 7].tolist())):
        r = t[t[:, 7] == grid].double()
        cols = {"gemv_us": r[:, 1] - r[:, 0], "stores_us": r[:, 2] - r[:, 1], "first_peer_us": r[:, 3] - r[:, 2],
                "last_peer_us": r[:, 4] - r[:, 2], "epilogue_us": r[:, 5] - r[:, 4], "total_us": r[:, 5] - r[:, 0]}
        means = torch.tensor([float(v.mean()) / 1e3 for v in cols.values()], device=dev)
        mx = means.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        mn = means.clone()
        dist.all_reduce(mn, op=dist.ReduceOp.MIN)
        table[f"grid{int(grid)}"] = {"calls": int(r.shape[0]),
                                     **{k: [round(float(a), 2), round(float(b), 2)] for k, a, b in zip(cols, mn.tolist(), mx.tolist())}}
    out["stamps_min_max_over_ranks"] = table
    C.comm_trace_set(None)

    # 2. step time: sources polled together vs one after the other (fresh graphs each time)
    for name, serial in (("together", False), ("serial", True)):
        C.comm_serial_polls_set(serial)
        eng.ex.graphs.clear()
        ms, pos = _step_ms(eng, feed, pos, args.steps, args.warmup, dev)
        out[f"step_ms_polls_{name}"] = ms
    C.comm_serial_polls_set(False)
    eng.check()
    n_ar = sum(1 for _ in cfg.layer_kinds) * 2
    out["allreduces_per_step"] = n_ar
    if rank == 0:
        line = json.dumps(out)
        print(line)
        if args.out:
            with open(args.out, "w") as f:
                f.write(line + "\n")
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
