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
    ap.add_argument("--fused-layers", default="auto", choices=["auto", "on", "off"],
                    help="decode rows through the persistent layer kernel (auto = yes under tensor parallelism)")
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
    eng = Engine(cfg, None, EngineConfig(n_slots=1, max_ctx=args.ctx + 4 * (args.steps + args.warmup) + 64,
                                         fused_layers={"auto": None, "on": True, "off": False}[args.fused_layers]),
                 device=str(dev), seed=0, tp=tp)
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
    dl = torch.zeros(1024 * 16, dtype=torch.int64, device=dev)
    C.decode_layer_trace_set(dl)
    ms, pos = _step_ms(eng, feed, pos, args.steps, args.warmup, dev)
    out["step_ms_traced"] = ms
    C.decode_layer_trace_set(None)
    d = dl.view(1024, 16).cpu()
    d = d[d[:, 0] > 0]
    if d.shape[0] > 8:
        # phases of the persistent layer kernel (CTA 0), per kind of launch; max over ranks of the per-rank means
        d = d[torch.argsort(d[:, 0])].double()
        gap = torch.cat([d[1:, 0] - d[:-1, 11], d[:1, 0] * 0])            # launch start - end of the launch before it
        gap[gap > 2e5] = float("nan")                                      # (across steps)
        phases = {}
        for kind, first, name in ((1, True, "deltanet_layer_first_of_launch"), (1, False, "deltanet_layer_later_in_launch"),
                                  (3, True, "after_attention")):
            sel = (d[:, 12] == kind) & ((d[:, 14] == 0) == first)
            r = d[sel]
            if r.shape[0] == 0:
                continue
            cols = {}
            if kind == 1:
                cols.update({"wait_at_entry": r[:, 13] - r[:, 0], "in_proj": r[:, 1] - r[:, 13], "barrier": r[:, 2] - r[:, 1],
                             "heads": r[:, 3] - r[:, 2], "barrier_2": r[:, 4] - r[:, 3], "out_proj": r[:, 5] - r[:, 4]})
            else:
                cols.update({"wait_at_entry": r[:, 13] - r[:, 0], "out_proj": r[:, 5] - r[:, 13]})
            cols.update({"sum_over_ranks_store": r[:, 6] - r[:, 5], "barrier_3": r[:, 7] - r[:, 6], "gate_up": r[:, 8] - r[:, 7],
                         "barrier_4": r[:, 9] - r[:, 8], "down": r[:, 10] - r[:, 9], "sum_over_ranks_store_2": r[:, 11] - r[:, 10],
                         "kernel_total": r[:, 11] - r[:, 0], "gap_before_launch": gap[sel][~torch.isnan(gap[sel])]})
            means = torch.tensor([float(v.mean()) / 1e3 if v.numel() else 0.0 for v in cols.values()], device=dev)
            dist.all_reduce(means, op=dist.ReduceOp.MAX)
            phases[name] = {"launches": int(r.shape[0]), **{k: round(float(v), 2) for k, v in zip(cols, means.tolist())}}
        out["persistent_layer_kernel_us"] = phases
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
