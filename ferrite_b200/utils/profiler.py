"""Per-operation timing of engine steps: a proxy around the op set that brackets every call with CUDA events (wall
clock on the CPU) and sums the time per op name. The role of the reference's step profiles (`FE_PROF`, the per-kernel
timers of `crates/fe-model/src/selftest.rs`).

    prof = OpProfiler(engine)                 # wraps engine.ex.ops; CUDA graphs are bypassed while it is attached
    engine.forward(segments); engine.forward(segments)
    print(prof.report())                       # {"linear": {"calls": 514, "ms": 8.1}, ...}
    prof.detach()

Under tensor parallelism the collective-fused calls of `parallel/tp.py` (`linear_allreduce`, `ag_linear`, `rs_linear`,
`gather_rows`, `allreduce_rows`, `gather_logits`) are bracketed too, under `tp.<name>`; the ops they call inside are
then counted twice (once under their own name), which the table says. As a program it prints the table of one prompt
step, the max over ranks of every entry:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        -m ferrite_b200.utils.profiler --rows 2048 --layers 16
"""
from __future__ import annotations

import time
from typing import Any, Dict

import torch


class _TimedOps:
    def __init__(self, ops, sink: Dict[str, list], on_gpu: bool, nvtx: bool = False):
        object.__setattr__(self, "_ops", ops)
        object.__setattr__(self, "_sink", sink)
        object.__setattr__(self, "_gpu", on_gpu)
        object.__setattr__(self, "_nvtx", nvtx and on_gpu)

    def __getattr__(self, name: str) -> Any:
        attr = getattr(self._ops, name)
        if not callable(attr) or name.startswith("_") or name in ("status",):
            return attr
        sink, gpu, nvtx = self._sink, self._gpu, self._nvtx

        def timed(*a, **kw):
            if gpu:
                e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
                if nvtx:
                    torch.cuda.nvtx.range_push(name)        # named ranges for a timeline tool attached to the process
                e0.record()
                out = attr(*a, **kw)
                e1.record()
                if nvtx:
                    torch.cuda.nvtx.range_pop()
                sink.setdefault(name, []).append((e0, e1))
            else:
                t0 = time.perf_counter()
                out = attr(*a, **kw)
                sink.setdefault(name, []).append((time.perf_counter() - t0) * 1e3)
            return out
        return timed

    def __setattr__(self, name, value):
        setattr(self._ops, name, value)


class _TimedTP(_TimedOps):
    """The same bracket around the tensor-parallel calls; entries are named `tp.<call>`."""
    _NAMES = ("linear_allreduce", "ag_linear", "rs_linear", "gather_rows", "allreduce_rows", "gather_logits")

    def __getattr__(self, name: str) -> Any:
        if name not in self._NAMES:
            return getattr(self._ops, name)
        attr = getattr(self._ops, name)
        sink, gpu = self._sink, self._gpu

        def timed(*a, **kw):
            e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
            if gpu:
                e0.record()
            t0 = time.perf_counter()
            out = attr(*a, **kw)
            if gpu:
                e1.record()
                sink.setdefault("tp." + name, []).append((e0, e1))
            else:
                sink.setdefault("tp." + name, []).append((time.perf_counter() - t0) * 1e3)
            return out
        return timed


class OpProfiler:
    def __init__(self, engine, nvtx: bool = False):
        """`nvtx`: also open an NVTX range per op call (the reference's tracing spans), for a timeline tool."""
        self.engine = engine
        self.ex = engine.ex
        self.records: Dict[str, list] = {}
        self._orig = self.ex.ops
        self._gpu = self.ex.device.type == "cuda"
        self.ex.ops = _TimedOps(self._orig, self.records, self._gpu, nvtx)
        self.ex.profile = self.records            # a set profile makes the executor run eagerly (no graph replay)
        self._orig_tp = self.ex.tp
        if self.ex.tp is not None:
            self.ex.tp = _TimedTP(self.ex.tp, self.records, self._gpu)

    def detach(self) -> None:
        self.ex.ops = self._orig
        self.ex.tp = self._orig_tp
        self.ex.profile = None

    def report(self) -> Dict[str, Dict[str, float]]:
        if self._gpu:
            torch.cuda.synchronize(self.ex.device)
        out = {}
        for name, recs in self.records.items():
            ms = sum((a.elapsed_time(b) if self._gpu else 0.0) for a, b in recs) if self._gpu else sum(recs)
            out[name] = {"calls": len(recs), "ms": round(float(ms), 4)}
        return dict(sorted(out.items(), key=lambda kv: -kv[1]["ms"]))


def main() -> int:
    import argparse
    import json
    import os

    import torch.distributed as dist

    from ..config import EngineConfig, hybrid_27b, scaled
    from ..engine.engine import Engine
    from ..engine.executor import Segment

    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    tp = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        from ..parallel.tp import TensorParallel
        tp = TensorParallel(dist.group.WORLD, dev)
    cfg = scaled(hybrid_27b(), args.layers)
    eng = Engine(cfg, None, EngineConfig(n_slots=1, max_ctx=2 * args.rows + 64, prefill_chunk=args.rows,
                                         max_step_rows=max(args.rows, 64)), device=str(dev), seed=0, tp=tp)
    toks = torch.randint(0, cfg.vocab, (args.rows,), generator=torch.Generator().manual_seed(3)).tolist()
    for _ in range(2):                                   # warm up (lazy setup, tensor maps)
        eng.reset_slot(0)
        eng.forward([Segment(0, 0, toks, "last")])
    torch.cuda.synchronize(dev)
    prof = OpProfiler(eng)
    eng.reset_slot(0)
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
    e0.record()
    eng.forward([Segment(0, 0, toks, "last")])
    e1.record()
    rep = prof.report()
    prof.detach()
    total = e0.elapsed_time(e1)
    names = sorted(rep)
    if world > 1:
        box = [None] * world
        dist.all_gather_object(box, {k: rep[k]["ms"] for k in names})
        names = sorted(set().union(*[set(b) for b in box]))
        ms = {k: max(b.get(k, 0.0) for b in box) for k in names}
        t = torch.tensor([total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total = float(t.item())
    else:
        ms = {k: rep[k]["ms"] for k in names}
    out = {"world": world, "layers": args.layers, "rows": args.rows, "step_ms": round(total, 3),
           "ops_ms_max_over_ranks": dict(sorted(((k, round(v, 3)) for k, v in ms.items()), key=lambda kv: -kv[1])),
           "calls": {k: rep[k]["calls"] for k in rep},
           "note": "eager step with events around every call; tp.* entries include the ops they call"}
    if rank == 0:
        print(json.dumps(out))
        if args.out:
            with open(args.out, "w") as f:
                f.write(json.dumps(out) + "\n")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
