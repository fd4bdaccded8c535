"""Per-operation timing of engine steps: a proxy around the op set that brackets every call with CUDA events (wall
clock on the CPU) and sums the time per op name. The role of the reference's step profiles (`FE_PROF`, the per-kernel
timers of `crates/fe-model/src/selftest.rs`).

    prof = OpProfiler(engine)                 # wraps engine.ex.ops; CUDA graphs are bypassed while it is attached
    engine.forward(segments); engine.forward(segments)
    print(prof.report())                       # {"linear": {"calls": 514, "ms": 8.1}, ...}
    prof.detach()
"""
from __future__ import annotations

import time
from typing import Any, Dict

import torch


class _TimedOps:
    def __init__(self, ops, sink: Dict[str, list], on_gpu: bool):
        object.__setattr__(self, "_ops", ops)
        object.__setattr__(self, "_sink", sink)
        object.__setattr__(self, "_gpu", on_gpu)

    def __getattr__(self, name: str) -> Any:
        attr = getattr(self._ops, name)
        if not callable(attr) or name.startswith("_") or name in ("status",):
            return attr
        sink, gpu = self._sink, self._gpu

        def timed(*a, **kw):
            if gpu:
                e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
                e0.record()
                out = attr(*a, **kw)
                e1.record()
                sink.setdefault(name, []).append((e0, e1))
            else:
                t0 = time.perf_counter()
                out = attr(*a, **kw)
                sink.setdefault(name, []).append((time.perf_counter() - t0) * 1e3)
            return out
        return timed

    def __setattr__(self, name, value):
        setattr(self._ops, name, value)


class OpProfiler:
    def __init__(self, engine):
        self.engine = engine
        self.ex = engine.ex
        self.records: Dict[str, list] = {}
        self._orig = self.ex.ops
        self._gpu = self.ex.device.type == "cuda"
        self.ex.ops = _TimedOps(self._orig, self.records, self._gpu)
        self.ex.profile = self.records            # a set profile makes the executor run eagerly (no graph replay)

    def detach(self) -> None:
        self.ex.ops = self._orig
        self.ex.profile = None

    def report(self) -> Dict[str, Dict[str, float]]:
        if self._gpu:
            torch.cuda.synchronize(self.ex.device)
        out = {}
        for name, recs in self.records.items():
            ms = sum((a.elapsed_time(b) if self._gpu else 0.0) for a, b in recs) if self._gpu else sum(recs)
            out[name] = {"calls": len(recs), "ms": round(float(ms), 4)}
        return dict(sorted(out.items(), key=lambda kv: -kv[1]["ms"]))
