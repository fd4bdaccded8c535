"""Summarise the scheduler's per-step trace (`FE_SCHED_PROF=1` prints `step N: dec D rows, prompt P rows, T ms` on
stderr): step count, decode / prompt rows, time per kind of step (the role of the reference's `tools/sched_steps.py`).

    FE_SCHED_PROF=1 python -m ferrite_b200.server ... 2> server.log ; python -m ferrite_b200.tools.sched_steps server.log
"""
from __future__ import annotations

import json
import re
import sys

LINE = re.compile(r"step (\d+): dec (\d+) rows, prompt (\d+) rows, ([0-9.]+) ms")


def summarise(lines):
    kinds = {"decode": [0, 0.0, 0], "prompt": [0, 0.0, 0], "mixed": [0, 0.0, 0]}
    for ln in lines:
        m = LINE.search(ln)
        if not m:
            continue
        dec, pre, ms = int(m.group(2)), int(m.group(3)), float(m.group(4))
        kind = "mixed" if dec and pre else ("decode" if dec else "prompt")
        k = kinds[kind]
        k[0] += 1
        k[1] += ms
        k[2] += dec + pre
    return {name: {"steps": v[0], "ms": round(v[1], 3), "rows": v[2], "ms_per_step": round(v[1] / v[0], 3) if v[0] else None}
            for name, v in kinds.items()}


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    with (open(argv[0]) if argv else sys.stdin) as f:
        print(json.dumps(summarise(f)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
