"""Counterfactual draft budgets from a scheduler trace: how many drafted tokens would have been accepted, and what rate a
stream would have run at, had every verify step been given only B draft rows.

`FE_SCHED_PROF=2` makes the scheduler print, for every verify step, the slots, the rows each request fed (1 + drafts) and
the row indices of the accepted path. Draft trees are grown best-first and chains in order, so a budget of B draft rows
is the first B of them: under budget B a step keeps the leading nodes of its accepted path whose row index is <= B.
Per slot this prints E[accepted] at each budget and, with a forward-time table (`--fwd "rows:ms,rows:ms,..."`, measured
verify step times; linear in between), the tokens/s of one stream: (accepted + 1) / (fixed + fwd(B + 1 rows)).

    FE_SCHED_PROF=2 FE_SPEC=16 python -m ferrite_b200.server ... 2> server.log
    python -m ferrite_b200.tools.sched_budget server.log --first 100 --last 2000 --fwd 2:8.9,9:9.4,17:15.1 --fixed-ms 1.5

The role of the reference's `tools/sched_budget.py`.
"""
from __future__ import annotations

import argparse
import collections
import json
import re
import sys
from typing import Dict, List, Optional, Sequence, Tuple

LINE = re.compile(r"step (\d+): dec (\d+) rows, prompt (\d+) rows, ([0-9.]+) ms \| slots (\[[^\]]*\]) rows (\[[^\]]*\]) paths (\[.*\])\s*$")
BUDGETS = (1, 2, 3, 5, 7, 9, 11, 13, 15, 23, 31)


def parse(lines) -> List[Tuple[int, float, List[int], List[int], List[List[int]]]]:
    out = []
    for ln in lines:
        m = LINE.search(ln)
        if m:
            out.append((int(m.group(1)), float(m.group(4)), json.loads(m.group(5)), json.loads(m.group(6)), json.loads(m.group(7))))
    return out


def interp(table: Sequence[Tuple[int, float]], rows: int) -> float:
    if not table:
        return 0.0
    if rows <= table[0][0]:
        return table[0][1]
    for (r0, t0), (r1, t1) in zip(table, table[1:]):
        if rows <= r1:
            return t0 + (t1 - t0) * (rows - r0) / (r1 - r0)
    return table[-1][1]


def budgets(steps, fwd: Sequence[Tuple[int, float]] = (), fixed_ms: float = 0.0, first: int = 0, last: Optional[int] = None) -> Dict:
    per: Dict[int, List[Tuple[int, List[int]]]] = collections.defaultdict(list)
    for no, _ms, slots, rows, paths in steps:
        if no < first or (last is not None and no > last):
            continue
        for s, r, p in zip(slots, rows, paths):
            per[s].append((r - 1, p))
    out = {}
    for s, seen in sorted(per.items()):
        used = max((b for b, _ in seen), default=0)
        row = {"steps": len(seen), "mean_drafted": round(sum(b for b, _ in seen) / len(seen), 2),
               "mean_accepted": round(sum(len(p) - 1 for _, p in seen) / len(seen), 3), "budgets": {}}
        for B in [b for b in BUDGETS if b <= max(used, 1)]:
            acc = sum(sum(1 for node in p[1:] if node <= B) for _, p in seen) / len(seen)
            cell = {"accepted": round(acc, 3)}
            if fwd:
                cell["tok_s"] = round(1e3 * (acc + 1) / (fixed_ms + interp(fwd, B + 1)), 1)
            row["budgets"][B] = cell
        out[s] = row
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("log", nargs="?")
    ap.add_argument("--first", type=int, default=0)
    ap.add_argument("--last", type=int, default=None)
    ap.add_argument("--fwd", default="", help='verify forward time by rows: "2:8.9,9:9.4,17:15.1" (ms)')
    ap.add_argument("--fixed-ms", type=float, default=0.0, help="per-step cost outside the forward (draft + commit + absorb)")
    a = ap.parse_args(argv)
    fwd = sorted((int(r), float(t)) for r, t in (x.split(":") for x in a.fwd.split(",") if x))
    with (open(a.log, errors="replace") if a.log else sys.stdin) as f:
        steps = parse(f)
    print(json.dumps({"verify_steps": len(steps), "slots": budgets(steps, fwd, a.fixed_ms, a.first, a.last)}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
