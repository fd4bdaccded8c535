"""Release gate: the checks a build has to pass before it is handed out, run against a live server, one pass or fail.

    python -m ferrite_b200.tools.release_gate --base-url http://127.0.0.1:8000 [--mock] [--min-tok-s 50] [--lanes 1,2,4]

Steps (each PASS / FAIL, exit code 1 on any failure): the conformance suite (quick tier, heavy tier with `--heavy`), the
lanes gate (every lane of an N-lane call equals the same request sent alone, greedy), a serving benchmark whose aggregate
decode rate has to reach `--min-tok-s`, and the agents workload without a failed turn. Counterpart of the reference's
`tools/release-gate.sh`, which strings the same clients together from the shell.
"""
from __future__ import annotations

import argparse
import contextlib
import io
import json
import sys
from typing import Callable, List, Tuple


def _captured(fn: Callable[[], int]) -> Tuple[int, str]:
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        try:
            rc = fn()
        except SystemExit as e:
            rc = int(e.code or 0)
        except Exception as e:  # noqa: BLE001 - a crashed step fails the gate, it does not end it
            return 1, repr(e)
    return rc, buf.getvalue()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="")
    ap.add_argument("--mock", action="store_true")
    ap.add_argument("--heavy", action="store_true")
    ap.add_argument("--lanes", default="1,2,4")
    ap.add_argument("--prefix-tokens", type=int, default=600)
    ap.add_argument("--min-tok-s", type=float, default=0.0)
    ap.add_argument("--streams", type=int, default=4)
    a = ap.parse_args(argv)
    from . import conformance, quickbench, workloads
    base = ["--base-url", a.base_url] + (["--model", a.model] if a.model else [])
    steps: List[Tuple[str, bool, str]] = []

    rc, out = _captured(lambda: conformance.main(base + (["--mock"] if a.mock else []) + ["--tier", "all" if a.heavy else "quick"]))
    fails = [l for l in out.splitlines() if l.startswith("FAIL")]
    steps.append(("conformance", rc == 0, "; ".join(fails) or out.strip().splitlines()[-1] if out.strip() else ""))

    rc, out = _captured(lambda: workloads.main(["lanes"] + base + ["--lanes", a.lanes, "--prefix-tokens", str(a.prefix_tokens),
                                                                   "--max-tokens", "48", "--runs", "1", "--gate"]))
    steps.append(("lanes gate", rc == 0, out.strip()[-300:]))

    rc, out = _captured(lambda: quickbench.main(base + ["--streams", str(a.streams), "--prompt-tokens", "64", "--max-tokens", "48"]))
    rate = 0.0
    try:
        line = json.loads(out.strip().splitlines()[-1])
        rate = float(line.get("aggregate_tok_s") or 0.0)
        ok = rc == 0 and line.get("ok") == a.streams and rate >= a.min_tok_s
    except (ValueError, IndexError):
        ok = False
    steps.append(("serving rate", ok, f"{rate:.1f} tok/s against a floor of {a.min_tok_s}"))

    rc, out = _captured(lambda: workloads.main(["agents"] + base + ["--agents", "2", "--turns", "3", "--prefix-tokens", "200", "--max-tokens", "48"]))
    steps.append(("agents", rc == 0, out.strip()[-300:]))

    for name, ok, note in steps:
        print(("PASS " if ok else "FAIL ") + name + ("" if ok else "  -- " + note))
    bad = sum(1 for _, ok, _ in steps if not ok)
    print("release gate: " + ("PASS" if not bad else f"FAIL ({bad} of {len(steps)} steps)"))
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
