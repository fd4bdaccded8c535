"""Concurrency sweep over a running server: runs `quickbench` at several stream counts and prints one JSON line per
point plus a summary table (the role of the reference's `tools/bench/sweep.py` / `sweep.sh`).

    python -m ferrite_b200.tools.sweep --base-url http://127.0.0.1:8000 --streams 1,2,4,8 --prompt-tokens 512 --max-tokens 128
"""
from __future__ import annotations

import argparse
import contextlib
import io
import json

from . import quickbench


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="")
    ap.add_argument("--streams", default="1,2,4")
    ap.add_argument("--prompt-tokens", type=int, default=256)
    ap.add_argument("--max-tokens", type=int, default=128)
    a = ap.parse_args(argv)
    points = []
    for n in [int(x) for x in a.streams.split(",") if x]:
        buf = io.StringIO()
        with contextlib.redirect_stdout(buf):
            quickbench.main(["--base-url", a.base_url, "--model", a.model, "--streams", str(n), "--prompt-tokens",
                             str(a.prompt_tokens), "--max-tokens", str(a.max_tokens)])
        line = json.loads(buf.getvalue().strip().splitlines()[-1])
        points.append(line)
        print(json.dumps(line), flush=True)
    print(f"{'streams':>8} {'agg tok/s':>10} {'per-stream':>11} {'ttft s':>8}")
    for p in points:
        print(f"{p['streams']:>8} {p['aggregate_tok_s'] or 0:>10} {p['per_stream_decode_tok_s_median'] or 0:>11} {p['ttft_s_median'] or 0:>8}")
    return 0 if all(p["ok"] == p["streams"] for p in points) else 1


if __name__ == "__main__":
    raise SystemExit(main())
