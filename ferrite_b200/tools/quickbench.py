"""Serving benchmark client: N concurrent streamed chat requests, time to first token and decode rate per stream and
in aggregate (the role of the reference's `tools/bench/quickbench.py` / `lanes.py`).

    python -m ferrite_b200.tools.quickbench --base-url http://127.0.0.1:8000 --streams 4 --prompt-tokens 512 --max-tokens 128

Prints one JSON line. Token counts come from the server's usage block of the final streamed chunk when present,
else from the number of content deltas.
"""
from __future__ import annotations

import argparse
import json
import random
import statistics
import threading
import time

from .httpc import Client


def one_stream(base_url, model, prompt, max_tokens, out, idx):
    c = Client(base_url)
    first = last = None
    n = 0
    usage = None
    try:
        for t, ev in c.stream("/v1/chat/completions", {"model": model, "messages": [{"role": "user", "content": prompt}],
                                                        "max_tokens": max_tokens, "temperature": 0,
                                                        "stream_options": {"include_usage": True}}):
            if ev is None:
                break
            if ev.get("usage"):
                usage = ev["usage"]
            for ch in ev.get("choices", []):
                d = ch.get("delta", {})
                if d.get("content") or d.get("reasoning_content") or d.get("tool_calls"):
                    n += 1
                    first = t if first is None else first
                    last = t
        out[idx] = {"ttft_s": first, "end_s": last, "tokens": (usage or {}).get("completion_tokens", n), "error": None}
    except Exception as e:  # noqa: BLE001
        out[idx] = {"ttft_s": None, "end_s": None, "tokens": 0, "error": repr(e)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="")
    ap.add_argument("--streams", type=int, default=1)
    ap.add_argument("--prompt-tokens", type=int, default=256)
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    model = a.model or Client(a.base_url).get("/v1/models")[1]["data"][0]["id"]
    rng = random.Random(a.seed)
    words = ["alpha", "beta", "gamma", "delta", "epsilon", "zeta", "eta", "theta", "iota", "kappa"]
    prompts = [" ".join(rng.choice(words) for _ in range(a.prompt_tokens)) for _ in range(a.streams)]
    out = [None] * a.streams
    t0 = time.perf_counter()
    ths = [threading.Thread(target=one_stream, args=(a.base_url, model, prompts[i], a.max_tokens, out, i)) for i in range(a.streams)]
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    wall = time.perf_counter() - t0
    ok = [o for o in out if o and not o["error"] and o["ttft_s"] is not None]
    total = sum(o["tokens"] for o in ok)
    rates = [(o["tokens"] - 1) / (o["end_s"] - o["ttft_s"]) for o in ok if o["tokens"] > 1 and o["end_s"] > o["ttft_s"]]
    print(json.dumps({"streams": a.streams, "ok": len(ok), "errors": [o["error"] for o in out if o and o["error"]],
                      "wall_s": round(wall, 3), "total_tokens": total, "aggregate_tok_s": round(total / wall, 2) if wall else None,
                      "ttft_s_median": round(statistics.median(o["ttft_s"] for o in ok), 4) if ok else None,
                      "per_stream_decode_tok_s_median": round(statistics.median(rates), 2) if rates else None}))
    return 0 if len(ok) == a.streams else 1


if __name__ == "__main__":
    raise SystemExit(main())
