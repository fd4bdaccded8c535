"""Workload clients for an OpenAI-compatible server (client only, standard library):

    python -m ferrite_b200.tools.workloads edit   --base-url URL --streams 4 --max-tokens 800 [--out PREFIX]
    python -m ferrite_b200.tools.workloads lanes  --base-url URL --lanes 1,2,4 --prefix-tokens 2000 [--gate]
    python -m ferrite_b200.tools.workloads mixed  --base-url URL --decoders 2 --prompts 3 --prompt-tokens 4000
    python -m ferrite_b200.tools.workloads agents --base-url URL --agents 4 --turns 5

    python -m ferrite_b200.tools.workloads modes  --base-url URL --save ref.json | --compare ref.json
    python -m ferrite_b200.tools.workloads turns  --base-url URL --turns 8

Each prints one JSON line.
  edit    a Python standard-library module in the prompt, an instruction that keeps most of it, the whole updated module
          back (greedy): the workload context-copy speculation is built for. Streams start together; tok/s per stream.
  lanes   N chats sent together that share a long opening text and end in a tail of their own: output tok/s of the whole
          set, per-lane tok/s, prompt tokens sent / served from the cache. `--gate`: every lane's text in the N-lane call
          must equal the text of the same request sent alone (greedy), exit code 1 otherwise.
  mixed   long prompts arrive while decode streams are running: the gaps between a running stream's chunks (median, p99,
          max) show what a prompt costs the streams; time to first token of the prompts shows what the streams cost them.
  agents  sessions of several turns with a tool call per turn, each turn re-sending the conversation so far: turn latency
          and the share of prompt tokens the server took from its cache.
  modes   the mode gate: a fixed set of greedy requests (with and without a system message, short and long, a follow-up
          turn, a file edit) sent one by one to a server; a hash per case is saved (`--save`) or compared with the hashes
          another configuration of the server produced (`--compare`: prompt cache on / off, drafter kinds, weight
          formats that must not change greedy text); exit code 1 and the first differing characters on a mismatch.
  turns   one conversation behind a long system prompt grows turn by turn (each turn appends the reply and a tool
          result): per turn the prompt tokens, the tokens served from the cache, time to first token and a reply hash.
The clients read GET /health first and never send more requests at once than `max_batch_size` (points beyond are reported
as skipped). Counterparts of the reference's `tools/bench/edit.py`, `lanes.py`, `mixed.py`, `agents.py`, `modes.py`, `agentturns.py`.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import statistics
import sys
import threading
import time
from typing import Any, Dict, List, Optional

from .httpc import Client

WORDS = ("buffer index token layer cache stream kernel block shard queue batch scale tile warp row column state step "
         "draft verify prompt decode sample").split()


def filler(n_tokens: int, seed: int) -> str:
    """About n_tokens tokens of plain words (one word is about one token for the tokenizers in use)."""
    r = random.Random(seed)
    return " ".join(r.choice(WORDS) for _ in range(max(1, n_tokens)))


def server_limits(c: Client) -> Dict[str, int]:
    status, body = c.get("/health")
    if status != 200 or not isinstance(body, dict):
        return {"max_batch_size": 1 << 30, "max_model_len": 1 << 30}
    return {"max_batch_size": int(body.get("max_batch_size") or (1 << 30)), "max_model_len": int(body.get("max_model_len") or (1 << 30))}


def model_of(c: Client, model: str) -> str:
    if model:
        return model
    status, body = c.get("/v1/models")
    return body["data"][0]["id"] if status == 200 and body.get("data") else ""


class Run:
    """One streamed chat request: text, chunk times, usage."""

    def __init__(self):
        self.text = ""
        self.times: List[float] = []
        self.usage: Dict[str, Any] = {}
        self.calls: List[Dict[str, str]] = []
        self.error: Optional[str] = None
        self.t_end = 0.0

    @property
    def tokens(self) -> int:
        return int(self.usage.get("completion_tokens") or len(self.times))

    @property
    def cached(self) -> int:
        return int((self.usage.get("prompt_tokens_details") or {}).get("cached_tokens") or 0)


def stream_chat(base_url: str, body: Dict[str, Any], out: Run) -> None:
    try:
        calls: Dict[int, Dict[str, str]] = {}
        for t, ev in Client(base_url).stream("/v1/chat/completions", dict(body, stream_options={"include_usage": True})):
            if ev is None:
                out.t_end = t
                break
            if ev.get("usage"):
                out.usage = ev["usage"]
            for ch in ev.get("choices", []):
                d = ch.get("delta", {})
                piece = d.get("content") or ""
                for tc in d.get("tool_calls") or []:
                    slot = calls.setdefault(tc.get("index", 0), {"name": "", "arguments": "", "id": ""})
                    slot["id"] = tc.get("id") or slot["id"]
                    slot["name"] += tc.get("function", {}).get("name") or ""
                    slot["arguments"] += tc.get("function", {}).get("arguments") or ""
                if piece or d.get("reasoning_content") or d.get("tool_calls"):
                    out.times.append(t)
                out.text += piece
        out.calls = [calls[k] for k in sorted(calls)]
    except Exception as e:  # noqa: BLE001 - a failed stream is a result, not a crash of the bench
        out.error = repr(e)


def together(base_url: str, bodies: List[Dict[str, Any]]) -> List[Run]:
    runs = [Run() for _ in bodies]
    ts = [threading.Thread(target=stream_chat, args=(base_url, b, r)) for b, r in zip(bodies, runs)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    return runs


def rate(r: Run) -> float:
    return r.tokens / r.t_end if r.t_end > 0 else 0.0


# ---- edit -------------------------------------------------------------------------------------------------------------
EDIT_MODULES = ("textwrap.py", "shlex.py", "string.py", "bisect.py")


def module_source(name: str) -> str:
    """The running interpreter's own copy of a small standard-library module (any version: the bench compares builds of
    the server on the same client machine, not numbers across machines)."""
    path = os.path.join(os.path.dirname(os.__file__), name)
    with open(path, "r", encoding="utf-8") as f:
        return f.read()


def cmd_edit(a) -> int:
    c = Client(a.base_url)
    model = model_of(c, a.model)
    lim = server_limits(c)
    n = min(a.streams, lim["max_batch_size"])
    bodies = []
    for i in range(n):
        src = module_source(EDIT_MODULES[i % len(EDIT_MODULES)])
        if a.max_source_chars:
            src = src[:a.max_source_chars]
        ask = ("Here is a Python module.\n\n```python\n" + src + "\n```\n\nRename the first function's first parameter to `value` "
               "everywhere it is used, change nothing else, and reply with the whole updated module.")
        bodies.append({"model": model, "messages": [{"role": "user", "content": ask}], "max_tokens": a.max_tokens, "temperature": 0})
    t0 = time.perf_counter()
    runs = together(a.base_url, bodies)
    wall = time.perf_counter() - t0
    if a.out:
        for i, r in enumerate(runs):
            with open(f"{a.out}-{i}.txt", "w", encoding="utf-8") as f:
                f.write(r.text)
    ok = [r for r in runs if not r.error]
    print(json.dumps({"workload": "edit", "streams": n, "skipped_streams": a.streams - n, "errors": [r.error for r in runs if r.error],
                      "tokens": [r.tokens for r in ok], "tok_s_per_stream": [round(rate(r), 2) for r in ok],
                      "tok_s_total": round(sum(r.tokens for r in ok) / wall, 2) if wall > 0 else 0.0, "wall_s": round(wall, 3)}))
    return 0 if len(ok) == n else 1


# ---- lanes ------------------------------------------------------------------------------------------------------------
def lane_bodies(model: str, n: int, prefix_tokens: int, max_tokens: int, seed: int, job: str) -> List[Dict[str, Any]]:
    shared = f"job {job}\n" + filler(prefix_tokens, seed)
    return [{"model": model, "temperature": 0, "max_tokens": max_tokens,
             "messages": [{"role": "system", "content": "You write code."},
                          {"role": "user", "content": shared + f"\n\nlane {i}: " + filler(24, seed * 1000 + i)}]} for i in range(n)]


def cmd_lanes(a) -> int:
    c = Client(a.base_url)
    model = model_of(c, a.model)
    lim = server_limits(c)
    points, bad = [], 0
    for n in [int(x) for x in a.lanes.split(",") if x]:
        if n > lim["max_batch_size"]:
            points.append({"lanes": n, "skipped": f"max_batch_size {lim['max_batch_size']}"})
            continue
        sets = []
        for run in range(a.runs + 1):                    # the first set is a warm-up
            bodies = lane_bodies(model, n, a.prefix_tokens, a.max_tokens, a.seed, f"{a.seed}-{n}-gate" if a.gate else f"{a.seed}-{n}-{run}-{time.time_ns()}")
            t0 = time.perf_counter()
            runs = together(a.base_url, bodies)
            wall = time.perf_counter() - t0
            if run:
                sets.append((wall, runs))
        wall, runs = sorted(sets, key=lambda s: s[0])[len(sets) // 2]
        point = {"lanes": n, "errors": [r.error for r in runs if r.error], "wall_s": round(wall, 3),
                 "tok_s_total": round(sum(r.tokens for r in runs) / wall, 2),
                 "tok_s_per_lane": round(statistics.mean(rate(r) for r in runs), 2),
                 "prompt_tokens": sum(int(r.usage.get("prompt_tokens") or 0) for r in runs),
                 "cached_tokens": sum(r.cached for r in runs)}
        if a.gate:
            # the same requests one at a time: a lane's text must not depend on who shared its steps
            bodies = lane_bodies(model, n, a.prefix_tokens, a.max_tokens, a.seed, f"{a.seed}-{n}-gate")
            alone = [together(a.base_url, [b])[0] for b in bodies]
            diff = [i for i, (x, y) in enumerate(zip(runs, alone)) if x.text != y.text]
            point["gate_lanes_differing_from_alone"] = diff
            bad += len(diff)
        bad += len(point["errors"])
        points.append(point)
    print(json.dumps({"workload": "lanes", "prefix_tokens": a.prefix_tokens, "max_tokens": a.max_tokens, "gate": bool(a.gate), "points": points}))
    return 1 if bad else 0


# ---- mixed ------------------------------------------------------------------------------------------------------------
def cmd_mixed(a) -> int:
    c = Client(a.base_url)
    model = model_of(c, a.model)
    lim = server_limits(c)
    n_dec = min(a.decoders, max(1, lim["max_batch_size"] - 1))
    dec_bodies = [{"model": model, "temperature": 0, "max_tokens": a.max_tokens,
                   "messages": [{"role": "user", "content": f"stream {i}: " + filler(32, 50 + i)}]} for i in range(n_dec)]
    dec_runs = [Run() for _ in dec_bodies]
    ts = [threading.Thread(target=stream_chat, args=(a.base_url, b, r)) for b, r in zip(dec_bodies, dec_runs)]
    [t.start() for t in ts]
    time.sleep(a.lead_s)                                  # the streams are decoding when the prompts arrive
    prompts: List[Run] = []
    for i in range(a.prompts):
        r = Run()
        stream_chat(a.base_url, {"model": model, "temperature": 0, "max_tokens": 8,
                                 "messages": [{"role": "user", "content": f"doc {i} {time.time_ns()}: " + filler(a.prompt_tokens, 70 + i)}]}, r)
        prompts.append(r)
    [t.join() for t in ts]
    gaps = sorted(g for r in dec_runs for g in (y - x for x, y in zip(r.times, r.times[1:])))
    pick = lambda q: round(gaps[min(len(gaps) - 1, int(q * len(gaps)))] * 1e3, 2) if gaps else None
    errors = [r.error for r in dec_runs + prompts if r.error]
    print(json.dumps({"workload": "mixed", "decoders": n_dec, "prompts": a.prompts, "prompt_tokens": a.prompt_tokens, "errors": errors,
                      "decode_tok_s_per_stream": [round(rate(r), 2) for r in dec_runs],
                      "chunk_gap_ms": {"median": pick(0.5), "p99": pick(0.99), "max": pick(1.0)},
                      "prompt_ttft_s": [round(r.times[0], 3) if r.times else None for r in prompts]}))
    return 1 if errors else 0


# ---- agents -----------------------------------------------------------------------------------------------------------
AGENT_TOOLS = [{"type": "function", "function": {
    "name": "read_file", "description": "read a file of the project",
    "parameters": {"type": "object", "properties": {"path": {"type": "string"}}, "required": ["path"]}}}]


def agent_session(base_url: str, model: str, idx: int, turns: int, max_tokens: int, shared: str, out: List[Dict[str, Any]]) -> None:
    msgs: List[Dict[str, Any]] = [{"role": "system", "content": "You are a coding agent. " + shared},
                                  {"role": "user", "content": f"agent {idx}: find the bug in module {idx}."}]
    for turn in range(turns):
        r = Run()
        t0 = time.perf_counter()
        stream_chat(base_url, {"model": model, "temperature": 0, "max_tokens": max_tokens, "messages": msgs, "tools": AGENT_TOOLS}, r)
        rec = {"agent": idx, "turn": turn, "latency_s": round(time.perf_counter() - t0, 3), "tokens": r.tokens,
               "prompt_tokens": int(r.usage.get("prompt_tokens") or 0), "cached_tokens": r.cached, "tool_calls": len(r.calls),
               "error": r.error}
        out.append(rec)
        if r.error:
            return
        if r.calls:
            msgs.append({"role": "assistant", "content": r.text or None,
                         "tool_calls": [{"id": cl["id"] or f"call_{turn}_{j}", "type": "function",
                                         "function": {"name": cl["name"], "arguments": cl["arguments"]}} for j, cl in enumerate(r.calls)]})
            for j, cl in enumerate(r.calls):
                msgs.append({"role": "tool", "tool_call_id": cl["id"] or f"call_{turn}_{j}", "content": filler(120, idx * 100 + turn)})
        else:
            msgs.append({"role": "assistant", "content": r.text})
            msgs.append({"role": "user", "content": f"turn {turn}: go on. " + filler(40, idx * 100 + turn)})


def cmd_agents(a) -> int:
    c = Client(a.base_url)
    model = model_of(c, a.model)
    lim = server_limits(c)
    n = min(a.agents, lim["max_batch_size"])
    shared = filler(a.prefix_tokens, a.seed)
    recs: List[Dict[str, Any]] = []
    t0 = time.perf_counter()
    ts = [threading.Thread(target=agent_session, args=(a.base_url, model, i, a.turns, a.max_tokens, shared, recs)) for i in range(n)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    wall = time.perf_counter() - t0
    good = [r for r in recs if not r["error"]]
    later = [r for r in good if r["turn"] > 0]
    sent = sum(r["prompt_tokens"] for r in later)
    print(json.dumps({"workload": "agents", "agents": n, "skipped_agents": a.agents - n, "turns": a.turns, "wall_s": round(wall, 3),
                      "errors": [r["error"] for r in recs if r["error"]],
                      "turn_latency_s": {"median": round(statistics.median(r["latency_s"] for r in good), 3) if good else None,
                                         "max": max((r["latency_s"] for r in good), default=None)},
                      "tokens_total": sum(r["tokens"] for r in good), "tool_calls": sum(r["tool_calls"] for r in good),
                      "cached_share_after_first_turn": round(sum(r["cached_tokens"] for r in later) / sent, 3) if sent else None}))
    return 0 if len(good) == len(recs) and recs else 1


# ---- modes ------------------------------------------------------------------------------------------------------------
def mode_cases(seed: int, long_tokens: int = 3000, source_chars: int = 8000) -> List[Dict[str, Any]]:
    review = module_source("bisect.py")[:source_chars]
    sysbig = "You are the coding agent of an inference-engine repository. Project notes follow.\n\n" + filler(long_tokens, seed)
    edit = module_source("shlex.py")[:source_chars]
    first = [{"role": "system", "content": sysbig}, {"role": "user", "content": "Which note mentions the cache? One sentence."}]
    return [
        {"name": "sys-short-review", "max_tokens": 200, "messages": [
            {"role": "system", "content": "You are a careful code reviewer."},
            {"role": "user", "content": "Review this Python file. Name the three most important issues.\n\n" + review}]},
        {"name": "nosys-review", "max_tokens": 160, "messages": [
            {"role": "user", "content": "Review this Python file. Name the three most important issues.\n\n" + review}]},
        {"name": "sys-short-chat", "max_tokens": 120, "messages": [
            {"role": "system", "content": "You answer in one short paragraph."},
            {"role": "user", "content": "Why does a recurrent layer make prompt caching harder?"}]},
        {"name": "code", "max_tokens": 200, "messages": [
            {"role": "user", "content": "Write a Python function that checks whether a string is a palindrome, with three tests."}]},
        {"name": "sys-long-turn1", "max_tokens": 120, "messages": first},
        {"name": "sys-long-turn2", "max_tokens": 120, "follow": "sys-long-turn1", "messages": first, "then": "And which one mentions a queue?"},
        {"name": "edit", "max_tokens": 400, "messages": [
            {"role": "user", "content": "Rename every local variable named `s` to `text` in this module and return the whole "
                                        "module.\n\n" + edit}]},
    ]


def cmd_modes(a) -> int:
    import hashlib
    c = Client(a.base_url)
    model = model_of(c, a.model)
    replies: Dict[str, str] = {}
    for case in mode_cases(a.seed, a.long_tokens, a.max_source_chars):
        msgs = list(case["messages"])
        if case.get("follow"):
            msgs = msgs + [{"role": "assistant", "content": replies[case["follow"]]}, {"role": "user", "content": case["then"]}]
        r = Run()
        stream_chat(a.base_url, {"model": model, "messages": msgs, "max_tokens": min(case["max_tokens"], a.max_tokens),
                                 "temperature": 0, "stream": True}, r)
        if r.error:
            print(json.dumps({"workload": "modes", "case": case["name"], "error": r.error}))
            return 2
        replies[case["name"]] = r.text
    hashes = {k: hashlib.sha256(v.encode("utf-8")).hexdigest()[:16] for k, v in replies.items()}
    out: Dict[str, Any] = {"workload": "modes", "cases": len(hashes), "hashes": hashes}
    rc = 0
    if a.save:
        with open(a.save, "w", encoding="utf-8") as f:
            json.dump({"hashes": hashes, "texts": replies}, f)
        out["saved"] = a.save
    if a.compare:
        with open(a.compare, "r", encoding="utf-8") as f:
            ref = json.load(f)
        diff = {}
        for k, h in hashes.items():
            if ref["hashes"].get(k) != h:
                want, got = ref.get("texts", {}).get(k, ""), replies[k]
                i = next((j for j, (x, y) in enumerate(zip(want, got)) if x != y), min(len(want), len(got)))
                diff[k] = {"at": i, "want": want[i:i + 40], "got": got[i:i + 40]}
        out["different"] = diff
        rc = 1 if diff else 0
    print(json.dumps(out))
    return rc


# ---- turns ------------------------------------------------------------------------------------------------------------
def cmd_turns(a) -> int:
    import hashlib
    c = Client(a.base_url)
    model = model_of(c, a.model)
    msgs: List[Dict[str, Any]] = [{"role": "system", "content": "You are a coding agent. Notes:\n" + filler(a.prefix_tokens, a.seed)},
                                  {"role": "user", "content": "Start by listing what you would inspect first."}]
    rows = []
    for t in range(a.turns):
        r = Run()
        t0 = time.time()
        stream_chat(a.base_url, {"model": model, "messages": msgs, "max_tokens": a.max_tokens, "temperature": 0, "stream": True}, r)
        if r.error:
            print(json.dumps({"workload": "turns", "turn": t, "error": r.error}))
            return 2
        rows.append({"turn": t, "prompt_tokens": int(r.usage.get("prompt_tokens") or 0), "cached_tokens": r.cached,
                     "ttft_s": round(r.times[0], 4) if r.times else None, "total_s": round(time.time() - t0, 4),
                     "hash": hashlib.sha256(r.text.encode("utf-8")).hexdigest()[:12]})
        msgs += [{"role": "assistant", "content": r.text},
                 {"role": "user", "content": "Tool result:\n" + filler(a.tool_tokens, a.seed + 100 + t) + "\nContinue."}]
    sent = sum(x["prompt_tokens"] for x in rows)
    cached = sum(x["cached_tokens"] for x in rows)
    print(json.dumps({"workload": "turns", "turns": rows, "prompt_tokens_sent": sent, "served_from_cache": cached,
                      "cache_share": round(cached / sent, 3) if sent else 0.0}))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="what", required=True)

    def common(p):
        p.add_argument("--base-url", default="http://127.0.0.1:8000")
        p.add_argument("--model", default="")
        p.add_argument("--max-tokens", type=int, default=256)
        p.add_argument("--seed", type=int, default=7)
        return p
    p = common(sub.add_parser("edit"))
    p.add_argument("--streams", type=int, default=4)
    p.add_argument("--out", default="", help="save every reply as PREFIX-<i>.txt (identity across builds)")
    p.add_argument("--max-source-chars", type=int, default=0, help="cut the module (small context windows)")
    p = common(sub.add_parser("lanes"))
    p.add_argument("--lanes", default="1,2,4")
    p.add_argument("--prefix-tokens", type=int, default=2000)
    p.add_argument("--runs", type=int, default=3)
    p.add_argument("--gate", action="store_true")
    p = common(sub.add_parser("mixed"))
    p.add_argument("--decoders", type=int, default=2)
    p.add_argument("--prompts", type=int, default=3)
    p.add_argument("--prompt-tokens", type=int, default=4000)
    p.add_argument("--lead-s", type=float, default=0.5)
    p = common(sub.add_parser("agents"))
    p.add_argument("--agents", type=int, default=4)
    p.add_argument("--turns", type=int, default=5)
    p.add_argument("--prefix-tokens", type=int, default=1500)
    p = common(sub.add_parser("modes"))
    p.add_argument("--save", default="")
    p.add_argument("--compare", default="")
    p.add_argument("--long-tokens", type=int, default=3000, help="words of the long system prompt")
    p.add_argument("--max-source-chars", type=int, default=8000, help="cut of the source files in the prompts")
    p = common(sub.add_parser("turns"))
    p.add_argument("--turns", type=int, default=8)
    p.add_argument("--prefix-tokens", type=int, default=5000)
    p.add_argument("--tool-tokens", type=int, default=1000)
    a = ap.parse_args(argv)
    return {"edit": cmd_edit, "lanes": cmd_lanes, "mixed": cmd_mixed, "agents": cmd_agents, "modes": cmd_modes,
            "turns": cmd_turns}[a.what](a)


if __name__ == "__main__":
    sys.exit(main())
