"""Tensor-parallel server gate: start a TP server, send concurrent requests through it, check them, stop it.

    python -m ferrite_b200.tools.tp_gate --gpus 2 [--port 8011] [--lanes 1,2,4] [-- server arguments]
    python -m ferrite_b200.tools.tp_gate --gpus 2 -- --preset tiny --device cpu          # gloo ranks, no GPU

Steps (each PASS / FAIL, exit code 1 on any failure):
  start     `torch.distributed.run` with one rank per GPU (rank 0 serves and schedules, the others follow); the server must
            answer /health within `--start-timeout` seconds with every rank still alive
  lanes     N chats sent together: every lane's greedy text equals the same request sent alone (a rank that drifted, a
            lost or reordered engine call on a follower, or a stale exchange buffer shows up here)
  repeat    the same request twice in a row gives the same text (the second is served from the prompt cache)
  spec      only when the server arguments name a draft model (`--drafter block`): /metrics shows drafted tokens, i.e. the
            mirrored drafter ran on every rank (a follower without one stops the stream with an error)
  ranks     after the requests every rank process is still running and the server's log holds no traceback
  stop      SIGTERM to the launcher ends all ranks within 60 s
The role of the reference's `tools/gate-serve-tp2.sh` (4 concurrent requests through the TP2 server, both ranks' logs).
"""
from __future__ import annotations

import argparse
import contextlib
import io
import json
import os
import signal
import socket
import subprocess
import sys
import tempfile
import time
from typing import List, Tuple

from .ctl import health, tail
from .launch import command


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def rank_pids(launcher_pid: int) -> List[int]:
    """Descendants of the launcher (the rank processes), from /proc."""
    kids: List[int] = []
    try:
        for name in os.listdir("/proc"):
            if not name.isdigit():
                continue
            try:
                with open(f"/proc/{name}/stat") as f:
                    ppid = int(f.read().rsplit(")", 1)[1].split()[1])
            except (OSError, ValueError, IndexError):
                continue
            if ppid == launcher_pid:
                kids.append(int(name))
    except OSError:
        pass
    return kids


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    rest: List[str] = []
    if "--" in argv:
        i = argv.index("--")
        argv, rest = argv[:i], argv[i + 1:]
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--port", type=int, default=0)
    ap.add_argument("--lanes", default="1,2,4")
    ap.add_argument("--prefix-tokens", type=int, default=300)
    ap.add_argument("--start-timeout", type=float, default=900.0)
    a = ap.parse_args(argv)
    port = a.port or free_port()
    from . import workloads
    from .httpc import Client
    steps: List[Tuple[str, bool, str]] = []
    log = tempfile.NamedTemporaryFile(prefix="tp-gate-", suffix=".log", delete=False)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = command(a.gpus, rest + ["--port", str(port)])
    child = subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT, stdin=subprocess.DEVNULL, env=env, start_new_session=True)
    try:
        t0 = time.time()
        up = False
        while time.time() - t0 < a.start_timeout and child.poll() is None:
            if health(port) is not None:
                up = True
                break
            time.sleep(0.3)
        steps.append(("start", up, "" if up else f"no /health answer; end of the log:\n{tail(log.name, 20)}"))
        if up:
            base = ["--base-url", f"http://127.0.0.1:{port}"]
            buf = io.StringIO()
            with contextlib.redirect_stdout(buf):
                try:
                    rc = workloads.main(["lanes"] + base + ["--lanes", a.lanes, "--prefix-tokens", str(a.prefix_tokens),
                                                           "--max-tokens", "32", "--runs", "1", "--gate"])
                except Exception as e:  # noqa: BLE001
                    rc, _ = 1, buf.write(repr(e))
            steps.append(("lanes", rc == 0, buf.getvalue().strip()[-300:]))
            c = Client(f"http://127.0.0.1:{port}")
            body = {"model": "", "messages": [{"role": "user", "content": "Name three uses of a prompt cache."}],
                    "max_tokens": 24, "temperature": 0}
            texts = []
            for _ in range(2):
                status, rep, _ = c.post("/v1/chat/completions", body)
                texts.append(json.dumps(rep.get("choices", [{}])[0].get("message")) if status == 200 else f"HTTP {status}")
            steps.append(("repeat", len(set(texts)) == 1 and not texts[0].startswith("HTTP"), str(texts)[:300]))
            if "--drafter" in rest and rest[rest.index("--drafter") + 1:][:1] not in ([], ["none"]):
                _, text = c.get("/metrics")
                n = next((float(ln.split()[1]) for ln in str(text).splitlines() if ln.startswith("ferrite_engine_drafted ")), 0.0)
                steps.append(("spec", n > 0, f"ferrite_engine_drafted = {n}"))
            ranks = rank_pids(child.pid)
            text = tail(log.name, 10 ** 6)
            ok = child.poll() is None and len(ranks) >= a.gpus - (1 if a.gpus == 1 else 0) and "Traceback" not in text
            steps.append(("ranks", ok, f"{len(ranks)} rank processes alive; traceback in the log: {'Traceback' in text}"))
    finally:
        t0 = time.time()
        if child.poll() is None:
            os.killpg(child.pid, signal.SIGTERM)
        while child.poll() is None and time.time() - t0 < 60:
            time.sleep(0.1)
        stopped = child.poll() is not None
        if not stopped:
            os.killpg(child.pid, signal.SIGKILL)
        steps.append(("stop", stopped, "" if stopped else "ranks did not end within 60 s of SIGTERM"))
    for name, ok, note in steps:
        print(("PASS " if ok else "FAIL ") + name + ("" if ok else "  -- " + note))
    bad = sum(1 for _, ok, _ in steps if not ok)
    print("tp gate: " + ("PASS" if not bad else f"FAIL ({bad} of {len(steps)} steps)") + f"  (log {log.name})")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
