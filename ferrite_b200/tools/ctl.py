"""Run a server in the background and manage it: start / stop / restart / status / log.

    python -m ferrite_b200.tools.ctl start [--preset 27b] [--port 8000] [-- extra launcher / server arguments]
    python -m ferrite_b200.tools.ctl stop | restart | status | log [-f]  [--port 8000]

One server a port. The log is `<log dir>/server-<port>.log` (the previous run's is kept as `.log.1`), the launcher's pid
is in `<log dir>/server-<port>.pid`; `FERRITE_LOG_DIR` (default `./logs`) moves both.

  start    starts `tools/launch.py` in its own session (so it outlives this shell and takes the GPU lock files itself),
           waits until GET /health answers (`FERRITE_START_TIMEOUT` seconds, default 900) and prints the address; if the
           server exits while loading, the end of its log is printed and the command fails
  stop     SIGTERM to the launcher (which forwards it; open streams get their grace period), SIGKILL after 60 s
  status   running or not, and the /health document
  log      prints the log (`-f` follows it)

The role of the reference's `scripts/ferritectl.sh`.
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import time
import urllib.error
import urllib.request
from typing import List, Optional, Tuple


def paths(port: int) -> Tuple[str, str]:
    d = os.environ.get("FERRITE_LOG_DIR", os.path.join(os.getcwd(), "logs"))
    os.makedirs(d, exist_ok=True)
    return os.path.join(d, f"server-{port}.log"), os.path.join(d, f"server-{port}.pid")


def read_pid(pidf: str) -> Optional[int]:
    try:
        pid = int(open(pidf).read().strip())
        os.kill(pid, 0)
        return pid
    except (OSError, ValueError):
        return None


def health(port: int, timeout: float = 2.0) -> Optional[dict]:
    try:
        with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=timeout) as r:
            return json.loads(r.read().decode("utf-8"))
    except (urllib.error.URLError, OSError, ValueError):
        return None


def tail(path: str, n: int = 30) -> str:
    try:
        with open(path, "r", errors="replace") as f:
            return "".join(f.readlines()[-n:])
    except OSError:
        return ""


def start(port: int, preset: str, rest: List[str], wait_s: float) -> int:
    log, pidf = paths(port)
    if read_pid(pidf) is not None:
        print(f"already running (pid {read_pid(pidf)}, port {port}): stop it first", file=sys.stderr)
        return 1
    if os.path.exists(log):
        os.replace(log, log + ".1")
    cmd = [sys.executable, "-m", "ferrite_b200.tools.launch", "--port", str(port)]
    if preset:
        cmd += ["--preset", preset]
    cmd += rest
    with open(log, "ab") as f:
        child = subprocess.Popen(cmd, stdout=f, stderr=subprocess.STDOUT, stdin=subprocess.DEVNULL, start_new_session=True)
    with open(pidf, "w") as f:
        f.write(str(child.pid))
    t0 = time.time()
    while time.time() - t0 < wait_s:
        if child.poll() is not None:
            print(f"the server exited with code {child.returncode} while loading; end of {log}:\n{tail(log)}", file=sys.stderr)
            os.remove(pidf)
            return 1
        if health(port) is not None:
            print(f"serving on http://127.0.0.1:{port} (pid {child.pid}, log {log})")
            return 0
        time.sleep(0.25)
    print(f"no answer from /health after {wait_s:.0f} s (pid {child.pid} still loading?); see {log}", file=sys.stderr)
    return 1


def stop(port: int, grace_s: float = 60.0) -> int:
    _, pidf = paths(port)
    pid = read_pid(pidf)
    if pid is None:
        print("not running")
        return 0
    os.kill(pid, signal.SIGTERM)
    t0 = time.time()
    while time.time() - t0 < grace_s:
        try:
            done, _ = os.waitpid(pid, os.WNOHANG)          # our own child (started from this process): reap it
            if done:
                break
        except ChildProcessError:
            pass
        if read_pid(pidf) is None:
            break
        time.sleep(0.1)
    else:
        try:
            os.killpg(pid, signal.SIGKILL)                  # the launcher started its own session: pid == process group
        except OSError:
            pass
    try:
        os.remove(pidf)
    except OSError:
        pass
    print("stopped")
    return 0


def status(port: int) -> int:
    _, pidf = paths(port)
    pid = read_pid(pidf)
    h = health(port)
    print(json.dumps({"running": pid is not None, "pid": pid, "port": port, "health": h}))
    return 0 if pid is not None and h is not None else 1


def show_log(port: int, follow: bool) -> int:
    log, _ = paths(port)
    if not follow:
        sys.stdout.write(tail(log, 10 ** 9))
        return 0
    with open(log, "r", errors="replace") as f:
        while True:
            line = f.readline()
            if line:
                sys.stdout.write(line)
                sys.stdout.flush()
            else:
                time.sleep(0.2)


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    rest: List[str] = []
    if "--" in argv:
        i = argv.index("--")
        argv, rest = argv[:i], ["--"] + argv[i + 1:]
    ap = argparse.ArgumentParser()
    ap.add_argument("cmd", choices=["start", "stop", "restart", "status", "log"])
    ap.add_argument("--port", type=int, default=int(os.environ.get("FERRITE_PORT", "8000")))
    ap.add_argument("--preset", default="")
    ap.add_argument("-f", "--follow", action="store_true")
    a = ap.parse_args(argv)
    wait_s = float(os.environ.get("FERRITE_START_TIMEOUT", "900"))
    if a.cmd == "start":
        return start(a.port, a.preset, rest, wait_s)
    if a.cmd == "stop":
        return stop(a.port)
    if a.cmd == "restart":
        stop(a.port)
        return start(a.port, a.preset, rest, wait_s)
    if a.cmd == "status":
        return status(a.port)
    return show_log(a.port, a.follow)


if __name__ == "__main__":
    raise SystemExit(main())
