"""Launcher for the server: one process on one GPU, or one process per GPU with tensor parallelism (rank 0 serves HTTP
and schedules, the other ranks follow its engine calls). The role of the reference's `scripts/serve.sh`,
`tools/serve-tp2.sh` and `tools/tp2.sh`.

    python -m ferrite_b200.tools.launch --gpus 1 -- --preset 27b --port 8000
    python -m ferrite_b200.tools.launch --gpus 8 -- --model-dir /models/27b --weights bf16 --port 8000

Everything after `--` goes to `python -m ferrite_b200.server`. Environment read by the server and the engine
(`config.py`): FERRITE_MODEL_DIR, FERRITE_WEIGHTS, FERRITE_SLOTS, FERRITE_CTX, FERRITE_CHUNK, FERRITE_PROFILE, FE_SPEC,
FE_POOL, FE_BATCH_ROWS, FE_NO_GRAPHS, FE_KV_DTYPE, FE_NO_SEQ_PARALLEL, FE_SHARE_MIN.
"""
from __future__ import annotations

import argparse
import os
import socket
import subprocess
import sys


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def command(gpus: int, server_args, master_port: int = 0):
    if gpus <= 1:
        return [sys.executable, "-m", "ferrite_b200.server", *server_args]
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}", "--master-addr",
            "127.0.0.1", "--master-port", str(master_port or free_port()), "-m", "ferrite_b200.server", *server_args]


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    rest = []
    if "--" in argv:
        i = argv.index("--")
        argv, rest = argv[:i], argv[i + 1:]
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--master-port", type=int, default=0)
    ap.add_argument("--dry-run", action="store_true", help="print the command instead of running it")
    a = ap.parse_args(argv)
    cmd = command(a.gpus, rest, a.master_port)
    if a.dry_run:
        print(" ".join(cmd))
        return 0
    env = dict(os.environ)
    if a.gpus > 1:
        env.setdefault("MASTER_ADDR", "127.0.0.1")
    return subprocess.call(cmd, env=env)


if __name__ == "__main__":
    raise SystemExit(main())
