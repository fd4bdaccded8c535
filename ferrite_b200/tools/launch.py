"""Launcher for the server: one process on one GPU, or one process per GPU with tensor parallelism (rank 0 serves HTTP
and schedules, the other ranks follow its engine calls). The role of the reference's `scripts/serve.sh`,
`tools/serve-tp2.sh`, `tools/tp2.sh` and `tools/launch-lib.sh`.

    python -m ferrite_b200.tools.launch --gpus 1 -- --preset 27b --port 8000
    python -m ferrite_b200.tools.launch --gpus 8 -- --model-dir /models/27b --weights bf16 --port 8000
    python -m ferrite_b200.tools.launch --preset 27b-spec --port 8000           # a named bundle of arguments + environment
    python -m ferrite_b200.tools.launch --list-presets

Everything after `--` goes to `python -m ferrite_b200.server`. Environment read by the server and the engine
(`config.py`): FERRITE_MODEL_DIR, FERRITE_WEIGHTS, FERRITE_SLOTS, FERRITE_CTX, FERRITE_CHUNK, FERRITE_PROFILE, FE_SPEC,
FE_POOL, FE_BATCH_ROWS, FE_NO_GRAPHS, FE_KV_DTYPE, FE_NO_SEQ_PARALLEL, FE_SHARE_MIN.

GPU locks: the launcher holds one lock file per GPU it uses (`<FERRITE_GPU_LOCK>.<index>`, default
`/var/tmp/ferrite-b200-gpu.lock`) exclusively for the life of the server, taken in ascending GPU order (so two
launchers that overlap can never hold each other's first lock). A second launcher on a taken GPU stops at once and
names the holder's PID and command; `FERRITE_LOCK_WAIT=1` waits instead. `--gpu-ids 4,5` picks the GPUs (exported as
CUDA_VISIBLE_DEVICES). The port is checked before anything is loaded. Ctrl-C / SIGTERM are forwarded to the server.
"""
from __future__ import annotations

import argparse
import fcntl
import os
import signal
import socket
import subprocess
import sys
from typing import Dict, List, Optional, Tuple

# name -> (GPUs, server arguments, environment). Sizes are for 180 GB per GPU.
PRESETS: Dict[str, Tuple[int, List[str], Dict[str, str]]] = {
    "27b": (1, ["--preset", "27b", "--slots", "8", "--max-model-len", "32768"], {}),
    "27b-nvfp4": (1, ["--preset", "27b", "--weights", "nvfp4", "--slots", "8", "--max-model-len", "32768"], {}),
    "27b-exl3": (1, ["--preset", "27b", "--weights", "exl3", "--slots", "8", "--max-model-len", "32768"], {}),
    "27b-spec": (1, ["--preset", "27b", "--slots", "8", "--max-model-len", "32768", "--drafter", "block"],
                 {"FE_SPEC": "16", "FE_TREE": "48"}),
    "27b-mtp": (1, ["--preset", "27b", "--slots", "8", "--max-model-len", "32768", "--drafter", "mtp"], {"FE_SPEC": "8"}),
    "27b-long": (1, ["--preset", "27b", "--slots", "2", "--max-model-len", "262144"], {"FE_KV_DTYPE": "fp8"}),
    "27b-tp2": (2, ["--preset", "27b", "--slots", "8", "--max-model-len", "32768"], {}),
    "27b-tp8": (8, ["--preset", "27b", "--slots", "16", "--max-model-len", "65536"], {}),
    "moe80b-ep8": (8, ["--preset", "moe80b", "--weights", "nvfp4", "--slots", "16", "--max-model-len", "32768"], {}),
    "mla671b-ep8": (8, ["--preset", "mla671b", "--weights", "nvfp4", "--slots", "64", "--max-model-len", "32768"], {}),
    "mock": (0, ["--engine", "mock"], {}),
}


class LockBusy(RuntimeError):
    pass


def take_gpu_locks(gpu_ids: List[int], base: Optional[str] = None, wait: bool = False, note: str = "") -> List[int]:
    """Exclusive lock file per GPU, ascending order. Returns the open file descriptors (keep them for the job's life).
    Raises LockBusy naming the holder when a lock is taken and `wait` is false."""
    base = base or os.environ.get("FERRITE_GPU_LOCK", "/var/tmp/ferrite-b200-gpu.lock")
    fds: List[int] = []
    try:
        for g in sorted(set(gpu_ids)):
            path = f"{base}.{g}"
            fd = os.open(path, os.O_RDWR | os.O_CREAT, 0o666)
            try:
                fcntl.flock(fd, fcntl.LOCK_EX | (0 if wait else fcntl.LOCK_NB))
            except BlockingIOError:
                holder = os.pread(fd, 512, 0).decode("utf-8", "replace").strip() or "unknown"
                os.close(fd)
                raise LockBusy(f"GPU {g} is in use ({path}): held by {holder}; FERRITE_LOCK_WAIT=1 waits for it") from None
            os.ftruncate(fd, 0)
            os.pwrite(fd, f"pid {os.getpid()} {note}".strip().encode(), 0)
            fds.append(fd)
    except BaseException:
        release_locks(fds)
        raise
    return fds


def release_locks(fds: List[int]) -> None:
    for fd in fds:
        try:
            os.ftruncate(fd, 0)
            fcntl.flock(fd, fcntl.LOCK_UN)
            os.close(fd)
        except OSError:
            pass


def port_of(server_args: List[str]) -> int:
    for i, a in enumerate(server_args):
        if a == "--port" and i + 1 < len(server_args):
            return int(server_args[i + 1])
        if a.startswith("--port="):
            return int(a.split("=", 1)[1])
    return 0


def port_in_use(port: int, host: str = "127.0.0.1") -> bool:
    with socket.socket() as s:
        s.settimeout(0.5)
        return s.connect_ex((host, port)) == 0


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
    rest: List[str] = []
    if "--" in argv:
        i = argv.index("--")
        argv, rest = argv[:i], argv[i + 1:]
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=0, help="ranks (default: the preset's, else 1)")
    ap.add_argument("--gpu-ids", default="", help="which GPUs, e.g. 4,5 (default 0..gpus-1)")
    ap.add_argument("--preset", default="", help="named bundle of server arguments and environment")
    ap.add_argument("--list-presets", action="store_true")
    ap.add_argument("--port", type=int, default=0, help="shorthand for `-- --port N`")
    ap.add_argument("--master-port", type=int, default=0)
    ap.add_argument("--no-lock", action="store_true", help="do not take the GPU lock files")
    ap.add_argument("--dry-run", action="store_true", help="print the command instead of running it")
    a = ap.parse_args(argv)
    if a.list_presets:
        for name, (g, args, env) in PRESETS.items():
            print(f"{name:14s} gpus={g}  {' '.join(args)}  {' '.join(f'{k}={v}' for k, v in env.items())}".rstrip())
        return 0
    env = dict(os.environ)
    gpus = a.gpus
    if a.preset:
        if a.preset not in PRESETS:
            print(f"unknown preset {a.preset!r}; --list-presets shows them", file=sys.stderr)
            return 2
        pg, pargs, penv = PRESETS[a.preset]
        gpus = gpus or pg
        rest = list(pargs) + rest                       # later arguments win in argparse: the caller's override the preset's
        for k, v in penv.items():
            env.setdefault(k, v)
    if a.port:
        rest += ["--port", str(a.port)]
    uses_gpu = not (a.preset and PRESETS[a.preset][0] == 0) and "mock" not in rest and "fake" not in rest
    gpus = max(1, gpus)
    ids = [int(x) for x in a.gpu_ids.split(",") if x] if a.gpu_ids else list(range(gpus))
    if len(ids) != gpus:
        print(f"--gpu-ids names {len(ids)} GPUs, --gpus says {gpus}", file=sys.stderr)
        return 2
    cmd = command(gpus, rest, a.master_port)
    if a.gpu_ids:
        env["CUDA_VISIBLE_DEVICES"] = ",".join(str(i) for i in ids)
    if a.dry_run:
        shown = " ".join(f"{k}={env[k]}" for k in sorted(env) if env.get(k) != os.environ.get(k))
        print((shown + " " if shown else "") + " ".join(cmd))
        return 0
    port = port_of(rest)
    if port and port_in_use(port):
        print(f"port {port} already answers: a server is running there", file=sys.stderr)
        return 3
    fds: List[int] = []
    if uses_gpu and not a.no_lock:
        try:
            fds = take_gpu_locks(ids, wait=os.environ.get("FERRITE_LOCK_WAIT", "0") == "1", note=" ".join(cmd[-6:]))
        except LockBusy as e:
            print(str(e), file=sys.stderr)
            return 4
    if gpus > 1:
        env.setdefault("MASTER_ADDR", "127.0.0.1")
    try:
        child = subprocess.Popen(cmd, env=env)

        def forward(signum, _frame):
            child.send_signal(signum)
        for sg in (signal.SIGINT, signal.SIGTERM):
            signal.signal(sg, forward)
        return child.wait()
    finally:
        release_locks(fds)


if __name__ == "__main__":
    raise SystemExit(main())
