"""Build a release archive of the framework: the Python package with its kernel sources and the built extension, the
bench and entry scripts, the docs and profiles.

    python -m ferrite_b200.tools.package [--no-build] [--dev] [--out DIR] [--allow PATTERN ...]

Output: DIR/ferrite-b200-<version>-sm100a.tar.gz and its .sha256 (DIR defaults to dist/); <version> is the package's
`__version__`, `--dev` adds `git describe` to the name. Inside the archive, under one top folder of the same name:
  ferrite_b200/          the package: Python, `csrc/` (every kernel's source), `_C.so` (built for sm_100a)
  bench.py, __graft_entry__.py, README.md, profiles/, tests/
  BUILD-INFO             commit, describe, build time, Python / PyTorch / CUDA versions, the nvcc arch flags, and the
                         SHA-256 of every file in the archive
Unpacked, the release runs from its own folder (`python -m ferrite_b200.server ...`); `python -m
ferrite_b200.tools.check_env` tells whether the extension loads against the PyTorch found there.

Before anything is written the packed text files are scanned for this machine's traces (the home folder, the user and
host names, private network addresses): any hit stops the release and names file and line. `--allow` exempts a regular
expression (loopback addresses in docs and tests are exempt already).

The role of the reference's `scripts/package-release.sh`.
"""
from __future__ import annotations

import argparse
import getpass
import hashlib
import io
import json
import os
import re
import socket
import subprocess
import sys
import tarfile
import time
from typing import Dict, List, Tuple

ROOT_FILES = ["bench.py", "__graft_entry__.py", "README.md"]
ROOT_DIRS = ["ferrite_b200", "profiles", "tests"]
SKIP_DIRS = {"__pycache__", "build", ".pytest_cache", ".hypothesis"}
SKIP_SUFFIXES = (".pyc", ".o", ".a", ".ncu-rep")
TEXT_SUFFIXES = (".py", ".md", ".txt", ".json", ".cu", ".cuh", ".cpp", ".h", ".toml", ".cfg", ".sh", ".jinja")
PRIVATE_NET = re.compile(r"\b(?:10\.\d{1,3}|192\.168|172\.(?:1[6-9]|2\d|3[01]))\.\d{1,3}\.\d{1,3}\b")


def repo_root() -> str:
    return os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def collect(root: str) -> List[str]:
    """Paths (relative to the repository root) of everything that goes into the archive, sorted."""
    out: List[str] = [f for f in ROOT_FILES if os.path.isfile(os.path.join(root, f))]
    for d in ROOT_DIRS:
        for base, dirs, files in os.walk(os.path.join(root, d)):
            dirs[:] = sorted(x for x in dirs if x not in SKIP_DIRS)
            for f in sorted(files):
                if not f.endswith(SKIP_SUFFIXES):
                    out.append(os.path.relpath(os.path.join(base, f), root))
    return sorted(out)


def machine_traces() -> List[Tuple[str, "re.Pattern[str]"]]:
    pats: List[Tuple[str, re.Pattern]] = [("a private network address", PRIVATE_NET)]
    home = os.path.expanduser("~")
    if len(home) > 5 and home not in ("/root", "/home"):
        pats.append(("this machine's home folder", re.compile(re.escape(home))))
    try:
        user = getpass.getuser()
    except Exception:  # noqa: BLE001 - no passwd entry in some containers
        user = ""
    if len(user) > 3 and user not in ("root", "user", "ubuntu"):
        pats.append(("this machine's user name", re.compile(r"\b" + re.escape(user) + r"\b")))
    host = socket.gethostname().split(".")[0]
    if len(host) > 3 and host not in ("localhost",):
        pats.append(("this machine's host name", re.compile(r"\b" + re.escape(host) + r"\b")))
    return pats


def scan(root: str, files: List[str], allow: List[str]) -> List[str]:
    """Lines of the packed text files that carry a trace of this machine: `path:line: what`."""
    pats = machine_traces()
    ok = [re.compile(a) for a in allow]
    hits: List[str] = []
    for rel in files:
        if not rel.endswith(TEXT_SUFFIXES):
            continue
        try:
            with open(os.path.join(root, rel), "r", encoding="utf-8", errors="replace") as f:
                for n, line in enumerate(f, 1):
                    for what, p in pats:
                        m = p.search(line)
                        if m and not any(a.search(line) for a in ok):
                            hits.append(f"{rel}:{n}: {what} ({m.group(0)})")
        except OSError:
            continue
    return hits


def git(root: str, *args: str) -> str:
    try:
        return subprocess.run(["git", "-C", root] + list(args), capture_output=True, text=True, timeout=30).stdout.strip()
    except (OSError, subprocess.SubprocessError):
        return ""


def sha256_file(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 22), b""):
            h.update(block)
    return h.hexdigest()


def build_info(root: str, files: List[str]) -> Dict[str, object]:
    info: Dict[str, object] = {
        "commit": git(root, "rev-parse", "HEAD") or "unknown",
        "describe": git(root, "describe", "--tags", "--always", "--dirty") or "unknown",
        "built": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()),
        "python": sys.version.split()[0],
        "arch": "-gencode arch=compute_100a,code=sm_100a",
    }
    try:
        import torch
        info["torch"] = torch.__version__
        info["torch_cuda"] = torch.version.cuda
    except ImportError:
        info["torch"] = None
    info["files"] = {rel: sha256_file(os.path.join(root, rel)) for rel in files}
    return info


def package(root: str, out_dir: str, build: bool = True, dev: bool = False, allow: List[str] = ()) -> Tuple[str, Dict[str, object]]:
    with open(os.path.join(root, "ferrite_b200", "__init__.py"), "r", encoding="utf-8") as f:
        m = re.search(r'^__version__\s*=\s*["\']([^"\']+)["\']', f.read(), re.M)
    version = m.group(1) if m else "0"
    if build:
        r = subprocess.run([sys.executable, "-m", "ferrite_b200.build"], cwd=root)
        if r.returncode:
            raise SystemExit("package: the extension did not build")
    so = os.path.join(root, "ferrite_b200", "_C.so")
    if not os.path.exists(so):
        raise SystemExit("package: ferrite_b200/_C.so is missing (build first, or drop --no-build)")
    files = collect(root)
    hits = scan(root, files, list(allow))
    if hits:
        raise SystemExit("package: traces of this machine in the packed files:\n  " + "\n  ".join(hits[:20]))
    info = build_info(root, files)
    name = f"ferrite-b200-{version}-sm100a"
    if dev:
        name = f"ferrite-b200-{version}-{info['describe']}-sm100a"
    if str(info["describe"]).endswith("-dirty"):
        print(f"package: warning: the work tree has uncommitted changes ({info['describe']})", file=sys.stderr)
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, name + ".tar.gz")
    with tarfile.open(path, "w:gz") as tar:
        for rel in files:
            tar.add(os.path.join(root, rel), arcname=f"{name}/{rel}", recursive=False)
        blob = (json.dumps(info, indent=1, sort_keys=True) + "\n").encode()
        ti = tarfile.TarInfo(f"{name}/BUILD-INFO")
        ti.size, ti.mtime, ti.mode = len(blob), int(time.time()), 0o644
        tar.addfile(ti, io.BytesIO(blob))
    with open(path + ".sha256", "w", encoding="utf-8") as f:
        f.write(f"{sha256_file(path)}  {os.path.basename(path)}\n")
    return path, info


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="ferrite_b200.tools.package")
    ap.add_argument("--no-build", action="store_true")
    ap.add_argument("--dev", action="store_true")
    ap.add_argument("--out", default="")
    ap.add_argument("--allow", action="append", default=[r"127\.0\.0\.1", r"10\.0\.0\.0/8", r"192\.168\.0\.0/16"])
    a = ap.parse_args(argv)
    root = repo_root()
    path, info = package(root, a.out or os.path.join(root, "dist"), build=not a.no_build, dev=a.dev, allow=a.allow)
    print(json.dumps({"archive": path, "sha256_file": path + ".sha256", "files": len(info["files"]), "commit": info["commit"],
                      "bytes": os.path.getsize(path)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
