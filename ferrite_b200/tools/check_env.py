"""Check that this machine can build and run the engine: toolchain, libraries, GPUs, memory, peer access.

    python -m ferrite_b200.tools.check_env [--build] [--gpus N] [--min-free-gb G] [--json]

  always    Python and PyTorch versions, the CUDA version PyTorch was built with, NCCL, whether the in-tree extension
            `ferrite_b200/_C.so` exists and loads (its host-side classes need no GPU)
  --build   what building from source needs: nvcc (and that it accepts `-gencode arch=compute_100a,code=sm_100a`), g++,
            the CUDA include paths of PyTorch
  GPUs      when CUDA is available: every device's name, compute capability (10.0 = B200 is what the kernels are built
            for), memory, and with --gpus N that N devices are there and every ordered pair can reach each other's memory
            (`torch.cuda.can_device_access_peer`)
  memory    available host memory against --min-free-gb (inside a memory-limited cgroup the limit counts)

Exit status 1 when something required is missing; warnings do not fail. The role of the reference's
`scripts/check-deps.sh`.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import tempfile
from typing import Any, Dict, List


def host_memory_gb() -> float:
    avail = 0.0
    try:
        for ln in open("/proc/meminfo"):
            if ln.startswith("MemAvailable:"):
                avail = int(ln.split()[1]) / (1 << 20)
    except OSError:
        pass
    for p in ("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory/memory.limit_in_bytes"):
        try:
            v = open(p).read().strip()
            if v.isdigit() and int(v) < (1 << 60):
                used = 0
                for q in ("/sys/fs/cgroup/memory.current", "/sys/fs/cgroup/memory/memory.usage_in_bytes"):
                    try:
                        used = int(open(q).read().strip())
                        break
                    except OSError:
                        pass
                avail = min(avail, (int(v) - used) / (1 << 30)) if avail else (int(v) - used) / (1 << 30)
        except OSError:
            pass
    return round(avail, 1)


def check(build: bool = False, gpus: int = 0, min_free_gb: float = 0.0) -> Dict[str, Any]:
    rep: Dict[str, Any] = {"errors": [], "warnings": []}
    err, warn = rep["errors"].append, rep["warnings"].append
    rep["python"] = sys.version.split()[0]
    try:
        import torch
        rep["torch"] = torch.__version__
        rep["torch_cuda"] = torch.version.cuda
        try:
            rep["nccl"] = ".".join(str(x) for x in torch.cuda.nccl.version())
        except Exception:  # noqa: BLE001
            rep["nccl"] = None
            warn("NCCL version not readable: tensor parallelism needs torch.distributed with the nccl backend")
    except ImportError as e:
        err(f"PyTorch does not import: {e}")
        return rep
    from .. import _ext
    rep["extension"] = str(_ext.so_path())
    if not _ext.so_path().exists():
        (err if not build else warn)("ferrite_b200/_C.so is not built: run `python -m ferrite_b200.build`")
    else:
        try:
            m = _ext.load(build_if_missing=False)
            rep["extension_loads"] = True
            rep["host_runtime"] = hasattr(m, "CopyIndex")
        except Exception as e:  # noqa: BLE001
            rep["extension_loads"] = False
            err(f"ferrite_b200/_C.so does not load (built for another PyTorch?): {e}")
    if build:
        nvcc = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
        if not os.path.exists(nvcc):
            err("nvcc not found (CUDA_HOME or PATH)")
        else:
            rep["nvcc"] = subprocess.run([nvcc, "--version"], capture_output=True, text=True).stdout.strip().splitlines()[-1]
            with tempfile.TemporaryDirectory() as d:
                src = os.path.join(d, "t.cu")
                open(src, "w").write("__global__ void k() {}\n")
                r = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-c", src, "-o", os.path.join(d, "t.o")],
                                   capture_output=True, text=True)
                rep["nvcc_sm_100a"] = r.returncode == 0
                if r.returncode:
                    err("nvcc does not accept arch=compute_100a,code=sm_100a (CUDA 12.8 or newer is needed): " + r.stderr.strip()[:200])
        if shutil.which("g++") is None:
            err("g++ not found")
    rep["host_memory_free_gb"] = host_memory_gb()
    if min_free_gb and rep["host_memory_free_gb"] < min_free_gb:
        warn(f"only {rep['host_memory_free_gb']} GB of host memory available, {min_free_gb} wanted")
    devs: List[Dict[str, Any]] = []
    if torch.cuda.is_available():
        n = torch.cuda.device_count()
        for i in range(n):
            p = torch.cuda.get_device_properties(i)
            devs.append({"index": i, "name": p.name, "capability": f"{p.major}.{p.minor}",
                         "memory_gb": round(p.total_memory / (1 << 30), 1), "sms": p.multi_processor_count})
            if (p.major, p.minor) != (10, 0):
                err(f"GPU {i} ({p.name}) has compute capability {p.major}.{p.minor}: the kernels are built for 10.0 (sm_100a) only")
        if gpus:
            if n < gpus:
                err(f"{gpus} GPUs wanted, {n} visible")
            else:
                bad = [(a, b) for a in range(gpus) for b in range(gpus) if a != b and not torch.cuda.can_device_access_peer(a, b)]
                rep["peer_access"] = not bad
                if bad:
                    err(f"no peer access between GPU pairs {bad[:8]}: the fused collectives need NVLink / NVSwitch peer mappings")
    else:
        (err if gpus else warn)("no CUDA device visible: only the CPU engine (fp32 oracle) runs here")
    rep["gpus"] = devs
    return rep


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--build", action="store_true")
    ap.add_argument("--gpus", type=int, default=0)
    ap.add_argument("--min-free-gb", type=float, default=0.0)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    rep = check(a.build, a.gpus, a.min_free_gb)
    if a.json:
        print(json.dumps(rep))
    else:
        for k, v in rep.items():
            if k not in ("errors", "warnings", "gpus"):
                print(f"{k:22s} {v}")
        for g in rep.get("gpus", []):
            print(f"gpu {g['index']}: {g['name']}, capability {g['capability']}, {g['memory_gb']} GB, {g['sms']} SMs")
        for w in rep["warnings"]:
            print("warning:", w)
        for e in rep["errors"]:
            print("ERROR:", e)
        print("ok" if not rep["errors"] else f"{len(rep['errors'])} problem(s)")
    return 1 if rep["errors"] else 0


if __name__ == "__main__":
    raise SystemExit(main())
