"""In-tree build of the CUDA extension `ferrite_b200/_C.so` for sm_100a.

Kernels (`csrc/*.cu`) include no torch header and export a plain C launch API (`csrc/api.h`), so each compiles
in seconds; `csrc/bindings*.cpp` is the only torch-dependent part. Objects are rebuilt when their source or
any header is newer. The role of the reference's `crates/fe-kbuild` (nested kernel build + `ptxas`,
`crates/fe-kbuild/src/lib.rs:94-172`), minus the arch detection: sm_100a is the only target.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = CSRC / "build"
SO = ROOT / "_C.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default", "--threads", "2",
]


def _nvcc() -> str:
    home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    return str(Path(home) / "bin" / "nvcc")


def _newer(src: Path, dst: Path, deps) -> bool:
    if not dst.exists():
        return True
    t = dst.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *deps])


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(map(str, cmd))}\n{r.stdout}\n{r.stderr}")
    return r.stdout + r.stderr


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension as ce

    OBJ.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh"))
    cu = sorted(CSRC.glob("*.cu"))
    cpp = sorted(CSRC.glob("*.cpp"))
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}", f"-I{CSRC}"]
    abi = f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"
    jobs = []
    logs = []
    for s in cu:
        o = OBJ / (s.stem + ".o")
        if force or _newer(s, o, headers):
            cmd = [_nvcc(), *NVCC_FLAGS, f"-I{CSRC}", "-c", str(s), "-o", str(o)]
            if ptxas_info:
                cmd += ["-Xptxas", "-v"]
            jobs.append(cmd)
    for s in cpp:
        o = OBJ / (s.stem + ".o")
        if force or _newer(s, o, headers):
            jobs.append(["g++", "-O2", "-std=c++17", "-fPIC", abi, "-DTORCH_EXTENSION_NAME=_C",
                         "-DTORCH_API_INCLUDE_EXTENSION_H", *inc, "-c", str(s), "-o", str(o)])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=max(1, (os.cpu_count() or 4) // 2)) as ex:
            for out in ex.map(lambda c: _run(c, verbose), jobs):
                logs.append(out)
    objs = [OBJ / (s.stem + ".o") for s in cu + cpp]
    if jobs or not SO.exists() or force:
        libdir = Path(torch.__file__).parent / "lib"
        cuda_lib = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "lib64"
        cmd = ["g++", "-shared", "-o", str(SO), *map(str, objs), f"-L{libdir}", f"-L{cuda_lib}", "-lc10", "-lc10_cuda",
               "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart",
               f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{cuda_lib}"]
        _run(cmd, verbose)
    if ptxas_info:
        print("\n".join(logs))
    return SO


if __name__ == "__main__":
    build(verbose="-v" in sys.argv, force="-f" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(SO)
