"""Loader of the in-tree CUDA extension.

`load()` imports `ferrite_b200/_C.so`, building it first when it is missing. On a machine with a GPU a
missing or unloadable extension is an error (never a silent fallback to PyTorch ops); on a CPU-only machine
the engine runs on `ops.torch_ops.TorchOps` and does not need the extension.
"""
from __future__ import annotations

import importlib
import os
from pathlib import Path

_mod = None


def so_path() -> Path:
    return Path(__file__).resolve().parent / "_C.so"


def load(build_if_missing: bool = True):
    global _mod
    if _mod is not None:
        return _mod
    if not so_path().exists():
        if not build_if_missing or os.environ.get("FERRITE_NO_BUILD"):
            raise ImportError(f"{so_path()} is missing: run `python -m ferrite_b200.build`")
        from .build import build
        build()
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    _mod = importlib.import_module("ferrite_b200._C")
    return _mod


def available() -> bool:
    try:
        load(build_if_missing=False)
        return True
    except Exception:
        return False


def host():
    """The extension when it is already built (its host-side classes need no GPU), else None: callers fall back to their
    plain-Python statement of the same behaviour. `FERRITE_NO_NATIVE_HOST=1` forces the fallback."""
    if os.environ.get("FERRITE_NO_NATIVE_HOST"):
        return None
    try:
        m = load(build_if_missing=False)
    except Exception:  # noqa: BLE001 - not built, or built for another torch: the Python paths serve
        return None
    return m if hasattr(m, "CopyIndex") else None
