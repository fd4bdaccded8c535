"""Check a model directory before serving it: does it load, is every tensor the engine needs there, do the shapes fit the
configuration, how many bytes is it and in which storage forms.

    python -m ferrite_b200.tools.check_model DIR [--preset 27b] [--manifest] [--verify MANIFEST.json]

Reads `config.json` (Hugging Face layout) or falls back to `--preset`, loads the checkpoint through the engine's own
loader (`formats/loader.py`: safetensors bf16, ModelOpt NVFP4 / FP8, EXL3; a `.gguf` file through `formats/gguf_model.py`)
without building an engine, and compares the result with `models/weights.py::weight_shapes`. Prints one JSON line: missing
and unexpected tensors, shape mismatches, a count and byte total per storage form, the parameter count. `--manifest` also
prints the SHA-256 and size of every file of the directory; `--verify` compares them with a stored manifest (a download
that was cut short or a file that changed fails here, not as garbage text later). Exit status 1 on any problem. The role
of the reference's `scripts/fetch-models.sh` checks against `scripts/models.manifest`.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
from typing import Any, Dict


def file_manifest(model_dir: str) -> Dict[str, Dict[str, Any]]:
    out = {}
    for name in sorted(os.listdir(model_dir)):
        path = os.path.join(model_dir, name)
        if not os.path.isfile(path):
            continue
        h = hashlib.sha256()
        with open(path, "rb") as f:
            for block in iter(lambda: f.read(1 << 22), b""):
                h.update(block)
        out[name] = {"bytes": os.path.getsize(path), "sha256": h.hexdigest()}
    return out


def storage_of(v) -> str:
    import torch
    if isinstance(v, torch.Tensor):
        return str(v.dtype).replace("torch.", "")
    return type(v).__name__


def nbytes_of(v) -> int:
    import torch
    if isinstance(v, torch.Tensor):
        return v.numel() * v.element_size()
    total = 0
    for x in vars(v).values():
        if isinstance(x, torch.Tensor):
            total += x.numel() * x.element_size()
        elif hasattr(x, "__dict__") and not isinstance(x, (str, int, float)):
            total += nbytes_of(x)
        elif isinstance(x, (list, tuple)):
            total += sum(nbytes_of(y) for y in x if hasattr(y, "__dict__") or isinstance(y, torch.Tensor))
    return total


def check(model_dir: str, preset: str = "") -> Dict[str, Any]:
    from ..config import PRESETS, ModelConfig
    from ..models.weights import weight_shapes
    rep: Dict[str, Any] = {"dir": model_dir, "problems": []}
    bad = rep["problems"].append
    cfg_path = os.path.join(model_dir, "config.json")
    files = sorted(os.listdir(model_dir))
    if os.path.exists(cfg_path):
        cfg = ModelConfig.from_hf(cfg_path)
    elif preset:
        cfg = PRESETS[preset]()
    else:
        bad("no config.json and no --preset")
        return rep
    try:
        if any(f.endswith(".safetensors") for f in files):
            from ..formats.loader import load_model_weights
            w = load_model_weights(model_dir, cfg)
        else:
            ggufs = [f for f in files if f.endswith(".gguf")]
            if not ggufs:
                bad("no .safetensors and no .gguf file")
                return rep
            from ..formats import gguf as G
            from ..formats.gguf_model import config_from_gguf, load_gguf_weights
            g = G.Gguf(os.path.join(model_dir, ggufs[0]))
            cfg = config_from_gguf(g, cfg)
            g.close()
            w = load_gguf_weights(os.path.join(model_dir, ggufs[0]), cfg)
    except Exception as e:  # noqa: BLE001 - the report is the point
        bad(f"the loader failed: {type(e).__name__}: {e}")
        return rep
    want = weight_shapes(cfg)
    rep["model"] = cfg.name
    rep["params"] = cfg.param_count()
    rep["missing"] = sorted(k for k in want if k not in w)
    rep["unexpected"] = sorted(k for k in w if k not in want)
    mism = {}
    forms: Dict[str, Dict[str, int]] = {}
    for k, v in w.items():
        shape = tuple(getattr(v, "shape", ()))
        if k in want and shape and tuple(want[k]) != shape:
            mism[k] = {"want": list(want[k]), "got": list(shape)}
        f = forms.setdefault(storage_of(v), {"tensors": 0, "bytes": 0})
        f["tensors"] += 1
        f["bytes"] += nbytes_of(v)
    rep["shape_mismatches"] = mism
    rep["storage"] = forms
    rep["bytes"] = sum(f["bytes"] for f in forms.values())
    if rep["missing"]:
        bad(f"{len(rep['missing'])} tensors missing, first: {rep['missing'][0]}")
    if mism:
        k = next(iter(mism))
        bad(f"{len(mism)} shape mismatches, first: {k} {mism[k]}")
    return rep


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("dir")
    ap.add_argument("--preset", default="")
    ap.add_argument("--manifest", action="store_true")
    ap.add_argument("--verify", default="", help="a stored manifest (the `files` object of an earlier --manifest run)")
    a = ap.parse_args(argv)
    rep = check(a.dir, a.preset)
    if a.manifest or a.verify:
        rep["files"] = file_manifest(a.dir)
    if a.verify:
        with open(a.verify, "r", encoding="utf-8") as f:
            ref = json.load(f)
        ref = ref.get("files", ref)
        for name, meta in ref.items():
            got = rep["files"].get(name)
            if got is None:
                rep["problems"].append(f"{name} is missing")
            elif got["sha256"] != meta["sha256"]:
                rep["problems"].append(f"{name} differs from the manifest ({got['bytes']} bytes against {meta['bytes']})")
    print(json.dumps(rep))
    return 1 if rep["problems"] else 0


if __name__ == "__main__":
    sys.exit(main())
