"""ModelOpt quantised checkpoints (NVFP4 and FP8), read as published.

Layout of a quantised `Linear` named `<base>` in the safetensors files:

* NVFP4: `<base>.weight` uint8 [out, in/2] (two e2m1 codes per byte, element 2i in the low nibble),
  `<base>.weight_scale` float8_e4m3fn [out, in/16] (one scale per 16-element block), `<base>.weight_scale_2` fp32
  scalar (tensor scale: w = e2m1 * weight_scale * weight_scale_2), `<base>.input_scale` fp32 scalar (static
  activation scale);
* FP8: `<base>.weight` float8_e4m3fn [out, in], `<base>.weight_scale` fp32 scalar, `<base>.input_scale` fp32 scalar.

Which modules are quantised, and how, is in `hf_quant_config.json` next to the weights
(`{"quantization": {"quant_algo": "NVFP4" | "FP8", "group_size": 16, "exclude_modules": [...]}}`) or in
`config.json` under `quantization_config`. Excluded modules (`lm_head`, routers, small projections) stay bf16.

Reference: `crates/fe-fp4/src/st.rs` (checkpoint reader, `algo`, `scalar`), `crates/fe-fp4/src/lib.rs:305-386`
(`HostLinear::load_sliced`: parts fused along the output rows, one alpha per row).
"""
from __future__ import annotations

import fnmatch
import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from . import nvfp4
from .packed import PackedFP8, PackedNVFP4
from .safetensors_io import SafeTensors, save_file


@dataclass
class QuantConfig:
    algo: str = ""                       # "NVFP4" | "FP8" | "" (not quantised)
    kv_cache_algo: str = ""
    group_size: int = 16
    exclude: List[str] = field(default_factory=list)

    def excluded(self, module: str) -> bool:
        return any(fnmatch.fnmatch(module, pat) or module == pat or module.endswith("." + pat.lstrip("*."))
                   for pat in self.exclude)


def read_quant_config(model_dir: str) -> QuantConfig:
    """`hf_quant_config.json`, else `config.json`'s `quantization_config`; an empty config when neither names an algo."""
    p = os.path.join(model_dir, "hf_quant_config.json") if os.path.isdir(model_dir) else ""
    if p and os.path.exists(p):
        q = json.load(open(p)).get("quantization", {})
        return QuantConfig(str(q.get("quant_algo") or "").upper(), str(q.get("kv_cache_quant_algo") or "").upper(),
                           int(q.get("group_size") or 16), list(q.get("exclude_modules") or []))
    p = os.path.join(model_dir, "config.json") if os.path.isdir(model_dir) else ""
    if p and os.path.exists(p):
        q = json.load(open(p)).get("quantization_config") or {}
        algo = str(q.get("quant_algo") or q.get("quant_method") or "").upper()
        if algo in ("NVFP4", "FP8"):
            return QuantConfig(algo, str(q.get("kv_cache_quant_algo") or "").upper(), int(q.get("group_size") or 16),
                               list(q.get("exclude_modules") or q.get("ignore") or []))
    return QuantConfig()


def _scalar(st: SafeTensors, name: str, default: Optional[float] = None) -> float:
    if not st.has(name):
        if default is None:
            raise KeyError(f"{name} is missing")
        return default
    return float(st.get(name).float().reshape(-1)[0])


def module_algo(st: SafeTensors, base: str) -> str:
    """What the tensors of one module say: "NVFP4" (packed codes + block scales + tensor scale), "FP8" (e4m3 weight +
    scalar scale) or "" (a plain weight). A uint8 weight without its scales is refused: it is code bytes, not values."""
    if not st.has(base + ".weight"):
        return ""
    dt = st.dtype(base + ".weight")
    if st.has(base + ".weight_scale_2") and st.has(base + ".weight_scale"):
        return "NVFP4"
    if dt == torch.float8_e4m3fn:
        if not st.has(base + ".weight_scale"):
            raise ValueError(f"{base}.weight is float8 but {base}.weight_scale is missing")
        return "FP8"
    if dt == torch.uint8:
        raise ValueError(f"{base}.weight is uint8 (packed codes) but its weight_scale / weight_scale_2 are missing")
    return ""


def load_packed(st: SafeTensors, base: str):
    """One quantised module as a packed linear ([out, in] surface); None for a plain weight."""
    algo = module_algo(st, base)
    if algo == "NVFP4":
        codes = st.get(base + ".weight")
        sc = st.get(base + ".weight_scale")
        n, kb = codes.shape
        if tuple(sc.shape) != (n, kb * 2 // nvfp4.BLOCK):
            raise ValueError(f"{base}: weight_scale {tuple(sc.shape)} does not match weight {tuple(codes.shape)}")
        alpha = torch.full((n,), _scalar(st, base + ".weight_scale_2"), dtype=torch.float32)
        return PackedNVFP4(codes.contiguous(), sc.view(torch.uint8).contiguous(), alpha, _scalar(st, base + ".input_scale", 0.0))
    if algo == "FP8":
        codes = st.get(base + ".weight").view(torch.uint8)
        alpha = torch.full((codes.shape[0],), _scalar(st, base + ".weight_scale"), dtype=torch.float32)
        return PackedFP8(codes.contiguous(), alpha, _scalar(st, base + ".input_scale", 0.0))
    return None


# ---- writer (synthetic checkpoints for tests and benchmarks) ---------------------------------------------------

def quantize_module(w: torch.Tensor, algo: str) -> Dict[str, torch.Tensor]:
    """The tensors ModelOpt would store for one `[out, in]` linear."""
    if algo == "NVFP4":
        q = nvfp4.quantize(w)
        return {"weight": q.packed, "weight_scale": q.scales, "weight_scale_2": torch.tensor(q.global_scale, dtype=torch.float32),
                "input_scale": torch.tensor(float(w.abs().max()) / (6.0 * 448.0) + 1e-8, dtype=torch.float32)}
    if algo == "FP8":
        s = float(w.abs().max()) / 448.0 or 1.0
        return {"weight": (w.float() / s).to(torch.float8_e4m3fn), "weight_scale": torch.tensor(s, dtype=torch.float32),
                "input_scale": torch.tensor(1.0, dtype=torch.float32)}
    raise ValueError(algo)


def save_checkpoint(tensors: Dict[str, torch.Tensor], model_dir: str, algo: str, quantised: List[str],
                    exclude: Optional[List[str]] = None) -> None:
    """Write `model.safetensors` + `hf_quant_config.json`: the modules named in `quantised` (names without `.weight`)
    are stored in ModelOpt's layout for `algo`, everything else as given."""
    os.makedirs(model_dir, exist_ok=True)
    out: Dict[str, torch.Tensor] = {}
    qset = set(quantised)
    for name, t in tensors.items():
        base = name[:-len(".weight")] if name.endswith(".weight") else None
        if base is not None and base in qset:
            for k, v in quantize_module(t, algo).items():
                out[f"{base}.{k}"] = v
        else:
            out[name] = t
    save_file(out, os.path.join(model_dir, "model.safetensors"), {"format": "pt"})
    with open(os.path.join(model_dir, "hf_quant_config.json"), "w") as f:
        json.dump({"producer": {"name": "modelopt"},
                   "quantization": {"quant_algo": algo, "kv_cache_quant_algo": None, "group_size": 16,
                                    "exclude_modules": exclude or []}}, f)
