"""Checkpoint -> engine weights. Reads Hugging Face safetensors checkpoints of the hybrid (Gated DeltaNet + gated
attention) family and this package's own flat layout, fusing the projections that share an input
(`models/weights.py`). Quantised modules stay packed (`formats/packed.py`): EXL3 triples (`.trellis/.suh/.svh`) and
ModelOpt NVFP4 / FP8 modules (`.weight` + `.weight_scale` [+ `.weight_scale_2`]) come back as `Packed*` objects that
the engine slices per rank and hands to the low-bit kernels; `dense=True` dequantises them at load instead
(the fp32 oracle and bf16 serving of a quantised checkpoint). A uint8 `.weight` without its scales is refused.
Reference: `Weights::load` (`crates/fe-model/src/model.rs:773-953`), `attach_fp4` (`:959-1114`), `reconstruct_bf16`
(`kernels/k-exl3/src/recon.rs`), `HostLinear::load_sliced` (`crates/fe-fp4/src/lib.rs:305`)."""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from ..config import ModelConfig
from ..models.weights import weight_shapes
from . import exl3, modelopt
from .packed import PackedEXL3, PackedLinear, cat_rows, dense_of
from .safetensors_io import SafeTensors, save_file


def save_native(weights: Dict[str, torch.Tensor], path: str, cfg: Optional[ModelConfig] = None) -> None:
    """Write engine-layout weights as one safetensors file (plus the config as metadata)."""
    meta = {"format": "ferrite_b200-native"}
    if cfg is not None:
        meta["config"] = cfg.to_json()
    save_file({k: v for k, v in weights.items() if isinstance(v, torch.Tensor)}, path, meta)


def _linear(st: SafeTensors, base: str, dtype, dense: bool):
    """A linear weight [out, in] whatever its storage: a plain `.weight`, a ModelOpt NVFP4 / FP8 module or an EXL3
    triple. Quantised storage comes back packed unless `dense` asks for the dequantised values."""
    if st.has(base + ".trellis"):
        p = PackedEXL3(exl3.load_tensor(st, base))                   # EXL3 stores [in, out]
        return p.dequantize(torch.float32).to(dtype) if dense else p
    if st.has(base + ".weight"):
        p = modelopt.load_packed(st, base)                           # raises on code bytes without scales
        if p is None:
            return st.get(base + ".weight").to(dtype)
        return p.dequantize(torch.float32).to(dtype) if dense else p
    raise KeyError(f"{base}: no .weight and no .trellis")


def _take(w, index: torch.Tensor):
    """Rows of a linear in a new order (regrouping of fused checkpoint tensors). EXL3 tensors are stored per
    projection and are never regrouped."""
    if isinstance(w, torch.Tensor):
        return w[index]
    if hasattr(w, "take"):
        return w.take(index)
    raise TypeError(f"{type(w).__name__} rows cannot be regrouped")


def load_model_weights(model_dir: str, cfg: ModelConfig, dtype=torch.bfloat16, dense: bool = False) -> Dict[str, torch.Tensor]:
    st = SafeTensors(model_dir)
    _dense = lambda st_, base, dt: _linear(st_, base, dt, dense)
    names = set(st.names())
    if "embed" in names and "final_norm" in names:                    # native layout
        return {k: st.get(k) for k in weight_shapes(cfg) if st.has(k)}
    pre = "model.language_model." if any(n.startswith("model.language_model.") for n in names) else "model."
    w: Dict[str, torch.Tensor] = {}
    w["embed"] = st.get(pre + "embed_tokens.weight").to(dtype)
    w["final_norm"] = st.get(pre + "norm.weight").to(dtype)
    if not cfg.tie_embeddings:
        w["lm_head"] = _dense(st, "lm_head", dtype) if (st.has("lm_head.weight") or st.has("lm_head.trellis")) else w["embed"]
    nk, nv, dk, dv = cfg.lin_k_heads, cfg.lin_v_heads, cfg.lin_dk, cfg.lin_dv
    rep = nv // max(nk, 1)
    for i, kind in enumerate(cfg.layer_kinds):
        p, q = f"l{i}.", f"{pre}layers.{i}."
        w[p + "input_norm"] = st.get(q + "input_layernorm.weight").to(dtype)
        w[p + "post_norm"] = st.get(q + "post_attention_layernorm.weight").to(dtype)
        if kind == "gdn":
            la = q + "linear_attn."
            if st.has(la + "in_proj_qkvz.weight") or st.has(la + "in_proj_qkvz.trellis"):
                # grouped per key head: [q dk | k dk | v rep*dv | z rep*dv], and b|a grouped the same way; the regrouping
                # is a row gather, which packed storage follows byte for byte
                qkvz = _dense(st, la + "in_proj_qkvz", dtype)
                ba = _dense(st, la + "in_proj_ba", dtype)
                per = 2 * dk + 2 * rep * dv
                ix = torch.arange(nk * per).view(nk, per)
                qq, kk = _take(qkvz, ix[:, :dk].reshape(-1)), _take(qkvz, ix[:, dk:2 * dk].reshape(-1))
                vv = _take(qkvz, ix[:, 2 * dk:2 * dk + rep * dv].reshape(-1))
                zz = _take(qkvz, ix[:, 2 * dk + rep * dv:].reshape(-1))
                ib = torch.arange(nk * 2 * rep).view(nk, 2 * rep)
                bb, aa = _take(ba, ib[:, :rep].reshape(-1)), _take(ba, ib[:, rep:].reshape(-1))
            else:
                qkv = _dense(st, la + "in_proj_qkv", dtype)
                qq, kk, vv = qkv[:nk * dk], qkv[nk * dk:2 * nk * dk], qkv[2 * nk * dk:]
                zz = _dense(st, la + "in_proj_z", dtype)
                bb, aa = _dense(st, la + "in_proj_b", dtype), _dense(st, la + "in_proj_a", dtype)
            w[p + "in_proj"] = cat_rows([qq, kk, vv, zz, bb, aa])
            w[p + "conv_w"] = st.get(la + "conv1d.weight").reshape(cfg.conv_dim, cfg.conv_k).to(dtype)
            w[p + "A_log"] = st.get(la + "A_log").float()
            w[p + "dt_bias"] = st.get(la + "dt_bias").float()
            w[p + "gnorm_w"] = st.get(la + "norm.weight").to(dtype)
            w[p + "out_proj"] = _dense(st, la + "out_proj", dtype)
        else:
            sa = q + "self_attn."
            w[p + "in_proj"] = cat_rows([_dense(st, sa + "q_proj", dtype), _dense(st, sa + "k_proj", dtype),
                                         _dense(st, sa + "v_proj", dtype)])
            w[p + "q_norm"] = st.get(sa + "q_norm.weight").to(dtype)
            w[p + "k_norm"] = st.get(sa + "k_norm.weight").to(dtype)
            w[p + "out_proj"] = _dense(st, sa + "o_proj", dtype)
        m = q + "mlp."
        w[p + "gate_up"] = cat_rows([_dense(st, m + "gate_proj", dtype), _dense(st, m + "up_proj", dtype)])
        w[p + "down"] = _dense(st, m + "down_proj", dtype)
    st.close()
    return w


def export_hf(weights: Dict[str, torch.Tensor], cfg: ModelConfig) -> Dict[str, torch.Tensor]:
    """Engine-layout dense weights under Hugging Face names (the inverse of `load_model_weights` for the separate
    `in_proj_qkv` / `in_proj_z` / `in_proj_b` / `in_proj_a` form): what the synthetic-checkpoint writers start from."""
    pre = "model."
    out: Dict[str, torch.Tensor] = {pre + "embed_tokens.weight": weights["embed"], pre + "norm.weight": weights["final_norm"]}
    if not cfg.tie_embeddings and "lm_head" in weights:
        out["lm_head.weight"] = weights["lm_head"]
    nk, nv, dk, dv = cfg.lin_k_heads, cfg.lin_v_heads, cfg.lin_dk, cfg.lin_dv
    for i, kind in enumerate(cfg.layer_kinds):
        p, q = f"l{i}.", f"{pre}layers.{i}."
        out[q + "input_layernorm.weight"] = weights[p + "input_norm"]
        out[q + "post_attention_layernorm.weight"] = weights[p + "post_norm"]
        ip = weights[p + "in_proj"]
        if kind == "gdn":
            la = q + "linear_attn."
            o1, o2 = 2 * nk * dk + nv * dv, 2 * nk * dk + 2 * nv * dv
            out[la + "in_proj_qkv.weight"] = ip[:o1]
            out[la + "in_proj_z.weight"] = ip[o1:o2]
            out[la + "in_proj_b.weight"] = ip[o2:o2 + nv]
            out[la + "in_proj_a.weight"] = ip[o2 + nv:]
            out[la + "conv1d.weight"] = weights[p + "conv_w"].reshape(cfg.conv_dim, 1, cfg.conv_k)
            out[la + "A_log"] = weights[p + "A_log"]
            out[la + "dt_bias"] = weights[p + "dt_bias"]
            out[la + "norm.weight"] = weights[p + "gnorm_w"]
            out[la + "out_proj.weight"] = weights[p + "out_proj"]
        else:
            sa = q + "self_attn."
            nq_rows = cfg.n_q * cfg.head_dim * (2 if cfg.attn_gate else 1)
            out[sa + "q_proj.weight"] = ip[:nq_rows]
            out[sa + "k_proj.weight"] = ip[nq_rows:nq_rows + cfg.n_kv * cfg.head_dim]
            out[sa + "v_proj.weight"] = ip[nq_rows + cfg.n_kv * cfg.head_dim:]
            out[sa + "q_norm.weight"] = weights[p + "q_norm"]
            out[sa + "k_norm.weight"] = weights[p + "k_norm"]
            out[sa + "o_proj.weight"] = weights[p + "out_proj"]
        m = q + "mlp."
        gu = weights[p + "gate_up"]
        out[m + "gate_proj.weight"] = gu[:gu.shape[0] // 2]
        out[m + "up_proj.weight"] = gu[gu.shape[0] // 2:]
        out[m + "down_proj.weight"] = weights[p + "down"]
    return {k: v.contiguous() for k, v in out.items()}
