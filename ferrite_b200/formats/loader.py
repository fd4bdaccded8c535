"""Checkpoint -> engine weights. Reads Hugging Face safetensors checkpoints of the hybrid (Gated DeltaNet + gated
attention) family and this package's own flat layout, fusing the projections that share an input
(`models/weights.py`). EXL3 tensors found in the checkpoint are reconstructed to dense weights at load; NVFP4
(ModelOpt) tensors are kept packed. Reference: `Weights::load` (`crates/fe-model/src/model.rs:773-953`),
`attach_fp4` (`:959-1114`), `reconstruct_bf16` (`kernels/k-exl3/src/recon.rs`)."""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from ..config import ModelConfig
from ..models.weights import weight_shapes
from . import exl3
from .safetensors_io import SafeTensors, save_file


def save_native(weights: Dict[str, torch.Tensor], path: str, cfg: Optional[ModelConfig] = None) -> None:
    """Write engine-layout weights as one safetensors file (plus the config as metadata)."""
    meta = {"format": "ferrite_b200-native"}
    if cfg is not None:
        meta["config"] = cfg.to_json()
    save_file({k: v for k, v in weights.items() if isinstance(v, torch.Tensor)}, path, meta)


def _dense(st: SafeTensors, base: str, dtype) -> torch.Tensor:
    """A linear weight [out, in] whatever its storage: plain `.weight`, or an EXL3 triple reconstructed here."""
    if st.has(base + ".weight"):
        return st.get(base + ".weight").to(dtype)
    if st.has(base + ".trellis"):
        return exl3.load_tensor(st, base).weight(torch.float32).t().contiguous().to(dtype)    # EXL3 stores [in, out]
    raise KeyError(f"{base}: no .weight and no .trellis")


def load_model_weights(model_dir: str, cfg: ModelConfig, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    st = SafeTensors(model_dir)
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
                # grouped per key head: [q dk | k dk | v rep*dv | z rep*dv], and b|a grouped the same way
                qkvz = _dense(st, la + "in_proj_qkvz", dtype).view(nk, 2 * dk + 2 * rep * dv, cfg.hidden)
                ba = _dense(st, la + "in_proj_ba", dtype).view(nk, 2 * rep, cfg.hidden)
                qq, kk = qkvz[:, :dk].reshape(nk * dk, -1), qkvz[:, dk:2 * dk].reshape(nk * dk, -1)
                vv = qkvz[:, 2 * dk:2 * dk + rep * dv].reshape(nv * dv, -1)
                zz = qkvz[:, 2 * dk + rep * dv:].reshape(nv * dv, -1)
                bb, aa = ba[:, :rep].reshape(nv, -1), ba[:, rep:].reshape(nv, -1)
            else:
                qkv = _dense(st, la + "in_proj_qkv", dtype)
                qq, kk, vv = qkv[:nk * dk], qkv[nk * dk:2 * nk * dk], qkv[2 * nk * dk:]
                zz = _dense(st, la + "in_proj_z", dtype)
                bb, aa = _dense(st, la + "in_proj_b", dtype), _dense(st, la + "in_proj_a", dtype)
            w[p + "in_proj"] = torch.cat([qq, kk, vv, zz, bb, aa], 0).contiguous()
            w[p + "conv_w"] = st.get(la + "conv1d.weight").reshape(cfg.conv_dim, cfg.conv_k).to(dtype)
            w[p + "A_log"] = st.get(la + "A_log").float()
            w[p + "dt_bias"] = st.get(la + "dt_bias").float()
            w[p + "gnorm_w"] = st.get(la + "norm.weight").to(dtype)
            w[p + "out_proj"] = _dense(st, la + "out_proj", dtype)
        else:
            sa = q + "self_attn."
            w[p + "in_proj"] = torch.cat([_dense(st, sa + "q_proj", dtype), _dense(st, sa + "k_proj", dtype),
                                          _dense(st, sa + "v_proj", dtype)], 0).contiguous()
            w[p + "q_norm"] = st.get(sa + "q_norm.weight").to(dtype)
            w[p + "k_norm"] = st.get(sa + "k_norm.weight").to(dtype)
            w[p + "out_proj"] = _dense(st, sa + "o_proj", dtype)
        m = q + "mlp."
        w[p + "gate_up"] = torch.cat([_dense(st, m + "gate_proj", dtype), _dense(st, m + "up_proj", dtype)], 0).contiguous()
        w[p + "down"] = _dense(st, m + "down_proj", dtype)
    st.close()
    return w
