"""GGUF checkpoints -> engine configuration and weights, and a writer for synthetic ones.

Tensor names and metadata keys are llama.cpp's for the hybrid (Gated DeltaNet + gated attention) dense and MoE families,
the ones the reference's MoE engines read (`crates/fe-fnext/src/config.rs:55-120` metadata, `crates/fe-fnext/src/engine.rs`
and `fast/mod.rs` tensor names; `crates/fe-dsc/src/tensors.rs`):

    token_embd.weight  output_norm.weight  output.weight
    blk.N.attn_norm.weight  blk.N.post_attention_norm.weight
    attention layers:  blk.N.attn_q / attn_k / attn_v / attn_output .weight,  attn_q_norm / attn_k_norm .weight
    GDN layers:        blk.N.attn_qkv.weight (q | k | v)  attn_gate.weight (z)  ssm_beta.weight  ssm_alpha.weight
                       ssm_conv1d.weight  ssm_a  ssm_dt.bias  ssm_norm.weight  ssm_out.weight
    dense MLP:         blk.N.ffn_gate / ffn_up / ffn_down .weight
    MoE:               blk.N.ffn_gate_inp.weight (router)  ffn_gate_exps / ffn_up_exps / ffn_down_exps .weight
                       ffn_gate_shexp / ffn_up_shexp / ffn_down_shexp .weight  ffn_gate_inp_shexp.weight

Conventions of the conversion that produced such files: RMSNorm weights are stored as multipliers (this engine keeps
them zero-centred, so 1 is subtracted at load), `ssm_a` is -exp(A_log). Quantised 2-D tensors stay in their block
format (`PackedGGUF`): decode rows run the dequantising GEMV on the checkpoint's own blocks. Expert stacks are
dequantised at load (or re-quantised to NVFP4 by the engine's `weight_dtype`).
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Optional

import numpy as np
import torch

from ..config import ModelConfig
from . import gguf as G
from .packed import PackedGGUF, cat_rows


def config_from_gguf(g: G.Gguf, base: Optional[ModelConfig] = None) -> ModelConfig:
    """ModelConfig from the `<arch>.*` metadata keys (fields without a key keep the values of `base`)."""
    arch = str(g.meta.get("general.architecture", ""))
    m = lambda k, d=None: g.meta.get(f"{arch}.{k}", d)
    c = base or ModelConfig()
    kw = {}
    def put(field, key, cast=int):
        v = m(key)
        if v is not None and hasattr(c, field):
            kw[field] = cast(v)
    put("n_layers", "block_count"); put("hidden", "embedding_length"); put("inter", "feed_forward_length")
    put("n_q", "attention.head_count"); put("n_kv", "attention.head_count_kv"); put("head_dim", "attention.key_length")
    put("rotary_dim", "rope.dimension_count"); put("rope_theta", "rope.freq_base", float)
    put("eps", "attention.layer_norm_rms_epsilon", float)
    put("conv_k", "ssm.conv_kernel"); put("lin_dk", "ssm.state_size"); put("lin_dv", "ssm.state_size")
    put("lin_k_heads", "ssm.group_count"); put("lin_v_heads", "ssm.time_step_rank")
    put("n_experts", "expert_count"); put("top_k", "expert_used_count"); put("expert_inter", "expert_feed_forward_length")
    if "token_embd.weight" in g.tensors:
        kw["vocab"] = g.tensors["token_embd.weight"].shape[0]
    kw["tie_embeddings"] = "output.weight" not in g.tensors
    if m("expert_shared_feed_forward_length"):
        kw["n_shared"] = max(1, int(m("expert_shared_feed_forward_length")) // max(1, int(m("expert_feed_forward_length", 1))))
    return dataclasses.replace(c, **{k: v for k, v in kw.items() if hasattr(c, k)})


def _linear(g: G.Gguf, name: str, dtype, dense: bool):
    t = g.tensors[name]
    if dense or t.type_name in ("F32", "F16", "BF16") or len(t.shape) != 2:
        return g.get(name, dtype)
    rows, cols = t.shape
    return PackedGGUF(torch.from_numpy(g.raw(name).copy()).view(rows, -1), t.type_id, cols)


def load_gguf_weights(path: str, cfg: ModelConfig, dtype=torch.bfloat16, dense: bool = False) -> Dict[str, torch.Tensor]:
    g = G.Gguf(path)
    w: Dict[str, torch.Tensor] = {}
    vec = lambda n: g.get(n, torch.float32)
    norm = lambda n: (vec(n) - 1.0).to(dtype)                       # stored as multipliers, kept zero-centred
    w["embed"] = g.get("token_embd.weight", dtype)
    w["final_norm"] = norm("output_norm.weight")
    if not cfg.tie_embeddings:
        w["lm_head"] = _linear(g, "output.weight", dtype, dense) if "output.weight" in g.tensors else w["embed"]
    for i, kind in enumerate(cfg.layer_kinds):
        p, q = f"l{i}.", f"blk.{i}."
        w[p + "input_norm"] = norm(q + "attn_norm.weight")
        w[p + "post_norm"] = norm(q + "post_attention_norm.weight")
        lin = lambda n: _linear(g, q + n + ".weight", dtype, dense)
        if kind == "gdn":
            w[p + "in_proj"] = cat_rows([lin("attn_qkv"), lin("attn_gate"), lin("ssm_beta"), lin("ssm_alpha")])
            w[p + "conv_w"] = g.get(q + "ssm_conv1d.weight", dtype).reshape(cfg.conv_dim, cfg.conv_k)
            w[p + "A_log"] = torch.log(-vec(q + "ssm_a").reshape(-1))
            w[p + "dt_bias"] = vec(q + "ssm_dt.bias").reshape(-1)
            w[p + "gnorm_w"] = vec(q + "ssm_norm.weight").to(dtype)
            w[p + "out_proj"] = lin("ssm_out")
        else:
            w[p + "in_proj"] = cat_rows([lin("attn_q"), lin("attn_k"), lin("attn_v")])
            w[p + "q_norm"] = norm(q + "attn_q_norm.weight")
            w[p + "k_norm"] = norm(q + "attn_k_norm.weight")
            w[p + "out_proj"] = lin("attn_output")
        if cfg.is_moe(i):
            w[p + "router"] = g.get(q + "ffn_gate_inp.weight", dtype)
            if (q + "exp_probs_b.bias") in g.tensors:
                w[p + "router_bias"] = vec(q + "exp_probs_b.bias")
            w[p + "experts_gate_up"] = torch.cat([g.get(q + "ffn_gate_exps.weight", dtype), g.get(q + "ffn_up_exps.weight", dtype)], 1)
            w[p + "experts_down"] = g.get(q + "ffn_down_exps.weight", dtype)
            if cfg.n_shared:
                w[p + "shared_gate_up"] = cat_rows([lin("ffn_gate_shexp"), lin("ffn_up_shexp")])
                w[p + "shared_down"] = lin("ffn_down_shexp")
                w[p + "shared_gate"] = g.get(q + "ffn_gate_inp_shexp.weight", dtype).reshape(1, -1)
        else:
            w[p + "gate_up"] = cat_rows([lin("ffn_gate"), lin("ffn_up")])
            w[p + "down"] = lin("ffn_down")
    g.close()
    return w


_ENC = {"Q8_0": (G.quantize_q8_0, 32), "Q4_0": (G.quantize_q4_0, 32)}


def export_gguf(weights: Dict[str, torch.Tensor], cfg: ModelConfig, path: str, qtype: str = "Q8_0", arch: str = "hybrid") -> None:
    """Write dense engine-layout weights as a GGUF file under the names above: 2-D projections in `qtype` (Q8_0 / Q4_0;
    F32 when the row length is not a multiple of the block), vectors and embeddings in F32. For tests and synthetic
    benchmarks: the inverse of `load_gguf_weights`."""
    out = {}

    def put(name, t, quant=False):
        a = t.detach().float().cpu().numpy()
        if quant and a.ndim >= 2 and a.shape[-1] % _ENC[qtype][1] == 0:
            out[name] = (_ENC[qtype][0](a.reshape(-1)), G.TYPE_ID[qtype], list(a.shape))
        else:
            out[name] = (np.ascontiguousarray(a).view(np.uint8).reshape(-1), 0, list(a.shape))

    mult = lambda t: t.float() + 1.0
    put("token_embd.weight", weights["embed"])
    put("output_norm.weight", mult(weights["final_norm"]))
    if not cfg.tie_embeddings and "lm_head" in weights:
        put("output.weight", weights["lm_head"], True)
    nk, nv, dk, dv = cfg.lin_k_heads, cfg.lin_v_heads, cfg.lin_dk, cfg.lin_dv
    for i, kind in enumerate(cfg.layer_kinds):
        p, q = f"l{i}.", f"blk.{i}."
        put(q + "attn_norm.weight", mult(weights[p + "input_norm"]))
        put(q + "post_attention_norm.weight", mult(weights[p + "post_norm"]))
        ip = weights[p + "in_proj"]
        if kind == "gdn":
            o1, o2 = 2 * nk * dk + nv * dv, 2 * nk * dk + 2 * nv * dv
            put(q + "attn_qkv.weight", ip[:o1], True); put(q + "attn_gate.weight", ip[o1:o2], True)
            put(q + "ssm_beta.weight", ip[o2:o2 + nv], True); put(q + "ssm_alpha.weight", ip[o2 + nv:], True)
            put(q + "ssm_conv1d.weight", weights[p + "conv_w"])
            put(q + "ssm_a", -torch.exp(weights[p + "A_log"].float()))
            put(q + "ssm_dt.bias", weights[p + "dt_bias"])
            put(q + "ssm_norm.weight", weights[p + "gnorm_w"])
            put(q + "ssm_out.weight", weights[p + "out_proj"], True)
        else:
            nq_rows = cfg.n_q * cfg.head_dim * (2 if cfg.attn_gate else 1)
            kv_rows = cfg.n_kv * cfg.head_dim
            put(q + "attn_q.weight", ip[:nq_rows], True); put(q + "attn_k.weight", ip[nq_rows:nq_rows + kv_rows], True)
            put(q + "attn_v.weight", ip[nq_rows + kv_rows:], True)
            put(q + "attn_q_norm.weight", mult(weights[p + "q_norm"])); put(q + "attn_k_norm.weight", mult(weights[p + "k_norm"]))
            put(q + "attn_output.weight", weights[p + "out_proj"], True)
        if cfg.is_moe(i):
            put(q + "ffn_gate_inp.weight", weights[p + "router"])
            if p + "router_bias" in weights:
                put(q + "exp_probs_b.bias", weights[p + "router_bias"])
            gu = weights[p + "experts_gate_up"]
            h = gu.shape[1] // 2
            put(q + "ffn_gate_exps.weight", gu[:, :h], True); put(q + "ffn_up_exps.weight", gu[:, h:], True)
            put(q + "ffn_down_exps.weight", weights[p + "experts_down"], True)
            if cfg.n_shared:
                sg = weights[p + "shared_gate_up"]
                put(q + "ffn_gate_shexp.weight", sg[:sg.shape[0] // 2], True); put(q + "ffn_up_shexp.weight", sg[sg.shape[0] // 2:], True)
                put(q + "ffn_down_shexp.weight", weights[p + "shared_down"], True)
                put(q + "ffn_gate_inp_shexp.weight", weights[p + "shared_gate"].reshape(-1))
        else:
            gu = weights[p + "gate_up"]
            put(q + "ffn_gate.weight", gu[:gu.shape[0] // 2], True); put(q + "ffn_up.weight", gu[gu.shape[0] // 2:], True)
            put(q + "ffn_down.weight", weights[p + "down"], True)
    meta = {"general.architecture": arch, f"{arch}.block_count": cfg.n_layers, f"{arch}.embedding_length": cfg.hidden,
            f"{arch}.feed_forward_length": cfg.inter, f"{arch}.attention.head_count": cfg.n_q,
            f"{arch}.attention.head_count_kv": cfg.n_kv, f"{arch}.attention.key_length": cfg.head_dim,
            f"{arch}.rope.dimension_count": cfg.rotary_dim, f"{arch}.rope.freq_base": float(cfg.rope_theta),
            f"{arch}.attention.layer_norm_rms_epsilon": float(cfg.eps), f"{arch}.ssm.conv_kernel": cfg.conv_k,
            f"{arch}.ssm.state_size": cfg.lin_dk, f"{arch}.ssm.group_count": cfg.lin_k_heads,
            f"{arch}.ssm.time_step_rank": cfg.lin_v_heads, f"{arch}.ssm.inner_size": cfg.lin_v_heads * cfg.lin_dv}
    if cfg.n_experts:
        meta.update({f"{arch}.expert_count": cfg.n_experts, f"{arch}.expert_used_count": cfg.top_k,
                     f"{arch}.expert_feed_forward_length": cfg.expert_inter,
                     f"{arch}.expert_shared_feed_forward_length": cfg.expert_inter * cfg.n_shared})
    G.write_gguf(path, meta, out)
