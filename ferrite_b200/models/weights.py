"""Weight naming, seeded random initialisation and tensor-parallel slicing.

Layout choices that differ from the reference's per-projection tensors (`crates/fe-model/src/model.rs:406-460`):
projections that share an input are stored fused, so a decode step issues one weight-streaming kernel per input:

* GDN  `in_proj`  rows = [q | k | v | z | b | a]            (`gdn_in_dim` x hidden)
* attn `in_proj`  rows = [per q head: q, gate] | k | v      (`attn_in_dim` x hidden)
* MLP  `gate_up`  rows = [gate | up]                        (2*inter x hidden)

RMSNorm weights are stored zero-centred (effective weight 1 + w), the GDN gated-norm weight as used
(reference convention, the design notes of `crates/fe-xe`, lines 56-57).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config import ModelConfig
from ..formats.packed import cat_rows

Weights = Dict[str, torch.Tensor]


def layer_weight_shapes(cfg: ModelConfig, i: int) -> Dict[str, tuple]:
    h = cfg.hidden
    p = f"l{i}."
    out: Dict[str, tuple] = {p + "input_norm": (h,), p + "post_norm": (h,)}
    kind = cfg.layer_kinds[i]
    if kind == "gdn":
        out[p + "in_proj"] = (cfg.gdn_in_dim, h)
        out[p + "conv_w"] = (cfg.conv_dim, cfg.conv_k)
        out[p + "A_log"] = (cfg.lin_v_heads,)
        out[p + "dt_bias"] = (cfg.lin_v_heads,)
        out[p + "gnorm_w"] = (cfg.lin_dv,)
        out[p + "out_proj"] = (h, cfg.lin_v_heads * cfg.lin_dv)
    elif kind == "attn":
        out[p + "in_proj"] = (cfg.attn_in_dim, h)
        out[p + "q_norm"] = (cfg.head_dim,)
        out[p + "k_norm"] = (cfg.head_dim,)
        out[p + "out_proj"] = (h, cfg.n_q * cfg.head_dim)
    else:  # mla
        qd = cfg.nope_head_dim + cfg.rope_head_dim
        out[p + "q_a"] = (cfg.q_lora, h)
        out[p + "q_a_norm"] = (cfg.q_lora,)
        out[p + "q_b"] = (cfg.n_q * qd, cfg.q_lora)
        out[p + "kv_a"] = (cfg.kv_lora + cfg.rope_head_dim, h)
        out[p + "kv_a_norm"] = (cfg.kv_lora,)
        out[p + "kv_b"] = (cfg.n_q * (cfg.nope_head_dim + cfg.v_head_dim), cfg.kv_lora)
        out[p + "out_proj"] = (h, cfg.n_q * cfg.v_head_dim)
    if cfg.is_moe(i):
        e, ei = cfg.n_experts, cfg.expert_inter
        out[p + "router"] = (e, h)
        if cfg.router == "sigmoid_group":
            out[p + "router_bias"] = (e,)
        out[p + "experts_gate_up"] = (e, 2 * ei, h)
        out[p + "experts_down"] = (e, h, ei)
        if cfg.n_shared:
            out[p + "shared_gate_up"] = (2 * ei * cfg.n_shared, h)
            out[p + "shared_down"] = (h, ei * cfg.n_shared)
            out[p + "shared_gate"] = (1, h)
    else:
        inter = cfg.dense_inter if (cfg.n_experts > 0 and cfg.dense_inter) else cfg.inter
        out[p + "gate_up"] = (2 * inter, h)
        out[p + "down"] = (h, inter)
    return out


def weight_shapes(cfg: ModelConfig) -> Dict[str, tuple]:
    out: Dict[str, tuple] = {"embed": (cfg.vocab, cfg.hidden), "final_norm": (cfg.hidden,)}
    if not cfg.tie_embeddings:
        out["lm_head"] = (cfg.vocab, cfg.hidden)
    for i in range(cfg.n_layers):
        out.update(layer_weight_shapes(cfg, i))
    return out


_F32_NAMES = ("A_log", "dt_bias", "router_bias")


def init_weights(cfg: ModelConfig, seed: int = 0, dtype=torch.float32, device="cpu", std: float = 0.02, post=None) -> Weights:
    """Seeded N(0, std) weights for every tensor of the architecture. The GDN gated-norm weight is drawn
    around one (it multiplies directly); all other norm weights are zero-centred offsets. `post(name, tensor)` may
    replace a tensor as soon as it is drawn (a quantised engine packs the big ones at once, so a model that only fits
    packed never exists unpacked)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w: Weights = {}
    for name, shape in weight_shapes(cfg).items():
        t = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std
        if name.endswith("gnorm_w"):
            t = t + 1.0
        keep32 = name.endswith(_F32_NAMES)
        t = t if keep32 else t.to(dtype)
        w[name] = post(name, t) if post is not None else t
    return w


# ---- tensor-parallel slicing ---------------------------------------------------------------------------

def _rows(t: torch.Tensor, lo: int, hi: int) -> torch.Tensor:
    return t[lo:hi]


def shard_weights(cfg: ModelConfig, w: Weights, rank: int, world: int) -> Weights:
    """Slice whole-model weights for one tensor-parallel rank. Column-parallel projections keep whole heads
    (KV heads are replicated when world > n_kv), row-parallel ones keep the matching input columns; norms,
    embeddings and the router are replicated, `lm_head` is split by vocabulary rows. Split table modelled
    on the reference's (`TP2.md:36-50`, `crates/fe-exl3/src/tp.rs`). Packed quantised linears (`formats/packed.py`)
    are cut the same way as dense ones: row and column slices move code and scale bytes, nothing is re-quantised."""
    if world == 1:
        return dict(w)
    out: Weights = {}
    h = cfg.hidden
    for name, t in w.items():
        base = name.split(".")[-1]
        li = int(name[1:name.index(".")]) if name.startswith("l") and "." in name else -1
        kind = cfg.layer_kinds[li] if li >= 0 else ""
        if name == "lm_head":
            per = (cfg.vocab + world - 1) // world
            out[name] = t[rank * per:min(cfg.vocab, (rank + 1) * per)].contiguous()
        elif base == "in_proj" and kind == "gdn":
            nk, nv, dk, dv = cfg.lin_k_heads, cfg.lin_v_heads, cfg.lin_dk, cfg.lin_dv
            nkr, nvr = nk // world, nv // world
            o = 0
            parts = []
            for n_heads, per_rank, d in ((nk, nkr, dk), (nk, nkr, dk), (nv, nvr, dv), (nv, nvr, dv)):
                parts.append(t[o + rank * per_rank * d:o + (rank + 1) * per_rank * d])
                o += n_heads * d
            for _ in range(2):  # b, a
                parts.append(t[o + rank * nvr:o + (rank + 1) * nvr])
                o += nv
            out[name] = cat_rows(parts)
        elif base == "conv_w":
            nk, nv, dk, dv = cfg.lin_k_heads, cfg.lin_v_heads, cfg.lin_dk, cfg.lin_dv
            nkr, nvr = nk // world, nv // world
            o = 0
            parts = []
            for n_heads, per_rank, d in ((nk, nkr, dk), (nk, nkr, dk), (nv, nvr, dv)):
                parts.append(t[o + rank * per_rank * d:o + (rank + 1) * per_rank * d])
                o += n_heads * d
            out[name] = cat_rows(parts)
        elif base in ("A_log", "dt_bias"):
            nvr = cfg.lin_v_heads // world
            out[name] = t[rank * nvr:(rank + 1) * nvr].contiguous()
        elif base == "in_proj" and kind == "attn":
            hd = cfg.head_dim
            qw = hd * (2 if cfg.attn_gate else 1)
            nqr = cfg.n_q // world
            nkvr = max(1, cfg.n_kv // world)
            kv_first = (rank * cfg.n_kv) // world if cfg.n_kv >= world else (rank * cfg.n_kv) // world
            q = t[rank * nqr * qw:(rank + 1) * nqr * qw]
            ko = cfg.n_q * qw
            vo = ko + cfg.n_kv * hd
            k = t[ko + kv_first * hd:ko + (kv_first + nkvr) * hd]
            v = t[vo + kv_first * hd:vo + (kv_first + nkvr) * hd]
            out[name] = cat_rows([q, k, v])
        elif base == "out_proj":
            if kind == "gdn":
                per = cfg.lin_v_heads // world * cfg.lin_dv
            elif kind == "attn":
                per = cfg.n_q // world * cfg.head_dim
            else:
                per = cfg.n_q // world * cfg.v_head_dim
            out[name] = t[:, rank * per:(rank + 1) * per].contiguous()
        elif base in ("gate_up", "shared_gate_up"):
            inter = t.shape[0] // 2
            per = inter // world
            out[name] = cat_rows([t[rank * per:(rank + 1) * per], t[inter + rank * per:inter + (rank + 1) * per]])
        elif base in ("down", "shared_down"):
            per = t.shape[1] // world
            out[name] = t[:, rank * per:(rank + 1) * per].contiguous()
        elif base in ("experts_gate_up", "experts_down"):
            # expert parallel: whole experts per rank
            per = cfg.n_experts // world
            out[name] = t[rank * per:(rank + 1) * per].contiguous()
        elif base == "q_b":
            per = t.shape[0] // world
            out[name] = t[rank * per:(rank + 1) * per].contiguous()
        elif base == "kv_b":
            per = t.shape[0] // world
            out[name] = t[rank * per:(rank + 1) * per].contiguous()
        else:
            out[name] = t
    return out
