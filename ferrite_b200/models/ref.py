"""Plain PyTorch fp32 reference of every model family: the oracle for the CUDA kernels and the CPU path.

Numerics follow the reference's written conventions (the design notes of `crates/fe-xe`, lines 44-60): RMSNorm with (1 + w),
per-head q/k norm and partial RoPE with a sigmoid output gate on attention, Gated DeltaNet with a causal
depthwise conv (tap 0 = oldest), `g = exp(-exp(A_log) * softplus(a + dt_bias))`, `beta = sigmoid(b)`,
`S = S g; delta = (v - S^T k) beta; S += k (x) delta; y = S^T q`, gated RMSNorm `rmsnorm(y) * w * silu(z)`.
It processes one sequence token by token, holding its own KV / conv / recurrent state, so it is slow and
obviously right; the CPU oracles of the reference play the same role (`crates/fe-dsc/src/refmodel.rs`,
`crates/fe-exl3/src/cpu.rs`).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from ..config import ModelConfig
from .weights import Weights


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, centred: bool = True) -> torch.Tensor:
    x = x.float()
    r = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return x * r * ((1.0 + w.float()) if centred else w.float())


def rope_tables(positions: torch.Tensor, rotary_dim: int, theta: float) -> tuple:
    half = rotary_dim // 2
    inv = theta ** (-torch.arange(half, dtype=torch.float64) / half)
    ang = positions.double()[:, None] * inv[None, :]
    return ang.cos().float(), ang.sin().float()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int) -> torch.Tensor:
    """x: [rows, heads, hd]; rotate-half pairing (i, i + rotary_dim/2) over the first rotary_dim dims."""
    half = rotary_dim // 2
    a, b = x[..., :half], x[..., half:rotary_dim]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., rotary_dim:]], -1)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 20, x, torch.log1p(torch.exp(torch.clamp(x, max=20.0))))


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    i = gu.shape[-1] // 2
    return F.silu(gu[..., :i]) * gu[..., i:]


def route(cfg: ModelConfig, logits: torch.Tensor, bias: Optional[torch.Tensor]):
    """Top-k routing. softmax: softmax over experts, top-k (ties to the lower id), renormalise.
    sigmoid_group: scores = sigmoid(logits); choice by scores + bias restricted to the best `topk_groups`
    groups (group score = sum of its top-2 biased scores); weights = picked scores / sum * route_scale
    (reference routers: `kernels/k-fnext/src/fast.rs:393`, `kernels/k-ds/src/moe.rs:11`)."""
    logits = logits.float()
    if cfg.router == "softmax":
        p = torch.softmax(logits, -1)
        val, idx = torch.sort(p, dim=-1, descending=True, stable=True)
        val, idx = val[..., :cfg.top_k], idx[..., :cfg.top_k]
        return idx, val / val.sum(-1, keepdim=True) * cfg.route_scale
    s = torch.sigmoid(logits)
    sb = s + (bias.float() if bias is not None else 0.0)
    n, e = sb.shape
    g = cfg.n_groups
    grp = sb.view(n, g, e // g)
    gscore = grp.topk(2, -1).values.sum(-1)
    _, gi = torch.sort(gscore, dim=-1, descending=True, stable=True)
    gmask = torch.zeros(n, g, dtype=torch.bool)
    gmask.scatter_(1, gi[:, :cfg.topk_groups], True)
    masked = torch.where(gmask[:, :, None].expand(n, g, e // g).reshape(n, e), sb, torch.full_like(sb, float("-inf")))
    _, idx = torch.sort(masked, dim=-1, descending=True, stable=True)
    idx = idx[:, :cfg.top_k]
    val = s.gather(1, idx)
    return idx, val / (val.sum(-1, keepdim=True) + 1e-20) * cfg.route_scale


class RefState:
    def __init__(self, cfg: ModelConfig):
        self.cfg = cfg
        self.pos = 0
        self.k: List[List[torch.Tensor]] = [[] for _ in range(cfg.n_layers)]
        self.v: List[List[torch.Tensor]] = [[] for _ in range(cfg.n_layers)]
        self.conv = [torch.zeros(cfg.conv_dim, cfg.conv_k - 1) for _ in range(cfg.n_layers)]
        self.rec = [torch.zeros(cfg.lin_v_heads, cfg.lin_dk, cfg.lin_dv) for _ in range(cfg.n_layers)]

    def clone(self) -> "RefState":
        s = RefState(self.cfg)
        s.pos = self.pos
        s.k = [list(x) for x in self.k]
        s.v = [list(x) for x in self.v]
        s.conv = [x.clone() for x in self.conv]
        s.rec = [x.clone() for x in self.rec]
        return s


class RefModel:
    """fp32 oracle. `forward(tokens, state)` appends the tokens to the sequence held by `state` and returns
    logits [len(tokens), vocab] (and the per-layer hidden taps when asked)."""

    def __init__(self, cfg: ModelConfig, weights: Weights):
        self.cfg = cfg
        self.w = {k: v.detach().float().cpu() for k, v in weights.items()}

    def new_state(self) -> RefState:
        return RefState(self.cfg)

    # ---- mixers ------------------------------------------------------------------------------------
    def _gdn(self, i: int, x: torch.Tensor, st: RefState) -> torch.Tensor:
        c, w = self.cfg, self.w
        p = f"l{i}."
        nk, nv, dk, dv = c.lin_k_heads, c.lin_v_heads, c.lin_dk, c.lin_dv
        proj = w[p + "in_proj"] @ x
        qkv, z, b, a = torch.split(proj, [c.conv_dim, nv * dv, nv, nv])
        win = torch.cat([st.conv[i], qkv[:, None]], 1)             # [conv_dim, conv_k], tap 0 oldest
        st.conv[i] = win[:, 1:].clone()
        qkv = F.silu((win * w[p + "conv_w"]).sum(1))
        q, k, v = torch.split(qkv, [nk * dk, nk * dk, nv * dv])
        q = q.view(nk, dk)
        k = k.view(nk, dk)
        v = v.view(nv, dv)
        q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + c.eps) / math.sqrt(dk)
        k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + c.eps)
        rep = nv // nk
        q = q.repeat_interleave(rep, 0)
        k = k.repeat_interleave(rep, 0)
        g = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(a + w[p + "dt_bias"]))
        beta = torch.sigmoid(b)
        S = st.rec[i] * g[:, None, None]
        kv = torch.einsum("hkv,hk->hv", S, k)
        delta = (v - kv) * beta[:, None]
        S = S + torch.einsum("hk,hv->hkv", k, delta)
        st.rec[i] = S
        y = torch.einsum("hkv,hk->hv", S, q)
        y = rmsnorm(y, w[p + "gnorm_w"], c.eps, centred=False) * F.silu(z.view(nv, dv))
        return w[p + "out_proj"] @ y.reshape(-1)

    def _attn(self, i: int, x: torch.Tensor, st: RefState) -> torch.Tensor:
        c, w = self.cfg, self.w
        p = f"l{i}."
        hd, nq, nkv = c.head_dim, c.n_q, c.n_kv
        proj = w[p + "in_proj"] @ x
        qd = c.attn_q_dim
        qg = proj[:qd].view(nq, -1)
        q = qg[:, :hd]
        gate = qg[:, hd:] if c.attn_gate else None
        k = proj[qd:qd + nkv * hd].view(nkv, hd)
        v = proj[qd + nkv * hd:].view(nkv, hd)
        q = rmsnorm(q, w[p + "q_norm"], c.eps)
        k = rmsnorm(k, w[p + "k_norm"], c.eps)
        cos, sin = rope_tables(torch.tensor([st.pos]), c.rotary_dim, c.rope_theta)
        q = apply_rope(q[None], cos, sin, c.rotary_dim)[0]
        k = apply_rope(k[None], cos, sin, c.rotary_dim)[0]
        st.k[i].append(k)
        st.v[i].append(v)
        K = torch.stack(st.k[i], 0)                                # [T, nkv, hd]
        V = torch.stack(st.v[i], 0)
        grp = nq // nkv
        qh = q.view(nkv, grp, hd)
        s = torch.einsum("kgd,tkd->kgt", qh, K) / math.sqrt(hd)
        pr = torch.softmax(s, -1)
        o = torch.einsum("kgt,tkd->kgd", pr, V).reshape(nq, hd)
        if gate is not None:
            o = o * torch.sigmoid(gate)
        return w[p + "out_proj"] @ o.reshape(-1)

    def _mla(self, i: int, x: torch.Tensor, st: RefState) -> torch.Tensor:
        c, w = self.cfg, self.w
        p = f"l{i}."
        nq, dn, dr, dvh = c.n_q, c.nope_head_dim, c.rope_head_dim, c.v_head_dim
        qa = rmsnorm(w[p + "q_a"] @ x, w[p + "q_a_norm"], c.eps)
        q = (w[p + "q_b"] @ qa).view(nq, dn + dr)
        kva = w[p + "kv_a"] @ x
        lat = rmsnorm(kva[:c.kv_lora], w[p + "kv_a_norm"], c.eps)
        kr = kva[c.kv_lora:]
        cos, sin = rope_tables(torch.tensor([st.pos]), dr, c.rope_theta)
        qr = apply_rope(q[None, :, dn:], cos, sin, dr)[0]
        kr = apply_rope(kr[None, None, :], cos, sin, dr)[0, 0]
        st.k[i].append(lat)
        st.v[i].append(kr)
        L = torch.stack(st.k[i], 0)                                # [T, kv_lora]
        R = torch.stack(st.v[i], 0)                                # [T, dr]
        kvb = w[p + "kv_b"].view(nq, dn + dvh, c.kv_lora)
        kn = torch.einsum("hdl,tl->thd", kvb[:, :dn], L)
        vv = torch.einsum("hdl,tl->thd", kvb[:, dn:], L)
        s = (torch.einsum("hd,thd->ht", q[:, :dn], kn) + torch.einsum("hd,td->ht", qr, R)) / math.sqrt(dn + dr)
        pr = torch.softmax(s, -1)
        o = torch.einsum("ht,thd->hd", pr, vv)
        return w[p + "out_proj"] @ o.reshape(-1)

    def _ffn(self, i: int, x: torch.Tensor) -> torch.Tensor:
        c, w = self.cfg, self.w
        p = f"l{i}."
        if not c.is_moe(i):
            return w[p + "down"] @ swiglu(w[p + "gate_up"] @ x)
        idx, wt = route(c, (w[p + "router"] @ x)[None], w.get(p + "router_bias"))
        out = torch.zeros_like(x)
        for e, g in zip(idx[0].tolist(), wt[0].tolist()):          # fixed pair order: rank of the pick
            out = out + g * (w[p + "experts_down"][e] @ swiglu(w[p + "experts_gate_up"][e] @ x))
        if c.n_shared:
            sh = w[p + "shared_down"] @ swiglu(w[p + "shared_gate_up"] @ x)
            if c.router == "softmax":
                sh = sh * torch.sigmoid(w[p + "shared_gate"] @ x)
            out = out + sh
        return out

    # ---- whole model -------------------------------------------------------------------------------
    def forward(self, tokens, st: RefState, return_hidden: bool = False):
        c, w = self.cfg, self.w
        logits, taps = [], []
        head = w["embed"] if c.tie_embeddings else w["lm_head"]
        for t in list(tokens):
            x = w["embed"][int(t)].clone()
            tap = []
            for i, kind in enumerate(c.layer_kinds):
                h = rmsnorm(x, w[f"l{i}.input_norm"], c.eps)
                if kind == "gdn":
                    x = x + self._gdn(i, h, st)
                elif kind == "attn":
                    x = x + self._attn(i, h, st)
                else:
                    x = x + self._mla(i, h, st)
                x = x + self._ffn(i, rmsnorm(x, w[f"l{i}.post_norm"], c.eps))
                if i in c.tap_layers:
                    tap.append(x.clone())
            st.pos += 1
            logits.append(head @ rmsnorm(x, w["final_norm"], c.eps))
            taps.append(tap)
        out = torch.stack(logits, 0)
        return (out, taps) if return_hidden else out

    @torch.no_grad()
    def generate(self, prompt, n_new: int) -> List[int]:
        st = self.new_state()
        lg = self.forward(prompt, st)
        out = []
        tok = int(lg[-1].argmax())
        for _ in range(n_new):
            out.append(tok)
            lg = self.forward([tok], st)
            tok = int(lg[-1].argmax())
        return out
