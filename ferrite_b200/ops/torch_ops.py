"""Plain PyTorch statement of every device op, with the same signatures as `cuda_ops.CudaOps`.

Two uses: it is the fp32 oracle each CUDA kernel test compares against, and it is the op set the engine runs
on when it is built on a CPU device (the plumbing configuration). It mutates the same paged KV cache and
state tensors the CUDA kernels do.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from .extras import TorchExtras


def _softplus(x):
    return torch.where(x > 20, x, torch.log1p(torch.exp(torch.clamp(x, max=20.0))))


class TorchOps(TorchExtras):
    name = "torch"

    def __init__(self, device="cpu", dtype=torch.float32):
        self.device = torch.device(device)
        self.dtype = dtype
        self.launches = 0

    # ---- rows ------------------------------------------------------------------------------------
    def embed(self, table, ids):
        return table[ids.long()].to(self.dtype)

    def rmsnorm(self, x, w, eps, centred=True, res=None):
        """Returns (normed, x') with x' = x + res when res is given (the folded residual add)."""
        if res is not None:
            x = (x.float() + res.float()).to(x.dtype)
        xf = x.float()
        r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        wf = w.float() + 1.0 if centred else w.float()
        return (xf * r * wf).to(self.dtype), x

    def linear(self, x, w, norm_w=None, eps=1e-6, res=None, swiglu=False, out_f32=False):
        """y = x W^T with optional RMSNorm(1+w) prologue, SwiGLU (W = [gate|up]) or residual epilogue."""
        if hasattr(w, "dense"):
            w = w.dense                      # quantised weight: the oracle multiplies by its dequantised values
        xf = x.float()
        if norm_w is not None:
            r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
            xf = (xf * r * (1.0 + norm_w.float())).to(x.dtype).float()
        y = xf @ w.float().t()
        if swiglu:
            i = y.shape[-1] // 2
            y = F.silu(y[:, :i]) * y[:, i:]
        if res is not None:
            y = y + res.float()
        return y if out_f32 else y.to(self.dtype)

    def silu_mul(self, gu):
        i = gu.shape[-1] // 2
        return (F.silu(gu[:, :i].float()) * gu[:, i:].float()).to(self.dtype)

    def gated_norm(self, y, proj, z_off, w, heads, dv, eps):
        yf = y.float().view(-1, heads, dv)
        z = proj[:, z_off:z_off + heads * dv].float().view(-1, heads, dv)
        r = torch.rsqrt(yf.pow(2).mean(-1, keepdim=True) + eps)
        return (yf * r * w.float() * F.silu(z)).reshape(-1, heads * dv).to(self.dtype)

    # ---- attention ---------------------------------------------------------------------------------
    def attn_prep(self, proj, q_norm, k_norm, inv_freq, row_slot, row_pos, block_table, k_cache, v_cache, kv_block,
                  nq, nkv, hd, rot, gated, eps, kv_scale=None, row_cpos=None, hrot=False, kv_bits=None):
        """With `kv_scale` the cache rows take the values a quantised cache would return (the oracle keeps them
        dequantised in its float cache): e4m3 with one scale per (token, kv head) = amax / 448, or 4- / 6-bit integer
        codes with one scale per 32 elements (`kv_bits`; 4 when the scale tensor has group scales and nothing is said).
        `hrot`: queries and keys are rotated by the orthonormal Walsh-Hadamard matrix of the head width first."""
        T = proj.shape[0]
        qw = hd * (2 if gated else 1)
        qg = proj[:, :nq * qw].float().view(T, nq, qw)
        q = qg[..., :hd]
        k = proj[:, nq * qw:nq * qw + nkv * hd].float().view(T, nkv, hd)
        v = proj[:, nq * qw + nkv * hd:nq * qw + 2 * nkv * hd].view(T, nkv, hd)

        def norm(x, w):
            return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + w.float())

        q, k = norm(q, q_norm), norm(k, k_norm)
        ang = row_pos.float()[:, None] * inv_freq.float()[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        half = rot // 2

        def rope(x):
            a, b = x[..., :half], x[..., half:rot]
            return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., rot:]], -1)

        q, k = rope(q), rope(k)
        if hrot:
            H = torch.ones(1, 1, device=q.device)
            while H.shape[0] < hd:
                H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
            H = H / math.sqrt(hd)
            q, k = q @ H, k @ H
        pos = row_pos.long() if row_cpos is None else row_cpos.long()     # trees: stored by row index, rotated by depth
        blk = block_table[row_slot.long(), pos // kv_block].long()
        off = pos % kv_block
        if kv_scale is not None:
            def fq(x):
                sc = (x.abs().amax(-1, keepdim=True) / 448.0)
                sc = torch.where(sc > 0, sc, torch.ones_like(sc))
                return (x / sc).to(torch.float8_e4m3fn).float() * sc

            def fq4(x):
                # 4-bit cache: groups of 32 elements, scale = amax / 7, codes in -8..7 (round half to even)
                g = x.reshape(*x.shape[:-1], hd // 32, 32)
                sc = g.abs().amax(-1, keepdim=True) / 7.0
                sc = torch.where(sc > 0, sc, torch.ones_like(sc))
                return (torch.round(g / sc).clamp(-8, 7) * sc).reshape(x.shape)
            def fq6(x):
                # 6-bit cache: groups of 32 elements, scale = amax / 31, codes in -32..31
                g = x.reshape(*x.shape[:-1], hd // 32, 32)
                sc = g.abs().amax(-1, keepdim=True) / 31.0
                sc = torch.where(sc > 0, sc, torch.ones_like(sc))
                return (torch.round(g / sc).clamp(-32, 31) * sc).reshape(x.shape)
            if kv_scale.shape[-1] != 2:
                fq = fq6 if kv_bits == 6 else fq4
            k, v = fq(k.float()), fq(v.float())
        k_cache[blk, off] = k.to(k_cache.dtype)
        v_cache[blk, off] = v.to(v_cache.dtype)
        return q.to(self.dtype)

    def attention(self, q, proj, k_cache, v_cache, row_slot, row_kvlen, block_table, kv_block, nq, nkv, hd, gated,
                  row_base=None, row_mask=None, nsplit=1, kv_scale=None, segs=None):
        T = q.shape[0]
        out = torch.zeros(T, nq, hd, dtype=torch.float32, device=q.device)
        grp = nq // nkv
        for t in range(T):
            L = int(row_kvlen[t])
            slot = int(row_slot[t])
            pos = torch.arange(L, device=q.device)
            blk = block_table[slot, pos // kv_block].long()
            K = k_cache[blk, pos % kv_block].float()            # [L, nkv, hd]
            V = v_cache[blk, pos % kv_block].float()
            qh = q[t].float().view(nkv, grp, hd)
            s = torch.einsum("kgd,tkd->kgt", qh, K) / math.sqrt(hd)
            if row_base is not None and row_mask is not None:
                base, mask = int(row_base[t]), int(row_mask[t])
                vis = torch.tensor([(p < base) or ((mask >> (p - base)) & 1) == 1 for p in range(L)], device=q.device)
                s = s.masked_fill(~vis[None, None, :], float("-inf"))
            p = torch.softmax(s, -1)
            out[t] = torch.einsum("kgt,tkd->kgd", p, V).reshape(nq, hd)
        if gated:
            gate = proj[:, :nq * 2 * hd].float().view(T, nq, 2 * hd)[..., hd:]
            out = out * torch.sigmoid(gate)
        return out.reshape(T, nq * hd).to(self.dtype)

    def attention_prefill(self, q, proj, k_cache, v_cache, seg_slot, seg_row0, seg_nrows, seg_pos0, block_table,
                          kv_block, nq, nkv, hd, gated, max_rows, row_slot=None, row_kvlen=None, kv_scale=None,
                          max_kvlen=None):
        if row_slot is None:
            T = q.shape[0]
            row_slot = torch.zeros(T, dtype=torch.int32, device=q.device)
            row_kvlen = torch.zeros(T, dtype=torch.int32, device=q.device)
            for s in range(len(seg_slot)):
                n, r0 = int(seg_nrows[s]), int(seg_row0[s])
                row_slot[r0:r0 + n] = int(seg_slot[s])
                row_kvlen[r0:r0 + n] = torch.arange(int(seg_pos0[s]) + 1, int(seg_pos0[s]) + n + 1, dtype=torch.int32)
        return self.attention(q, proj, k_cache, v_cache, row_slot, row_kvlen, block_table, kv_block, nq, nkv, hd, gated)

    # ---- gated delta net ---------------------------------------------------------------------------
    def gdn_conv(self, proj, conv_w, conv_state, seg_slot, seg_row0, seg_nrows, conv_dim):
        T = proj.shape[0]
        out = torch.zeros(T, conv_dim, dtype=self.dtype, device=proj.device)
        ck = conv_w.shape[1]
        for s in range(len(seg_slot)):
            n, r0, slot = int(seg_nrows[s]), int(seg_row0[s]), int(seg_slot[s])
            if n <= 0:
                continue
            x = torch.cat([conv_state[slot].float(), proj[r0:r0 + n, :conv_dim].float()], 0)     # [ck-1+n, C]
            win = x.unfold(0, ck, 1)                                                              # [n, C, ck]
            out[r0:r0 + n] = F.silu((win * conv_w.float()[None]).sum(-1)).to(self.dtype)
        return out

    def gdn_conv_tree(self, proj, conv_w, conv_state, seg_slot, seg_row0, seg_nrows, conv_dim, row_parent):
        """Verify-tree rows: the conv window of a row is its ancestors (nearest last), then the slot's saved tail."""
        T = proj.shape[0]
        out = torch.zeros(T, conv_dim, dtype=self.dtype, device=proj.device)
        ck = conv_w.shape[1]
        wf = conv_w.float()
        for s in range(len(seg_slot)):
            n, r0, slot = int(seg_nrows[s]), int(seg_row0[s]), int(seg_slot[s])
            tail = conv_state[slot].float()                                                       # [ck-1, C], oldest first
            for r in range(n):
                acc = wf[:, ck - 1] * proj[r0 + r, :conv_dim].float()
                i = r
                for j in range(ck - 2, -1, -1):
                    i = int(row_parent[r0 + i]) if i >= 0 else i - 1
                    x = proj[r0 + i, :conv_dim].float() if i >= 0 else tail[ck - 1 + i]
                    acc = acc + wf[:, j] * x
                out[r0 + r] = F.silu(acc).to(self.dtype)
        return out

    def gdn_rec_tree(self, qkv, proj, rec_state, A_log, dt_bias, seg_slot, seg_row0, seg_nrows, row_parent, row_flags, nk,
                     nv, dk, dv, eps):
        """Verify-tree rows (read-only): each row applies one delta-rule step to the state its parent left."""
        T = qkv.shape[0]
        conv_dim = 2 * nk * dk + nv * dv
        y = torch.zeros(T, nv * dv, dtype=torch.float32, device=qkv.device)
        rep = nv // nk
        for s in range(len(seg_slot)):
            n, r0, slot = int(seg_nrows[s]), int(seg_row0[s]), int(seg_slot[s])
            states = {-1: rec_state[slot].float().clone()}
            for r in range(n):
                S = states[int(row_parent[r0 + r])]
                x = qkv[r0 + r].float()
                q = x[:nk * dk].view(nk, dk)
                k = x[nk * dk:2 * nk * dk].view(nk, dk)
                v = x[2 * nk * dk:].view(nv, dv)
                q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + eps) / math.sqrt(dk)
                k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + eps)
                q, k = q.repeat_interleave(rep, 0), k.repeat_interleave(rep, 0)
                b = proj[r0 + r, conv_dim + nv * dv:conv_dim + nv * dv + nv].float()
                a = proj[r0 + r, conv_dim + nv * dv + nv:conv_dim + nv * dv + 2 * nv].float()
                g = torch.exp(-torch.exp(A_log.float()) * _softplus(a + dt_bias.float()))
                S = S * g[:, None, None]
                delta = (v - torch.einsum("hkv,hk->hv", S, k)) * torch.sigmoid(b)[:, None]
                S = S + torch.einsum("hk,hv->hkv", k, delta)
                y[r0 + r] = torch.einsum("hkv,hk->hv", S, q).reshape(-1)
                states[r] = S
        return y

    def gdn_rec(self, qkv, proj, rec_state, conv_state, A_log, dt_bias, seg_slot, seg_row0, seg_nrows, nk, nv, dk, dv,
                eps, commit=True, chunked=False, max_rows=None):
        T = qkv.shape[0]
        conv_dim = 2 * nk * dk + nv * dv
        y = torch.zeros(T, nv * dv, dtype=torch.float32, device=qkv.device)
        rep = nv // nk
        ck1 = conv_state.shape[1]
        for s in range(len(seg_slot)):
            n, r0, slot = int(seg_nrows[s]), int(seg_row0[s]), int(seg_slot[s])
            if n <= 0:
                continue
            S = rec_state[slot].float().clone()                  # [nv, dk, dv]
            for r in range(r0, r0 + n):
                x = qkv[r].float()
                q = x[:nk * dk].view(nk, dk)
                k = x[nk * dk:2 * nk * dk].view(nk, dk)
                v = x[2 * nk * dk:].view(nv, dv)
                q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + eps) / math.sqrt(dk)
                k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + eps)
                q, k = q.repeat_interleave(rep, 0), k.repeat_interleave(rep, 0)
                b = proj[r, conv_dim + nv * dv:conv_dim + nv * dv + nv].float()
                a = proj[r, conv_dim + nv * dv + nv:conv_dim + nv * dv + 2 * nv].float()
                g = torch.exp(-torch.exp(A_log.float()) * _softplus(a + dt_bias.float()))
                beta = torch.sigmoid(b)
                S = S * g[:, None, None]
                kv = torch.einsum("hkv,hk->hv", S, k)
                delta = (v - kv) * beta[:, None]
                S = S + torch.einsum("hk,hv->hkv", k, delta)
                y[r] = torch.einsum("hkv,hk->hv", S, q).reshape(-1)
            if commit:
                rec_state[slot] = S.to(rec_state.dtype)
                x = torch.cat([conv_state[slot].float(), proj[r0:r0 + n, :conv_dim].float()], 0)
                conv_state[slot] = x[-ck1:].to(conv_state.dtype)
        return y

    # ---- multi-head latent attention (absorbed form) ----------------------------------------------------
    def mla_prep(self, q, kva, norm_w, w_uk_t, inv_freq, row_slot, row_pos, block_table, cache, kv_block, nq, dn, L, R, eps):
        """Latent RMSNorm + key RoPE into the paged cache [blocks, kv_block, L + R]; returns the absorbed queries
        [T, nq, L + R] = [q_nope W_uk | rope(q_rope)]."""
        T = q.shape[0]
        q3 = q.reshape(T, nq, dn + R).float()
        kf = kva.float()
        lat = kf[:, :L] * torch.rsqrt(kf[:, :L].pow(2).mean(-1, keepdim=True) + eps) * (1.0 + norm_w.float())
        ang = row_pos.float()[:, None] * inv_freq.float()[None, :]
        cos, sin = ang.cos(), ang.sin()
        half = R // 2

        def rope(v, c, s):
            a, b = v[..., :half], v[..., half:]
            return torch.cat([a * c - b * s, b * c + a * s], -1)
        kr = rope(kf[:, L:], cos, sin)
        qr = rope(q3[..., dn:], cos[:, None, :], sin[:, None, :])
        rows = torch.cat([lat, kr], -1).to(cache.dtype)
        for t in range(T):
            slot, pos = int(row_slot[t]), int(row_pos[t])
            cache[int(block_table[slot, pos // kv_block]), pos % kv_block] = rows[t]
        qn = torch.einsum("thd,hld->thl", q3[..., :dn], w_uk_t.float())
        return torch.cat([qn, qr], -1).to(self.dtype)

    def mla_attention(self, qabs, cache, row_slot, row_kvlen, block_table, kv_block, nq, L, R, scale, nsplit=1):
        T = qabs.shape[0]
        out = torch.zeros(T, nq, L, dtype=torch.float32, device=qabs.device)
        for t in range(T):
            n, slot = int(row_kvlen[t]), int(row_slot[t])
            nb = (n + kv_block - 1) // kv_block
            keys = cache[block_table[slot, :nb].long()].reshape(-1, L + R)[:n].float()
            s = (qabs[t].float() @ keys.t()) * scale
            out[t] = torch.softmax(s, -1) @ keys[:, :L]
        return out.to(self.dtype)

    def mla_out(self, ol, w_uv):
        """ol [T, nq, L] latent-space outputs -> [T, nq * dv] through the per-head value up-projection [nq, dv, L]."""
        return torch.einsum("thl,hvl->thv", ol.float(), w_uv.float()).reshape(ol.shape[0], -1).to(self.dtype)

    def ffn(self, x, w_gu, w_down, norm_w, eps, res):
        """Dense FFN block: down(SwiGLU(gate|up(norm(x)))) + res."""
        return self.linear(self.linear(x, w_gu, norm_w=norm_w, eps=eps, swiglu=True), w_down, res=res)

    def head_linear(self, x, W, out=None):
        """y[t, h, :] = W[h] x[t, h, :] for x [T, heads, K], W [heads, N, K]."""
        y = torch.einsum("thk,hnk->thn", x.float(), W.float()).to(self.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y

    # ---- mixture of experts ---------------------------------------------------------------------------
    def moe_route(self, logits, bias, mode, top_k, n_groups, topk_groups, scale):
        from ..config import ModelConfig
        from ..models.ref import route
        c = ModelConfig(router="softmax" if mode == 0 else "sigmoid_group", top_k=top_k, n_groups=n_groups,
                        topk_groups=topk_groups, route_scale=scale, n_experts=logits.shape[1])
        idx, w = route(c, logits.float().cpu(), None if bias is None else bias.cpu())
        return idx.to(torch.int32).to(logits.device), w.float().to(logits.device)

    def experts_dense(self, w, which: int):
        from .qweight import ExpertsFP4
        return w.dequantize(torch.float32) if isinstance(w, ExpertsFP4) else w

    def moe_experts(self, h, ids, wts, w_gu, w_down, e_lo, e_hi, shared=None, shared_gate=None, res=None, out_f32=False):
        w_gu, w_down = self.experts_dense(w_gu, 0), self.experts_dense(w_down, 1)
        T, K = ids.shape
        out = torch.zeros(T, h.shape[1], dtype=torch.float32, device=h.device)
        hf = h.float()
        for t in range(T):
            for k in range(K):
                e = int(ids[t, k])
                if e < e_lo or e >= e_hi:
                    continue
                gu = w_gu[e - e_lo].float() @ hf[t]
                i = gu.shape[0] // 2
                a = (F.silu(gu[:i]) * gu[i:]).to(self.dtype).float()
                out[t] += float(wts[t, k]) * (w_down[e - e_lo].float() @ a)
        if shared is not None:
            g = torch.sigmoid(shared_gate.float()).reshape(-1, 1) if shared_gate is not None else 1.0
            out = out + shared.float() * g
        if res is not None:
            out = out + res.float()
        return out if out_f32 else out.to(self.dtype)

    # ---- selection ---------------------------------------------------------------------------------
    def hc_norm(self, res, w, eps):
        rows, hc, d = res.shape
        x = res.reshape(rows * hc, d).float()
        inv = torch.rsqrt(x.pow(2).mean(-1) + eps)
        wg = w.float()[torch.arange(rows * hc) % w.shape[0]]
        return (x * inv[:, None] * wg).to(self.dtype), inv

    def hc_mix(self, res, inv, w, gate):
        rows, hc, d = res.shape
        return (res.float() * inv.view(rows, hc, 1) * w.float()[None, :hc] * torch.sigmoid(gate.float())).mean(1)

    def hc_combine(self, res, out, inj):
        res += out.float()[:, None, :] * 2.0 * torch.sigmoid(inj.float())[:, :res.shape[1], None]
        return res

    def dynconv(self, x, coef, base, group, blk, res=None):
        T, H = x.shape
        G = H // group
        xf, cf, bf = x.float(), coef.float(), base.float().view(2, H)
        w0 = bf[0][None] + cf[:, :G].repeat_interleave(group, 1)
        w1 = bf[1][None] + cf[:, G:2 * G].repeat_interleave(group, 1)
        prev = torch.cat([torch.zeros(1, H), xf[:-1]], 0)
        inside = (torch.arange(T) % blk != 0).float()[:, None]
        y = w0 * xf + inside * w1 * prev
        if res is not None:
            res.copy_((res.float() + y.to(res.dtype).float()).to(res.dtype))
            return res
        return y.to(self.dtype)

    def topk16_merge(self, vals, ids):
        W, rows, _ = vals.shape
        v = vals.permute(1, 0, 2).reshape(rows, W * 16)
        i = ids.permute(1, 0, 2).reshape(rows, W * 16)
        # descending by value, ties to the lower id
        order = sorted
        ov = torch.empty(rows, 16)
        oi = torch.empty(rows, 16, dtype=torch.int32)
        for r in range(rows):
            pairs = order(zip(v[r].tolist(), i[r].tolist()), key=lambda p: (-p[0], p[1]))[:16]
            ov[r] = torch.tensor([p[0] for p in pairs])
            oi[r] = torch.tensor([p[1] for p in pairs], dtype=torch.int32)
        return ov, oi

    def draft_select(self, vals, ids, gate, a_cb, b_cb, anchor):
        out, pred = [], int(anchor)
        for r in range(vals.shape[0]):
            sc = vals[r].float() + ((a_cb[pred].float() * gate[r].float())[None] * b_cb[ids[r].long()].float()).sum(-1)
            pred = int(ids[r][int(sc.argmax())])
            out.append(pred)
        return torch.tensor(out, dtype=torch.int32)

    def argmax(self, logits):
        lf = logits.float()
        finite = torch.isfinite(lf).all(-1)
        return lf.argmax(-1).to(torch.int32), finite

    def status(self) -> int:
        return 0
