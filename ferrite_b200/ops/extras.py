"""Ops of model families beyond this repo's presets: sparse-attention selection (latent compressor, indexer scores, exact
top-k, candidate masks, selected-block tables), the Markov / confidence drafting heads and the Engram gate over
hyper-connection streams. `TorchExtras` states every op in plain fp32 PyTorch (the oracle of the GPU tests and the CPU
path); `CudaExtras` calls the kernels of `csrc/sparse_index.cu`, `csrc/dspark.cu` and `csrc/hyperconn.cu`. Both are mixed
into the op classes (`TorchOps`, `CudaOps`).

Reference: `kernels/k-ds/src/index.rs`, `kernels/k-fnext/src/fast.rs:157-247`, `kernels/k-dspark/src/lib.rs`,
`kernels/k-engram/src/lib.rs`.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def _argmax_order(v: torch.Tensor) -> torch.Tensor:
    """Index of the best entry per row in the order NaN first, then the larger value, then the lower index."""
    nan = torch.isnan(v)
    key = torch.where(nan, torch.full_like(v, float("inf")), v)
    anynan = nan.any(-1)
    first_nan = nan.float().argmax(-1)
    best = key.argmax(-1)                      # torch.argmax returns the first maximal index
    return torch.where(anynan, first_nan, best)


class TorchExtras:
    # ---- Engram gate ------------------------------------------------------------------------------------
    def engram_gate(self, h, kv, qk, eps):
        """h [rows, hc, d]; kv [rows, (hc + 1) d] (summed, bf16) or fp32 partials [world, rows, (hc + 1) d]: hc keys then
        the value; qk [hc, d]. out = h + sigmoid(ssqrt(<h qk, key> rstd(h) rstd(key) / sqrt(d))) * value."""
        rows, hc, d = h.shape
        if kv.dim() == 3:
            acc = kv[0].float().clone()
            for k in range(1, kv.shape[0]):
                acc = acc + kv[k].float()
            kv = acc.to(torch.bfloat16)
        kvf = kv.float().view(rows, hc + 1, d)
        key, val = kvf[:, :hc], kvf[:, hc]
        x = h.float()
        rstd = torch.rsqrt(x.pow(2).mean(-1) + eps) * torch.rsqrt(key.pow(2).mean(-1) + eps)
        dot = (x * qk.float()[None] * key).sum(-1) * rstd / math.sqrt(d)
        mag = dot.abs().clamp_min(1e-6).sqrt()
        gate = torch.sigmoid(torch.where(dot < 0, -mag, mag))
        return (x + gate[..., None] * val[:, None, :]).to(h.dtype)

    # ---- compressor -------------------------------------------------------------------------------------
    def comp_step(self, tail, kvc, sc, row_slot, row_pos, ratio):
        """Stash the rows' (kvc, sc) in the slot rings `tail` [slots, ring_len, 2 dim], then emit for rows that close a
        group of `ratio` tokens the channel-wise softmax(sc)-weighted sum of the group's kvc (zeros for other rows)."""
        rows, dim = kvc.shape
        ring = tail.shape[1]
        for r in range(rows):
            s, p = int(row_slot[r]), int(row_pos[r])
            tail[s, p % ring, :dim] = kvc[r].float()
            tail[s, p % ring, dim:] = sc[r].float() if sc is not None else 0.0
        out = torch.zeros(rows, dim, dtype=torch.float32, device=kvc.device)
        for r in range(rows):
            s, p = int(row_slot[r]), int(row_pos[r])
            if (p + 1) % ratio:
                continue
            idx = [(p - t) % ring for t in range(ratio - 1, -1, -1)]
            grp = tail[s, idx]
            wts = torch.softmax(grp[:, dim:], 0) if ratio > 1 else torch.ones_like(grp[:, :dim])
            out[r] = (grp[:, :dim] * wts).sum(0)
        return out.to(torch.bfloat16)

    # ---- indexer ----------------------------------------------------------------------------------------
    def index_score(self, q, w, scale, keys, row_slot, row_len, ld, mask=None, mask_block=8):
        """score[r, e] = sum_h w[r, h] relu(q[r, h] . keys[slot_r, e]) for e < len_r (and kept blocks), -inf elsewhere."""
        rows, nh, D = q.shape
        out = torch.full((rows, ld), float("-inf"), dtype=torch.float32, device=q.device)
        for r in range(rows):
            n = min(int(row_len[r]), ld)
            if n <= 0:
                continue
            k = keys[int(row_slot[r]), :n].float()
            dots = torch.relu(q[r].float() @ k.t())                      # [nh, n]
            wr = w[r].float() if w is not None else torch.full((nh,), float(scale), device=q.device)
            sc = (dots * wr[:, None]).sum(0)
            if mask is not None:
                keep = mask[r, torch.arange(n, device=q.device) // mask_block] != 0
                sc = torch.where(keep, sc, torch.full_like(sc, float("-inf")))
            out[r, :n] = sc
        return out

    def topk_select(self, score, k, row_n=None):
        """Exact top-k per row (ties to the lower index, -inf never counts): ascending indices, -1 padded, int32."""
        rows, ld = score.shape
        sel = torch.full((rows, k), -1, dtype=torch.int32, device=score.device)
        for r in range(rows):
            n = min(int(row_n[r]), ld) if row_n is not None else ld
            row = score[r, :n].float()
            valid = int((row != float("-inf")).sum())
            kk = min(k, valid)
            if kk == 0:
                continue
            order = torch.sort(row, descending=True, stable=True).indices[:kk]    # stable: equal scores keep index order
            sel[r, :kk] = torch.sort(order).values.to(torch.int32)
        return sel

    def block_mask(self, score, row_n, bsize, nblocks, mask_ld):
        """Candidate pool: keep the `nblocks` blocks (of `bsize` entries) with the largest maxima, the block of the row's
        last valid entry always among them; mask [rows, mask_ld] uint8."""
        rows, ld = score.shape
        bmax = torch.full((rows, mask_ld), float("-inf"), dtype=torch.float32, device=score.device)
        for r in range(rows):
            n = min(int(row_n[r]), ld)
            for b in range(min(mask_ld, (n + bsize - 1) // bsize)):
                bmax[r, b] = score[r, b * bsize:min(n, (b + 1) * bsize)].max()
            if n > 0 and (n - 1) // bsize < mask_ld:
                bmax[r, (n - 1) // bsize] = float("inf")
        sel = TorchExtras.topk_select(self, bmax, nblocks)
        mask = torch.zeros(rows, mask_ld, dtype=torch.uint8, device=score.device)
        for r in range(rows):
            ids = sel[r][sel[r] >= 0].long()
            mask[r, ids] = 1
        return mask

    # ---- selected-block attention -----------------------------------------------------------------------
    def qsa_pool(self, raw, w, pos0, inv_freq, eps):
        """raw [blocks, kp, D] fp32 -> rope(rmsnorm(mean over the block) * w) at pos0, rotation in halves over 2 * len(inv_freq) dims."""
        m = raw.float().mean(1)
        x = m * torch.rsqrt(m.pow(2).mean(-1, keepdim=True) + eps) * w.float()
        half = inv_freq.shape[0]
        ang = pos0.float()[:, None] * inv_freq.float()[None]
        a, b = x[:, :half], x[:, half:2 * half]
        rot = torch.cat([a * ang.cos() - b * ang.sin(), b * ang.cos() + a * ang.sin()], -1)
        return torch.cat([rot, x[:, 2 * half:]], -1).to(torch.bfloat16)

    def qsa_table(self, sel, row_slot, row_pos, block_table, kp):
        """Per-row page table of a selected-block attention: rows that see at most `top` finished blocks keep the dense
        table; others read their `top` selected blocks and the open tail block. Returns (table [rows, top + 1], kvlen)."""
        rows, top = sel.shape
        table = torch.zeros(rows, top + 1, dtype=torch.int32, device=sel.device)
        kvlen = torch.zeros(rows, dtype=torch.int32, device=sel.device)
        for r in range(rows):
            pos, slot = int(row_pos[r]), int(row_slot[r])
            nv, tail = (pos + 1) // kp, (pos + 1) % kp
            if nv <= top:
                logical = list(range(nv + (1 if tail else 0)))
                kvlen[r] = pos + 1
            else:
                logical = [int(b) for b in sel[r]] + ([nv] if tail else [])
                kvlen[r] = top * kp + tail
            for j, b in enumerate(logical):
                table[r, j] = block_table[slot, b]
        return table, kvlen

    # ---- drafting heads ---------------------------------------------------------------------------------
    def markov_bias(self, head, emb, tok, slot):
        """bias[r] = head @ emb[tok[r]] for rows without a cached bias row (slot < 0; others are left zero), bf16."""
        out = torch.zeros(tok.shape[0], head.shape[0], dtype=torch.float32, device=head.device)
        need = slot < 0
        out[need] = emb[tok[need].long()].float() @ head.float().t()
        return out.to(torch.bfloat16)

    def markov_step(self, draft, step, logits, stage, cache, slot, slot_of, col0=0, parts=1):
        """One step of the Markov head loop: pick = argmax(logits + bias) (NaN first, larger value, lower index) with the
        bias row from the cache (slot >= 0) or the staged rows; writes draft[:, step + 1]; returns (tok, next slot)."""
        n = stage.shape[1]
        bias = torch.where((slot >= 0)[:, None], cache[slot.clamp_min(0).long()].float(), stage.float())
        pick = _argmax_order(logits[:, :n].float() + bias) + col0
        draft[:, step + 1] = pick.to(draft.dtype)
        return pick.to(torch.int32), slot_of[pick.long()]

    def conf_head(self, xc, emb, draft, w, steps, block):
        """conf[s * steps + i] = [xc[s * block + i] | emb[draft[s, i]]] . w (fp32)."""
        streams, d = draft.shape[0], xc.shape[1]
        x = xc.float().view(streams, block, d)[:, :steps]
        e = emb[draft[:, :steps].long()].float()
        return (torch.cat([x, e], -1) * w.float()).sum(-1).reshape(-1)

    def stream_mean(self, h):
        """h [rows, hc, dim] -> bf16 mean over the streams, summed in stream order."""
        acc = h[:, 0].float()
        for j in range(1, h.shape[1]):
            acc = acc + h[:, j].float()
        return (acc / h.shape[1]).to(torch.bfloat16)

    def stream_collapse(self, h, pre):
        """xc[r] = sum_j pre[r, j] h[r, j] (bf16)."""
        return (h.float() * pre.float()[:, :h.shape[1], None]).sum(1).to(torch.bfloat16)

    def block_ring_attention(self, q, ring, kvb, meta, sink, scale, rope_tab, window, block, rope_dims=64):
        """Attention of a block drafter whose keys are their own values (one latent row per position, shared by all
        heads). Row r, described by meta[r] = (slot, pos, wend, b0), sees
          * the slot's ring rows of positions max(0, wend - window) .. wend - 1 (position p lives in ring row
            p % ring.shape[1]), and
          * the `block` rows kvb[b0 : b0 + block] of its own draft block, all of them (no mask inside the block);
        the head's sink logit joins the softmax denominator only. The result is rounded to bf16 and its last `rope_dims`
        elements are rotated back by the row's position (inverse of the interleaved-pair rotation the latent rows
        carry; rope_tab [positions, rope_dims] holds (cos, sin) pairs). q [rows, heads, D], ring [slots, ring_len, D],
        kvb [n, D], sink [heads] -> [rows, heads, D] fp32. Statement only: no kernel of this repo's presets needs it
        (reference `dspark_attn`, `kernels/k-dspark/src/lib.rs:276-402`)."""
        rows, heads, D = q.shape
        ring_len = ring.shape[1]
        out = torch.zeros(rows, heads, D, dtype=torch.float32, device=q.device)
        for r in range(rows):
            slot, pos, wend, b0 = (int(v) for v in meta[r].tolist())
            first = max(0, wend - window)
            idx = torch.tensor([p % ring_len for p in range(first, wend)], dtype=torch.long, device=q.device)
            keys = torch.cat([ring[slot].index_select(0, idx), kvb[b0:b0 + block]], 0).float()        # [n, D]
            s = (q[r].float() @ keys.t()) * scale                                                     # [heads, n]
            m = torch.maximum(s.max(-1).values, sink.float())
            p = torch.exp(s - m[:, None])
            den = p.sum(-1) + torch.exp(sink.float() - m)
            o = ((p @ keys) / den[:, None]).to(torch.bfloat16).float()
            cs = rope_tab[pos, 0::2].float()
            sn = rope_tab[pos, 1::2].float()
            a, b = o[:, D - rope_dims::2].clone(), o[:, D - rope_dims + 1::2].clone()
            o[:, D - rope_dims::2] = a * cs + b * sn
            o[:, D - rope_dims + 1::2] = b * cs - a * sn
            out[r] = o
        return out


class CudaExtras:
    """Kernel-backed forms; `self.C` is the extension, `self.status_word` the device status word, `self.device` the GPU."""

    def _i32(self, *shape):
        return torch.empty(*shape, dtype=torch.int32, device=self.device)

    def engram_gate(self, h, kv, qk, eps):
        out = torch.empty_like(h)
        self.launches += 1
        if kv.dim() == 3:
            self.C.engram_gate(out, h.contiguous(), kv.contiguous(), None, qk, eps)
        else:
            self.C.engram_gate(out, h.contiguous(), None, kv.contiguous(), qk, eps)
        return out

    def comp_step(self, tail, kvc, sc, row_slot, row_pos, ratio):
        out = torch.empty(kvc.shape, dtype=torch.bfloat16, device=self.device)
        self.launches += 2
        self.C.comp_step(out, tail, kvc.contiguous(), None if sc is None else sc.contiguous(), row_slot, row_pos, ratio)
        return out

    def index_score(self, q, w, scale, keys, row_slot, row_len, ld, mask=None, mask_block=8):
        score = torch.empty(q.shape[0], ld, dtype=torch.float32, device=self.device)
        self.launches += 1
        self.C.index_score(score, q.contiguous(), w, float(scale), keys, row_slot, row_len, mask, mask_block)
        return score

    def topk_select(self, score, k, row_n=None):
        sel = self._i32(score.shape[0], k)
        self.launches += 1
        self.C.topk_select(sel, score, row_n)
        return sel

    def block_mask(self, score, row_n, bsize, nblocks, mask_ld):
        rows = score.shape[0]
        bmax = torch.empty(rows, mask_ld, dtype=torch.float32, device=self.device)
        mask = torch.empty(rows, mask_ld, dtype=torch.uint8, device=self.device)
        self.launches += 3
        self.C.block_max(bmax, score, row_n, bsize)
        sel = self._i32(rows, nblocks)
        self.C.topk_select(sel, bmax, None)
        self.C.sel_to_mask(mask, sel)
        return mask

    def qsa_pool(self, raw, w, pos0, inv_freq, eps):
        pooled = torch.empty(raw.shape[0], raw.shape[2], dtype=torch.bfloat16, device=self.device)
        self.launches += 1
        self.C.qsa_pool(pooled, raw.contiguous(), w, pos0, inv_freq, eps)
        return pooled

    def qsa_table(self, sel, row_slot, row_pos, block_table, kp):
        rows, top = sel.shape
        table, kvlen = self._i32(rows, top + 1), self._i32(rows)
        self.launches += 1
        self.C.qsa_table(table, kvlen, sel, row_slot, row_pos, block_table, kp, self.status_word)
        return table, kvlen

    def markov_bias(self, head, emb, tok, slot):
        out = torch.zeros(tok.shape[0], head.shape[0], dtype=torch.bfloat16, device=self.device)
        self.launches += 1
        self.C.markov_bias(out, head, emb, tok, slot)
        return out

    def markov_step(self, draft, step, logits, stage, cache, slot, slot_of, col0=0, parts=8):
        rows = draft.shape[0]
        pair = self._i32(parts, rows, 2)
        tok, nslot = self._i32(rows), self._i32(rows)
        self.launches += 2
        self.C.markov_score(pair, logits, stage, cache, slot, col0)
        self.C.markov_pick(draft, tok, nslot, pair, slot_of, step, self.status_word)
        return tok, nslot

    def conf_head(self, xc, emb, draft, w, steps, block):
        conf = torch.empty(draft.shape[0] * steps, dtype=torch.float32, device=self.device)
        self.launches += 1
        self.C.conf_head(conf, xc, emb, draft, w, steps, block)
        return conf

    def stream_mean(self, h):
        out = torch.empty(h.shape[0], h.shape[2], dtype=torch.bfloat16, device=self.device)
        self.launches += 1
        self.C.stream_mean(out, h.contiguous())
        return out

    def stream_collapse(self, h, pre):
        xc = torch.empty(h.shape[0], h.shape[2], dtype=torch.bfloat16, device=self.device)
        self.launches += 1
        self.C.stream_collapse(xc, h.contiguous(), pre)
        return xc


def qsa_decode_attention(ops, q, proj, k_cache, v_cache, pooled, q_idx, row_slot, row_pos, block_table, kv_block, nq, nkv,
                         hd, gated, top, scale):
    """Selected-block attention of decode rows: block scores of the row's indexer queries `q_idx` [rows, nh, D] against the
    slot's pooled block keys `pooled` [slots, max_blocks, D], exact top-`top` finished blocks, then the ordinary paged
    decode attention over a per-row page table holding only those blocks and the open tail. Rows that see at most `top`
    finished blocks read everything (the table is the dense one)."""
    rows = q.shape[0]
    nv = ((row_pos + 1) // kv_block).to(torch.int32)
    score = ops.index_score(q_idx, None, scale, pooled, row_slot, nv, pooled.shape[1])
    sel = ops.topk_select(score, top, nv)
    table, kvlen = ops.qsa_table(sel, row_slot, row_pos, block_table, kv_block)
    own = torch.arange(rows, dtype=torch.int32, device=q.device)         # every row reads its own table
    return ops.attention(q, proj if proj is not None else q, k_cache, v_cache, own, kvlen, table, kv_block, nq, nkv, hd, gated)
