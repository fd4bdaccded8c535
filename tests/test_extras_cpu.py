"""fp32 statements of the sparse-attention selection ops and the Markov drafting head (the oracles of the GPU tests),
checked against brute force on the CPU."""
import math

import torch

from ferrite_b200.models.dspark import MarkovHead
from ferrite_b200.ops.extras import qsa_decode_attention
from ferrite_b200.ops.torch_ops import TorchOps

OPS = TorchOps("cpu", torch.float32)
NEG = float("-inf")


def test_topk_select_ties_and_minus_inf():
    s = torch.tensor([[1.0, 5.0, 5.0, NEG, 3.0, 5.0], [NEG, NEG, 2.0, NEG, NEG, NEG]])
    sel = OPS.topk_select(s, 3)
    assert sel.tolist() == [[1, 2, 5], [2, -1, -1]]
    assert OPS.topk_select(s, 2).tolist() == [[1, 2], [2, -1]]                 # ties go to the lower index
    assert OPS.topk_select(s, 3, torch.tensor([5, 2])).tolist() == [[1, 2, 4], [-1, -1, -1]]
    g = torch.Generator().manual_seed(0)
    big = torch.randn(3, 500, generator=g)
    want = [sorted(torch.topk(big[r], 17).indices.tolist()) for r in range(3)]
    assert OPS.topk_select(big, 17).tolist() == want


def test_compressor_pairs_tokens():
    dim, ring = 8, 4
    tail = torch.zeros(2, ring, 2 * dim)
    g = torch.Generator().manual_seed(1)
    kvc, sc = torch.randn(3, dim, generator=g), torch.randn(3, dim, generator=g)
    slot, pos = torch.tensor([1, 1, 1], dtype=torch.int32), torch.tensor([4, 5, 6], dtype=torch.int32)
    out = OPS.comp_step(tail, kvc, sc, slot, pos, 2).float()
    w = torch.softmax(torch.stack([sc[0], sc[1]]), 0)
    want = kvc[0] * w[0] + kvc[1] * w[1]
    assert torch.allclose(out[1], want.to(torch.bfloat16).float()) and not out[0].any() and not out[2].any()
    # the open group is finished by a later call through the ring
    out2 = OPS.comp_step(tail, kvc[:1], sc[:1], slot[:1], torch.tensor([7], dtype=torch.int32), 2).float()
    w2 = torch.softmax(torch.stack([sc[2], sc[0]]), 0)
    assert torch.allclose(out2[0], (kvc[2] * w2[0] + kvc[0] * w2[1]).to(torch.bfloat16).float())


def test_selected_block_attention_equals_masked_dense_attention():
    g = torch.Generator().manual_seed(2)
    nq, nkv, hd, kvb, nblk, top, D, nh = 4, 2, 16, 8, 12, 3, 16, 4
    k_cache, v_cache = torch.randn(2 * nblk, kvb, nkv, hd, generator=g), torch.randn(2 * nblk, kvb, nkv, hd, generator=g)
    bt = torch.randperm(2 * nblk, generator=g).to(torch.int32).view(2, nblk)
    pooled = torch.randn(2, nblk, D, generator=g)
    rows = 3
    slot = torch.tensor([0, 1, 1], dtype=torch.int32)
    pos = torch.tensor([70, 21, 63], dtype=torch.int32)             # 8 blocks + tail, 2 blocks + tail (dense), 8 blocks exactly
    q, q_idx = torch.randn(rows, nq * hd, generator=g), torch.randn(rows, nh, D, generator=g)
    got = qsa_decode_attention(OPS, q, None, k_cache, v_cache, pooled, q_idx, slot, pos, bt, kvb, nq, nkv, hd, False, top, 0.5)
    for r in range(rows):
        p, s = int(pos[r]), int(slot[r])
        nv = (p + 1) // kvb
        if nv <= top:
            cells = list(range(p + 1))
        else:
            sc = (torch.relu(q_idx[r] @ pooled[s, :nv].t()) * 0.5).sum(0)
            blocks = sorted(torch.topk(sc, top).indices.tolist())
            cells = [b * kvb + c for b in blocks for c in range(kvb)] + list(range(nv * kvb, p + 1))
        cells = torch.tensor(cells)
        K = k_cache[bt[s, cells // kvb].long(), cells % kvb]
        V = v_cache[bt[s, cells // kvb].long(), cells % kvb]
        qh = q[r].view(nkv, nq // nkv, hd)
        w = torch.softmax(torch.einsum("kgd,tkd->kgt", qh, K) / math.sqrt(hd), -1)
        want = torch.einsum("kgt,tkd->kgd", w, V).reshape(-1)
        assert torch.allclose(got[r], want, atol=1e-5), r


def test_block_mask_keeps_the_last_block():
    score = torch.tensor([[9.0, 1, 1, 1, 8, 1, 1, 1, 0, 0, 0, 0, 0.5, NEG, NEG, NEG]])
    mask = OPS.block_mask(score, torch.tensor([13]), 4, 2, 4)
    assert mask.tolist() == [[1, 0, 0, 1]]                          # best block and the block of the last valid entry
    s2 = OPS.index_score(torch.ones(1, 2, 4), torch.tensor([[1.0, 2.0]]), 0.0, torch.ones(1, 16, 4), torch.tensor([0]),
                         torch.tensor([13]), 16, mask=mask, mask_block=4)
    assert s2[0, 0] == 12.0 and s2[0, 4] == NEG and s2[0, 12] == 12.0 and s2[0, 13] == NEG


def test_markov_head_draft_and_confidence():
    g = torch.Generator().manual_seed(3)
    V, rank, rows, steps, d = 50, 16, 3, 4, 8
    head, emb = torch.randn(V, rank, generator=g).bfloat16(), torch.randn(V, rank, generator=g).bfloat16()
    logits = torch.randn(steps, rows, V, generator=g)
    anchors = torch.tensor([3, 7, 11])
    plain = MarkovHead(OPS, head, emb, cached_tokens=[], conf_w=torch.randn(d + rank, generator=g))
    cached = MarkovHead(OPS, head, emb, cached_tokens=list(range(0, V, 2)))
    da, db = plain.draft(anchors, logits), cached.draft(anchors, logits)
    assert torch.equal(da, db) and da[:, 0].tolist() == [3, 7, 11]
    for r in range(rows):
        t = int(anchors[r])
        for i in range(steps):
            bias = (emb[t].float() @ head.float().t()).bfloat16().float()
            t = int((logits[i, r] + bias).argmax())
            assert int(da[r, i + 1]) == t
    xc = torch.randn(rows * 6, d, generator=g).bfloat16()
    conf = plain.confidence(xc, da, block=6)
    j = 1 * steps + 2
    want = (torch.cat([xc[1 * 6 + 2].float(), emb[int(da[1, 2])].float()]) * plain.conf_w).sum()
    assert abs(float(conf.view(-1)[j]) - float(want)) < 1e-4
    cut = MarkovHead.cut(da, torch.tensor([[1.0, 1.0, -1.0, 1.0]] * rows), 0.0)
    assert cut[0] == da[0, 1:3].tolist()


def test_engram_gate_partials_match_summed_form():
    g = torch.Generator().manual_seed(4)
    rows, hc, d = 2, 3, 32
    h = torch.randn(rows, hc, d, generator=g).bfloat16()
    parts = torch.randn(2, rows, (hc + 1) * d, generator=g)
    qk = torch.randn(hc, d, generator=g)
    a = OPS.engram_gate(h, parts, qk, 1e-6)
    b = OPS.engram_gate(h, (parts[0] + parts[1]).bfloat16(), qk, 1e-6)
    assert torch.equal(a, b) and a.shape == h.shape
    assert (a.float() - h.float()).abs().max() > 0
    sm = OPS.stream_mean(h)
    assert torch.allclose(sm.float(), h.float().mean(1), atol=2e-2)
    pre = torch.rand(rows, hc, generator=g)
    assert torch.allclose(OPS.stream_collapse(h, pre).float(), (h.float() * pre[..., None]).sum(1), atol=3e-2)


def test_block_ring_attention_window_block_sink_and_inverse_rope():
    """The block drafter's ring attention: the window is read through the ring (positions modulo its length), the block's
    keys are all visible, the sink only weakens the result, and the tail of the output is rotated back by the position."""
    from ferrite_b200.ops.torch_ops import TorchOps
    ops = TorchOps(torch.device("cpu"), torch.float32)
    g = torch.Generator().manual_seed(5)
    heads, D, ring_len, window, block, rd = 3, 96, 8, 5, 4, 32
    ring = torch.randn(2, ring_len, D, generator=g)
    kvb = torch.randn(2 * block, D, generator=g)
    q = torch.randn(2, heads, D, generator=g)
    # row 0: slot 1, 11 tokens absorbed (the ring wrapped once), its block is the second one; row 1: a fresh slot
    meta = torch.tensor([[1, 11, 11, block], [0, 0, 0, 0]], dtype=torch.int32)
    inv = 1.0 / (10000.0 ** (torch.arange(rd // 2).float() / (rd // 2)))
    ang = torch.arange(16).float()[:, None] * inv[None]
    tab = torch.stack([ang.cos(), ang.sin()], -1).reshape(16, rd)
    no_sink = torch.full((heads,), -1e30)
    got = ops.block_ring_attention(q, ring, kvb, meta, no_sink, 0.1, tab, window, block, rope_dims=rd)
    # by hand, row 0: positions 6..10 live in ring rows 6, 7, 0, 1, 2
    keys = torch.cat([ring[1, [6, 7, 0, 1, 2]], kvb[block:2 * block]], 0)
    want = torch.softmax((q[0] @ keys.t()) * 0.1, -1) @ keys
    want = want.to(torch.bfloat16).float()
    head, tail = want[:, :D - rd], want[:, D - rd:].reshape(heads, rd // 2, 2)
    cs, sn = ang[11].cos(), ang[11].sin()
    back = torch.stack([tail[..., 0] * cs + tail[..., 1] * sn, tail[..., 1] * cs - tail[..., 0] * sn], -1).reshape(heads, rd)
    assert torch.allclose(got[0], torch.cat([head, back], -1), atol=1e-6)
    # the inverse rotation undoes the forward one: rotate forward again and the plain attention output is back
    t = got[0][:, D - rd:].reshape(heads, rd // 2, 2)
    fwd = torch.stack([t[..., 0] * cs - t[..., 1] * sn, t[..., 0] * sn + t[..., 1] * cs], -1).reshape(heads, rd)
    assert torch.allclose(fwd, want[:, D - rd:], atol=1e-5)
    # row 1 has no window at all: only its block's keys, position 0 leaves the tail as it is
    w1 = (torch.softmax((q[1] @ kvb[:block].t()) * 0.1, -1) @ kvb[:block]).to(torch.bfloat16).float()
    assert torch.allclose(got[1], w1, atol=1e-6)
    # a sink as large as the best logit takes its share of the denominator: same direction, smaller norm
    s0 = ((q[0] @ keys.t()) * 0.1).max(-1).values
    sunk = ops.block_ring_attention(q, ring, kvb, meta, s0, 0.1, tab, window, block, rope_dims=rd)
    ratio = sunk[0].norm(dim=-1) / got[0].norm(dim=-1)
    assert bool((ratio < 0.95).all()) and bool((ratio > 0.05).all())
    cosine = torch.nn.functional.cosine_similarity(sunk[0], got[0], dim=-1)
    assert bool((cosine > 0.99).all())
