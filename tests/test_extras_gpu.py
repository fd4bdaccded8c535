"""Kernels of `csrc/sparse_index.cu`, `csrc/dspark.cu` and the Engram gate against their fp32 PyTorch statements."""
import pytest
import torch

from ferrite_b200.models.dspark import MarkovHead
from ferrite_b200.ops.extras import qsa_decode_attention
from ferrite_b200.ops.torch_ops import TorchOps

pytestmark = pytest.mark.gpu
DEV = "cuda"
NEG = float("-inf")


@pytest.fixture(scope="module")
def ops(ext):
    from ferrite_b200.ops.cuda_ops import CudaOps
    return CudaOps(DEV)


@pytest.fixture(scope="module")
def tops():
    return TorchOps(DEV, torch.float32)


def _gen(seed):
    return torch.Generator(device=DEV).manual_seed(seed)


def test_engram_gate_and_stream_reductions(ops, tops):
    g = _gen(1)
    rows, hc, d = 5, 4, 1024
    h = torch.randn(rows, hc, d, generator=g, device=DEV).bfloat16()
    parts = torch.randn(3, rows, (hc + 1) * d, generator=g, device=DEV)
    qk = torch.randn(hc, d, generator=g, device=DEV)
    for kv in (parts, (parts[0] + parts[1] + parts[2]).bfloat16()):
        got, want = ops.engram_gate(h, kv, qk, 1e-6), tops.engram_gate(h, kv, qk, 1e-6)
        assert (got.float() - want.float()).abs().max().item() <= 0.04
    assert torch.equal(ops.engram_gate(h, parts, qk, 1e-6),
                       ops.engram_gate(h, (parts[0] + parts[1] + parts[2]).bfloat16(), qk, 1e-6))
    assert (ops.stream_mean(h).float() - tops.stream_mean(h).float()).abs().max().item() <= 0.02
    pre = torch.rand(rows, hc, generator=g, device=DEV)
    assert (ops.stream_collapse(h, pre).float() - tops.stream_collapse(h, pre).float()).abs().max().item() <= 0.04


@pytest.mark.parametrize("ratio", [1, 2, 4])
def test_compressor(ops, tops, ratio):
    g = _gen(2 + ratio)
    dim, ring, rows = 512, 8, 9
    ta = torch.randn(3, ring, 2 * dim, generator=g, device=DEV)
    tb = ta.clone()
    kvc, sc = torch.randn(rows, dim, generator=g, device=DEV), torch.randn(rows, dim, generator=g, device=DEV)
    slot = torch.tensor([0, 0, 0, 0, 0, 2, 2, 2, 2], dtype=torch.int32, device=DEV)
    pos = torch.tensor([10, 11, 12, 13, 14, 3, 4, 5, 6], dtype=torch.int32, device=DEV)
    got = ops.comp_step(ta, kvc, sc if ratio > 1 else None, slot, pos, ratio)
    want = tops.comp_step(tb, kvc, sc if ratio > 1 else None, slot, pos, ratio)
    assert (got.float() - want.float()).abs().max().item() <= 0.03
    assert torch.allclose(ta, tb)
    closing = ((pos + 1) % ratio == 0)
    assert not got[~closing].float().abs().sum().item()


@pytest.mark.parametrize("nh,D,ld", [(32, 128, 1000), (4, 128, 300), (64, 64, 129), (5, 32, 40)])
def test_index_score(ops, tops, nh, D, ld):
    g = _gen(nh + D)
    rows, slots = 4, 3
    q = (torch.randn(rows, nh, D, generator=g, device=DEV) * 0.3).bfloat16()
    keys = torch.randn(slots, ld, D, generator=g, device=DEV).bfloat16()
    w = torch.rand(rows, nh, generator=g, device=DEV)
    slot = torch.tensor([0, 2, 1, 2], dtype=torch.int32, device=DEV)
    length = torch.tensor([ld, ld // 2 + 3, 1, 0], dtype=torch.int32, device=DEV)
    for weights, scale in ((w, 0.0), (None, 0.25)):
        got = ops.index_score(q, weights, scale, keys, slot, length, ld)
        want = tops.index_score(q, weights, scale, keys, slot, length, ld)
        fin = torch.isfinite(want)
        assert torch.equal(torch.isfinite(got), fin)
        assert (got[fin] - want[fin]).abs().max().item() <= 2e-2 * max(1.0, want[fin].abs().max().item())
    mask = (torch.rand(rows, (ld + 7) // 8, generator=g, device=DEV) > 0.5).to(torch.uint8)
    got = ops.index_score(q, w, 0.0, keys, slot, length, ld, mask=mask, mask_block=8)
    want = tops.index_score(q, w, 0.0, keys, slot, length, ld, mask=mask, mask_block=8)
    assert torch.equal(torch.isfinite(got), torch.isfinite(want))


@pytest.mark.parametrize("n,k", [(37, 5), (1024, 64), (5000, 512), (70000, 2048), (100, 300)])
def test_topk_select_is_exact(ops, tops, n, k):
    g = _gen(n + k)
    score = torch.randn(3, n, generator=g, device=DEV)
    score[1] = torch.randint(0, 7, (n,), generator=g, device=DEV).float()          # many ties
    score[2, ::3] = NEG
    assert torch.equal(ops.topk_select(score, k), tops.topk_select(score, k))
    row_n = torch.tensor([n, n // 2, max(1, n // 3)], dtype=torch.int32, device=DEV)
    assert torch.equal(ops.topk_select(score, k, row_n), tops.topk_select(score, k, row_n))


def test_block_mask_and_tables(ops, tops):
    g = _gen(9)
    rows, ld, bsize, nblocks = 3, 640, 8, 16
    score = torch.randn(rows, ld, generator=g, device=DEV)
    row_n = torch.tensor([640, 333, 9], dtype=torch.int32, device=DEV)
    mask_ld = ld // bsize
    assert torch.equal(ops.block_mask(score, row_n, bsize, nblocks, mask_ld), tops.block_mask(score, row_n, bsize, nblocks, mask_ld))
    kp, top, nblk = 16, 4, 40
    bt = torch.randperm(2 * nblk, generator=g, device=DEV).to(torch.int32).view(2, nblk)
    slot = torch.tensor([0, 1, 1], dtype=torch.int32, device=DEV)
    pos = torch.tensor([200, 63, 40], dtype=torch.int32, device=DEV)
    sel = torch.tensor([[1, 5, 7, 11], [0, 1, 2, -1], [0, 1, -1, -1]], dtype=torch.int32, device=DEV)
    ta, la = ops.qsa_table(sel, slot, pos, bt, kp)
    tb, lb = tops.qsa_table(sel, slot, pos, bt, kp)
    assert torch.equal(la, lb)
    for r in range(3):
        used = (int(lb[r]) + kp - 1) // kp
        assert torch.equal(ta[r, :used], tb[r, :used])
    assert ops.status() == 0


def test_qsa_pool(ops, tops):
    g = _gen(10)
    raw = torch.randn(7, 16, 128, generator=g, device=DEV)
    w = torch.rand(128, generator=g, device=DEV) + 0.5
    pos0 = torch.arange(7, dtype=torch.int32, device=DEV) * 16
    inv = (1e4 ** (-torch.arange(32, dtype=torch.float64) / 32)).float().to(DEV)
    got, want = ops.qsa_pool(raw, w, pos0, inv, 1e-6), tops.qsa_pool(raw, w, pos0, inv, 1e-6)
    assert (got.float() - want.float()).abs().max().item() <= 0.03


def test_selected_block_attention_end_to_end(ops, tops):
    g = _gen(11)
    nq, nkv, hd, kvb, nblk, top, D, nh = 8, 2, 128, 64, 24, 4, 128, 4
    k_cache = torch.randn(2 * nblk, kvb, nkv, hd, generator=g, device=DEV).bfloat16()
    v_cache = torch.randn(2 * nblk, kvb, nkv, hd, generator=g, device=DEV).bfloat16()
    bt = torch.randperm(2 * nblk, generator=g, device=DEV).to(torch.int32).view(2, nblk)
    pooled = torch.randn(2, nblk, D, generator=g, device=DEV).bfloat16()
    slot = torch.tensor([0, 1, 1, 0], dtype=torch.int32, device=DEV)
    pos = torch.tensor([1400, 130, 1023, 700], dtype=torch.int32, device=DEV)
    q = torch.randn(4, nq * hd, generator=g, device=DEV).bfloat16()
    q_idx = torch.randn(4, nh, D, generator=g, device=DEV).bfloat16()
    got = qsa_decode_attention(ops, q, None, k_cache, v_cache, pooled, q_idx, slot, pos, bt, kvb, nq, nkv, hd, False, top, 0.5)
    want = qsa_decode_attention(tops, q, None, k_cache, v_cache, pooled, q_idx, slot, pos, bt, kvb, nq, nkv, hd, False, top, 0.5)
    assert (got.float() - want.float()).abs().max().item() <= 0.05
    assert ops.status() == 0


def test_markov_head_on_the_gpu(ops, tops):
    g = _gen(12)
    V, rank, rows, steps, d = 4099, 256, 5, 6, 512
    head = (torch.randn(V, rank, generator=g, device=DEV) * 0.1).bfloat16()
    emb = torch.randn(V, rank, generator=g, device=DEV).bfloat16()
    logits = torch.randn(steps, rows, V, generator=g, device=DEV)
    anchors = torch.tensor([3, 7, 11, 4000, 77], device=DEV)
    cw = torch.randn(d + rank, generator=g, device=DEV)
    a = MarkovHead(ops, head, emb, cached_tokens=list(range(0, V, 3)), conf_w=cw)
    b = MarkovHead(tops, head, emb, cached_tokens=list(range(0, V, 3)), conf_w=cw)
    assert (a.cache.float() - b.cache.float()).abs().max().item() <= 0.05
    # the loop itself, on the same bias rows: the picks are exact
    b.cache = a.cache
    da = a.draft(anchors, logits)
    tok, slot = da[:, 0].contiguous(), a.slot_of[da[:, 0].long()]
    for i in range(steps):
        stage = ops.markov_bias(head, emb, tok, slot)
        draft_b = da.clone()
        tok_b, slot_b = tops.markov_step(draft_b, i, logits[i], stage, a.cache, slot, a.slot_of)
        assert torch.equal(draft_b[:, i + 1], da[:, i + 1])
        tok, slot = tok_b, slot_b
    xc = torch.randn(rows * 8, d, generator=g, device=DEV).bfloat16()
    ca, cb = a.confidence(xc, da, block=8), b.confidence(xc, da, block=8)
    assert (ca - cb).abs().max().item() <= 1e-2 * max(1.0, cb.abs().max().item())
    nan_logits = logits[0].clone()
    nan_logits[0, 17] = float("nan")
    d2 = da.clone()
    t2, _ = ops.markov_step(d2, 0, nan_logits, stage, a.cache, slot, a.slot_of)
    assert int(t2[0]) == 17
    assert ops.status() == 0
