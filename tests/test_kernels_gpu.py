"""Numerics of each sm_100a kernel against the plain PyTorch fp32 statement of the same op (`TorchOps`)."""
import math

import pytest
import torch

from ferrite_b200.ops.torch_ops import TorchOps

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops(ext):
    from ferrite_b200.ops.cuda_ops import CudaOps
    return CudaOps(DEV)


@pytest.fixture(scope="module")
def tops():
    return TorchOps(DEV, torch.float32)


def rnd(*shape, scale=1.0, seed=0, dtype=torch.bfloat16):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=DEV) * scale).to(dtype)


# Attention outputs are averages of random value rows: their RMS is ~0.1 while the rounding of P (bf16 in the tensor-core
# kernels) and of V acts on values of order 1, so the absolute term is a tenth of the output RMS there.
ATT_ATOL = 0.1


def close(got, want, rtol=None, atol=None):
    """Every element within atol * rms(want) + rtol * |want|. Defaults by the kernel's output type: a bf16 result may be
    two bf16 roundings away (the kernel rounds once, the fp32 oracle's result is rounded for the comparison by the
    magnitude term); both kinds see the bf16 rounding of intermediates (normalised rows, activations) and the summation
    order as noise against the output's RMS: measured up to 1.2 % of it."""
    low = got.dtype in (torch.bfloat16, torch.float16)
    rtol = (1.6e-2 if low else 4e-3) if rtol is None else rtol
    atol = 1.5e-2 if atol is None else atol
    got, want = got.float(), want.float()
    rms = want.pow(2).mean().sqrt().item()
    excess = ((got - want).abs() - (atol * rms + rtol * want.abs())).max().item()
    assert excess <= 0, (f"worst element exceeds atol {atol} x rms {rms:.4g} + rtol {rtol} x |want| by {excess:.4g} "
                         f"(max |err| {(got - want).abs().max().item():.4g}, max |want| {want.abs().max().item():.4g})")


@pytest.mark.parametrize("M", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("N,K", [(512, 256), (1000, 768), (5120, 5120), (640, 17408)])
def test_gemv_plain(ops, tops, M, N, K):
    x, w = rnd(M, K, seed=1), rnd(N, K, scale=0.05, seed=2)
    res = rnd(M, N, seed=3)
    close(ops.linear(x, w), tops.linear(x, w))
    close(ops.linear(x, w, res=res), tops.linear(x, w, res=res))
    close(ops.linear(x, w, out_f32=True), tops.linear(x, w, out_f32=True))


@pytest.mark.parametrize("M", [1, 4, 8])
def test_gemv_norm_swiglu(ops, tops, M):
    K, I = 5120, 1024
    x, w, nw = rnd(M, K, seed=1), rnd(2 * I, K, scale=0.03, seed=2), rnd(K, scale=0.1, seed=4)
    # silu(g) * u: the relative errors of the two factors add
    close(ops.linear(x, w, norm_w=nw, eps=1e-6, swiglu=True), tops.linear(x, w, norm_w=nw, eps=1e-6, swiglu=True), rtol=2.5e-2)
    close(ops.linear(x, w[:I], norm_w=nw, eps=1e-6), tops.linear(x, w[:I], norm_w=nw, eps=1e-6))


def test_gemv_batch_invariance(ops):
    """A row's bits do not depend on how many rows share the launch, inside one kernel family: 2..8 rows run the
    same 8-token tile of the mma kernel; one row runs the SIMT GEMV, whose summation order differs (bf16 rounding)."""
    K, N = 5120, 2048
    x, w = rnd(8, K, seed=1), rnd(N, K, scale=0.05, seed=2)
    y8 = ops.linear(x, w)
    for m in (2, 4, 7):
        assert torch.equal(ops.linear(x[:m].contiguous(), w), y8[:m])
    close(ops.linear(x[:1].contiguous(), w), y8[:1])


@pytest.mark.parametrize("M,N,K", [(16, 512, 256), (33, 1024, 5120), (64, 5120, 2048), (128, 512, 512),
                                   (300, 1000 // 8 * 8, 768), (2048, 6144, 5120), (512, 5120, 17408)])
def test_gemm_tcgen05(ops, tops, M, N, K):
    x, w = rnd(M, K, seed=1), rnd(N, K, scale=0.05, seed=2)
    res = rnd(M, N, seed=3)
    close(ops.linear(x, w), tops.linear(x, w))
    close(ops.linear(x, w, res=res), tops.linear(x, w, res=res))
    assert ops.status() == 0


@pytest.mark.parametrize("M", [24, 64, 200, 1024])
def test_gemm_tcgen05_swiglu(ops, tops, M):
    K, I = 1024, 1536
    x, w = rnd(M, K, seed=1), rnd(2 * I, K, scale=0.05, seed=2)
    close(ops.linear(x, w, swiglu=True), tops.linear(x, w, swiglu=True))
    assert ops.status() == 0


def test_gemm_determinism(ops):
    x, w = rnd(48, 5120, seed=1), rnd(5120, 5120, scale=0.05, seed=2)
    a = ops.linear(x, w)
    for _ in range(5):
        assert torch.equal(ops.linear(x, w), a)


def test_rmsnorm_embed_silu(ops, tops):
    x, w, r = rnd(37, 5120, seed=1), rnd(5120, scale=0.1, seed=2), rnd(37, 5120, seed=3)
    a, _ = ops.rmsnorm(x, w, 1e-6)
    b, _ = tops.rmsnorm(x, w, 1e-6)
    close(a, b)
    a, xa = ops.rmsnorm(x, w, 1e-6, res=r)
    b, xb = tops.rmsnorm(x, w, 1e-6, res=r)
    close(a, b)
    close(xa, xb)
    table = rnd(1000, 256, seed=5)
    ids = torch.randint(0, 1000, (19,), device=DEV, dtype=torch.int32)
    assert torch.equal(ops.embed(table, ids), table[ids.long()])
    gu = rnd(9, 2 * 768, seed=6)
    close(ops.silu_mul(gu), tops.silu_mul(gu))


@pytest.mark.parametrize("hd,nq,nkv,rot", [(64, 4, 2, 64), (256, 24, 4, 64), (128, 8, 2, 128), (256, 3, 1, 64),
                                           (128, 32, 8, 128)])          # 40 heads: more than one CTA's 32 warps per row
def test_attention_paged(ops, tops, hd, nq, nkv, rot):
    kv_block, n_slots, max_blocks = 64, 3, 8
    nb = n_slots * max_blocks
    gated = True
    width = nq * hd * 2 + 2 * nkv * hd
    bt = torch.arange(nb, device=DEV, dtype=torch.int32).view(n_slots, max_blocks).flip(0).contiguous()
    inv = (1e6 ** (-torch.arange(rot // 2, dtype=torch.float64) / (rot // 2))).float().to(DEV)
    qn, kn = rnd(hd, scale=0.1, seed=7), rnd(hd, scale=0.1, seed=8)
    kc = [torch.zeros(nb, kv_block, nkv, hd, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    vc = [torch.zeros_like(kc[0]) for _ in range(2)]
    # a 300-token prompt in slot 1, then rows of two slots in one step
    proj = rnd(300, width, seed=9)
    slot = torch.full((300,), 1, device=DEV, dtype=torch.int32)
    pos = torch.arange(300, device=DEV, dtype=torch.int32)
    qa = ops.attn_prep(proj, qn, kn, inv, slot, pos, bt, kc[0], vc[0], kv_block, nq, nkv, hd, rot, gated, 1e-6)
    qb = tops.attn_prep(proj, qn, kn, inv, slot, pos, bt, kc[1], vc[1], kv_block, nq, nkv, hd, rot, gated, 1e-6)
    close(qa, qb)
    close(kc[0], kc[1])
    assert torch.equal(vc[0], vc[1])
    kvlen = pos + 1
    for nsplit in (1, 4):
        oa = ops.attention(qa, proj, kc[0], vc[0], slot, kvlen, bt, kv_block, nq, nkv, hd, gated, nsplit=nsplit)
        ob = tops.attention(qb, proj, kc[1], vc[1], slot, kvlen, bt, kv_block, nq, nkv, hd, gated)
        close(oa, ob, atol=ATT_ATOL)
    # flash prefill kernel: the same rows as two segments (a resumed prompt with a 100-key prefix, and a fresh one)
    seg_slot = torch.tensor([1], device=DEV, dtype=torch.int32)
    for r0, n, p0 in ((0, 300, 0), (100, 200, 100), (290, 10, 290)):
        segs = [seg_slot, torch.tensor([r0], device=DEV, dtype=torch.int32),
                torch.tensor([n], device=DEV, dtype=torch.int32), torch.tensor([p0], device=DEV, dtype=torch.int32)]
        of = ops.attention_prefill(qa, proj, kc[0], vc[0], *segs, bt, kv_block, nq, nkv, hd, gated, n)
        close(of[r0:r0 + n], ob[r0:r0 + n], atol=ATT_ATOL)
    # tree mask: rows see the first 290 keys plus chosen later ones
    base = torch.full((300,), 290, device=DEV, dtype=torch.int32)
    mask = torch.full((300,), 0b1010010011, device=DEV, dtype=torch.int64)
    lens = torch.full((300,), 300, device=DEV, dtype=torch.int32)
    oa = ops.attention(qa[:8], proj[:8], kc[0], vc[0], slot[:8], lens[:8], bt, kv_block, nq, nkv, hd, gated,
                       row_base=base[:8], row_mask=mask[:8], nsplit=2)
    ob = tops.attention(qb[:8], proj[:8], kc[1], vc[1], slot[:8], lens[:8], bt, kv_block, nq, nkv, hd, gated,
                        row_base=base[:8], row_mask=mask[:8])
    close(oa, ob, atol=ATT_ATOL)
    assert ops.status() == 0


@pytest.mark.parametrize("nk,nv,dk,dv", [(4, 4, 64, 64), (16, 16, 128, 128), (2, 4, 128, 128)])
def test_gdn_conv_and_recurrence(ops, tops, nk, nv, dk, dv):
    conv_dim = 2 * nk * dk + nv * dv
    width = conv_dim + nv * dv + 2 * nv
    n_slots = 3
    T = 23
    proj = rnd(T, width, seed=1)
    conv_w = rnd(conv_dim, 4, scale=0.5, seed=2)
    A_log = rnd(nv, scale=0.3, seed=3, dtype=torch.float32)
    dtb = rnd(nv, scale=0.3, seed=4, dtype=torch.float32)
    gw = (rnd(dv, scale=0.1, seed=5).float() + 1).to(torch.bfloat16)
    seg_slot = torch.tensor([2, 0], device=DEV, dtype=torch.int32)
    seg_row0 = torch.tensor([0, 17], device=DEV, dtype=torch.int32)
    seg_n = torch.tensor([17, 6], device=DEV, dtype=torch.int32)
    st = []
    for _ in range(2):
        st.append((rnd(n_slots, nv, dk, dv, scale=0.2, seed=6, dtype=torch.float32),
                   rnd(n_slots, 3, conv_dim, seed=7)))
    qa = ops.gdn_conv(proj, conv_w, st[0][1], seg_slot, seg_row0, seg_n, conv_dim, max_rows=17)
    qb = tops.gdn_conv(proj, conv_w, st[1][1], seg_slot, seg_row0, seg_n, conv_dim)
    close(qa, qb)
    # feed both recurrences the same conv output so only the recurrence is compared
    for commit in (False, True):
        ya = ops.gdn_rec(qa, proj, st[0][0], st[0][1], A_log, dtb, seg_slot, seg_row0, seg_n, nk, nv, dk, dv, 1e-6, commit=commit)
        yb = tops.gdn_rec(qa, proj, st[1][0], st[1][1], A_log, dtb, seg_slot, seg_row0, seg_n, nk, nv, dk, dv, 1e-6, commit=commit)
        close(ya, yb, atol=5e-3)
        close(st[0][0], st[1][0], atol=5e-3)
        assert torch.equal(st[0][1], st[1][1])
    oa = ops.gated_norm(ya, proj, conv_dim, gw, nv, dv, 1e-6)
    ob = tops.gated_norm(ya, proj, conv_dim, gw, nv, dv, 1e-6)
    close(oa, ob)


def test_verify_rows_carry_the_bits_of_decode_rows(ops):
    """A row computed inside a multi-row (verify) segment equals, bit for bit, the same row computed as a one-row decode
    step after its predecessors were committed: the Gated DeltaNet step kernel (conv window, delta rule and gated norm
    run row after row with the state in registers) and the split-KV decode attention (a row's keys, their order and the
    split boundaries do not depend on the rows that share its tile)."""
    nk, nv, dk, dv = 4, 8, 128, 128
    conv_dim = 2 * nk * dk + nv * dv
    width = conv_dim + nv * dv + 2 * nv
    T = 9
    proj = rnd(T, width, seed=1)
    conv_w = rnd(conv_dim, 4, scale=0.5, seed=2)
    A_log = rnd(nv, scale=0.3, seed=3, dtype=torch.float32)
    dtb = rnd(nv, scale=0.3, seed=4, dtype=torch.float32)
    gw = (rnd(dv, scale=0.1, seed=5).float() + 1).to(torch.bfloat16)
    i32 = lambda *v: torch.tensor(list(v), device=DEV, dtype=torch.int32)
    rec = [rnd(2, nv, dk, dv, scale=0.2, seed=6, dtype=torch.float32) for _ in range(2)]
    conv = [rnd(2, 3, conv_dim, seed=7) for _ in range(2)]
    whole = ops.gdn_step(proj, conv_w, rec[0], conv[0], A_log, dtb, gw, i32(1), i32(0), i32(T), nk, nv, dk, dv, 1e-6, commit=True)
    rows = [ops.gdn_step(proj[r:r + 1].contiguous(), conv_w, rec[1], conv[1], A_log, dtb, gw, i32(1), i32(0), i32(1), nk, nv, dk,
                         dv, 1e-6, commit=True) for r in range(T)]
    assert torch.equal(whole, torch.cat(rows))
    assert torch.equal(rec[0], rec[1]) and torch.equal(conv[0], conv[1])

    hd, nq, nkv, rot, kv_block = 256, 8, 2, 64, 64
    nb, ctx = 8, 200
    aw = nq * hd * 2 + 2 * nkv * hd
    bt = torch.arange(nb, device=DEV, dtype=torch.int32).view(1, nb)
    inv = (1e6 ** (-torch.arange(rot // 2, dtype=torch.float64) / (rot // 2))).float().to(DEV)
    qn, kn = rnd(hd, scale=0.1, seed=7), rnd(hd, scale=0.1, seed=8)
    kc = torch.zeros(nb, kv_block, nkv, hd, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    aproj = rnd(ctx + 5, aw, seed=9)
    slot = torch.zeros(ctx + 5, device=DEV, dtype=torch.int32)
    pos = torch.arange(ctx + 5, device=DEV, dtype=torch.int32)
    q = ops.attn_prep(aproj, qn, kn, inv, slot, pos, bt, kc, vc, kv_block, nq, nkv, hd, rot, True, 1e-6)
    # the last five rows as one verify segment ...
    r0 = ctx
    seg = (i32(0), i32(0), i32(5), 5)
    many = ops.attention(q[r0:].contiguous(), aproj[r0:].contiguous(), kc, vc, slot[r0:].contiguous(), (pos[r0:] + 1).contiguous(), bt,
                         kv_block, nq, nkv, hd, True, nsplit=2, segs=seg)
    # ... and one by one
    for i in range(5):
        one = ops.attention(q[r0 + i:r0 + i + 1].contiguous(), aproj[r0 + i:r0 + i + 1].contiguous(), kc, vc, slot[:1].contiguous(),
                            (pos[r0 + i:r0 + i + 1] + 1).contiguous(), bt, kv_block, nq, nkv, hd, True, nsplit=2,
                            segs=(i32(0), i32(0), i32(1), 1))
        assert torch.equal(one[0], many[i]), i
    assert ops.status() == 0


def test_argmax(ops):
    lg = rnd(5, 151936, seed=1, dtype=torch.float32)
    lg[2, 777] = 50.0
    lg[3, 5] = lg[3, 100] = 60.0
    ids, finite = ops.argmax(lg)
    assert ids.tolist() == lg.argmax(-1).tolist()
    assert ids[3].item() == 5 and finite.tolist() == [1] * 5
    lg[4, 9] = float("nan")
    _, finite = ops.argmax(lg.to(torch.bfloat16))
    assert finite.tolist() == [1, 1, 1, 1, 0]


@pytest.mark.parametrize("M", [1, 2, 4, 8])
@pytest.mark.parametrize("N,K", [(512, 1024), (5120, 5120), (640, 17408), (1024, 2048)])
def test_gemv_nvfp4(ops, tops, M, N, K):
    from ferrite_b200.ops.qweight import quantize_weight
    x, w = rnd(M, K, seed=1), rnd(N, K, scale=0.05, seed=2)
    q = quantize_weight(w)
    # the quantiser itself: dequantised weights stay within fp4 error of the originals
    assert (q.dense.float() - w.float()).abs().max().item() <= 0.27 * w.float().abs().max().item()
    res = rnd(M, N, seed=3)
    nw = rnd(K, scale=0.1, seed=4)
    close(ops.linear(x, q), tops.linear(x, q))
    close(ops.linear(x, q, res=res, norm_w=nw), tops.linear(x, q, res=res, norm_w=nw))
    close(ops.linear(x, q, out_f32=True), tops.linear(x, q, out_f32=True))


@pytest.mark.parametrize("M", [1, 4])
def test_gemv_nvfp4_swiglu(ops, tops, M):
    from ferrite_b200.ops.qweight import quantize_weight
    K, I = 5120, 2048
    x, w = rnd(M, K, seed=1), rnd(2 * I, K, scale=0.03, seed=2)
    q = quantize_weight(w)
    nw = rnd(K, scale=0.1, seed=4)
    close(ops.linear(x, q, norm_w=nw, swiglu=True), tops.linear(x, q, norm_w=nw, swiglu=True))


@pytest.mark.parametrize("nk,nv", [(2, 2), (2, 4)])
def test_gdn_chunked_scan(ops, tops, nk, nv):
    """Chunked prompt scan against the row-by-row fp32 recurrence: whole chunks, a ragged tail, a one-row segment,
    non-zero starting state; outputs, committed state and conv tail."""
    dk = dv = 128
    conv_dim = 2 * nk * dk + nv * dv
    width = conv_dim + nv * dv + 2 * nv
    lens = [130, 64, 1, 37]
    T = sum(lens)
    proj = rnd(T, width, seed=11)
    qkv = rnd(T, conv_dim, seed=12)
    A_log = rnd(nv, scale=0.3, seed=3, dtype=torch.float32)
    dtb = rnd(nv, scale=0.3, seed=4, dtype=torch.float32)
    seg_slot = torch.tensor([3, 0, 2, 1], device=DEV, dtype=torch.int32)
    row0 = [0, 130, 194, 195]
    seg_row0 = torch.tensor(row0, device=DEV, dtype=torch.int32)
    seg_n = torch.tensor(lens, device=DEV, dtype=torch.int32)
    mk = lambda: (rnd(4, nv, dk, dv, scale=0.2, seed=6, dtype=torch.float32), rnd(4, 3, conv_dim, seed=7))
    sa, sb, sc = mk(), mk(), mk()
    ya = ops.gdn_rec(qkv, proj, sa[0], sa[1], A_log, dtb, seg_slot, seg_row0, seg_n, nk, nv, dk, dv, 1e-6, commit=True,
                     chunked=True, max_rows=max(lens))
    yb = ops.gdn_rec(qkv, proj, sb[0], sb[1], A_log, dtb, seg_slot, seg_row0, seg_n, nk, nv, dk, dv, 1e-6, commit=True)
    yc = tops.gdn_rec(qkv, proj, sc[0], sc[1], A_log, dtb, seg_slot, seg_row0, seg_n, nk, nv, dk, dv, 1e-6, commit=True)
    close(yb, yc, atol=5e-3)
    close(ya, yc, atol=5e-3, rtol=1e-2)
    close(sa[0], sc[0], atol=5e-3, rtol=1e-2)
    assert torch.equal(sa[1], sc[1])
    assert float((ya - yb).abs().max()) < 2e-3


def test_device_sampler_filters(ops):
    """The device sampler keeps exactly the host sampler's candidate set (top-k, then top-p inside it, then min-p) and
    draws from it with the right frequencies."""
    from ferrite_b200.engine.sampler import Sampling, dist
    V = 4096
    g = torch.Generator(device=DEV).manual_seed(3)
    logits = (torch.randn(1, V, generator=g, device=DEV) * 3.0)
    for sp in (Sampling(temperature=0.8, top_k=40, top_p=0.9), Sampling(temperature=1.0, top_k=0, top_p=0.7),
               Sampling(temperature=1.2, top_k=10, top_p=1.0), Sampling(temperature=1.0, min_p=0.05),
               Sampling(temperature=0.7, top_k=50, top_p=0.95, min_p=0.02)):
        p = dist(logits[0].cpu(), sp)
        support = set(torch.nonzero(p > 0).flatten().tolist())
        n = 512
        ids = ops.sample(logits.expand(n, V).contiguous(), [sp] * n, list(range(1000, 1000 + n)))
        torch.cuda.synchronize()
        drawn = ids.tolist()
        assert set(drawn) <= support, (sp, sorted(set(drawn) - support)[:5])
        top = int(p.argmax())
        freq = drawn.count(top) / n
        assert abs(freq - float(p[top])) < 0.08, (sp, freq, float(p[top]))


@pytest.mark.parametrize("M", [1, 4, 8])
def test_w4_affine_gemv(ops, M):
    N, K = 320, 1024
    g = torch.Generator().manual_seed(M)
    q = torch.randint(0, 16, (N, K), generator=g)
    scales = (torch.rand(N, K // 64, generator=g) * 0.02 + 0.001).to(torch.bfloat16)
    biases = (torch.randn(N, K // 64, generator=g) * 0.05).to(torch.bfloat16)
    packed = torch.zeros(N, K // 8, dtype=torch.int64)
    for j in range(8):
        packed |= q[:, j::8] << (4 * j)
    packed = packed.to(torch.int32) if packed.max() < 2 ** 31 else (packed - (packed >= 2 ** 31) * 2 ** 32).to(torch.int32)
    w = q.float() * scales.float().repeat_interleave(64, 1) + biases.float().repeat_interleave(64, 1)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    res = torch.randn(M, N, generator=g).to(torch.bfloat16)
    want = x.float() @ w.t() + res.float()
    got = ops.w4_gemv(x.to(DEV), packed.to(DEV), scales.to(DEV), biases.to(DEV), res.to(DEV)).float().cpu()
    assert (got - want).abs().max().item() < 2e-2 * max(1.0, want.abs().max().item())


def test_topk16(ops):
    V = 131072
    g = torch.Generator(device=DEV).manual_seed(5)
    logits = torch.randn(3, V, generator=g, device=DEV)
    logits[1, 1000:1020] = 7.5                       # ties: lower index first
    ids, vals = ops.topk16(logits)
    for r in range(3):
        lr = logits[r].cpu().tolist()
        order = sorted(range(V), key=lambda i: (-lr[i], i))[:16] if r == 1 else None
        tv, ti = torch.topk(logits[r], 16)
        assert torch.allclose(vals[r], tv)
        if r == 1:
            assert ids[r].tolist() == order
        else:
            assert ids[r].tolist() == ti.tolist()
    idb, _ = ops.topk16(logits.to(torch.bfloat16))
    assert idb.shape == (3, 16)


@pytest.mark.parametrize("M,N,K", [(1, 512, 1024), (8, 384, 2048), (48, 1024, 1024), (300, 640, 1536), (2048, 1024, 4096)])
def test_gemm_fp8(ops, M, N, K):
    """e4m3 x e4m3 on the tcgen05 f8f6f4 path against the fp32 product of the dequantised operands."""
    x, w = rnd(M, K, seed=1), rnd(N, K, scale=0.05, seed=2)
    res = rnd(M, N, seed=3)
    wq, ws = ops.quantize_weight_fp8(w)
    got = ops.linear_fp8(x, wq, ws, res=res)
    xs = (x.float().abs().amax(1) / 448.0).clamp_min(1e-12)
    xd = (x.float() / xs[:, None]).to(torch.float8_e4m3fn).float() * xs[:, None]
    wd = wq.view(torch.float8_e4m3fn).float() * ws[:, None]
    want = xd @ wd.t() + res.float()
    assert (got.float() - want).abs().max().item() < 2e-2 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("M", [4, 200])
def test_gemm_fp8_norm_swiglu(ops, tops, M):
    N, K = 512, 1024
    x, w, nw = rnd(M, K, seed=1), rnd(2 * N, K, scale=0.05, seed=2), rnd(K, scale=0.1, seed=3)
    wq, ws = ops.quantize_weight_fp8(w)
    got = ops.linear_fp8(x, wq, ws, norm_w=nw, swiglu=True)
    want = tops.linear(x, wq.view(torch.float8_e4m3fn).float() * ws[:, None], norm_w=nw, eps=1e-6, swiglu=True)
    err = (got.float() - want.float()).abs().max().item()
    assert err < 6e-2 * max(1.0, want.abs().max().item()), err        # includes the e4m3 rounding of the activations


@pytest.mark.parametrize("M", [2, 4, 8, 9, 17, 24, 32])
@pytest.mark.parametrize("N,K", [(512, 1024), (1000, 4096), (5120, 2176)])
def test_gemv_mma(ops, tops, M, N, K):
    """Few-row weight-streaming linear on mma.sync: plain + residual, RMSNorm prologue + SwiGLU, fp32 output."""
    x, w, r = rnd(M, K, seed=M), rnd(N, K, scale=0.03, seed=2), rnd(M, N, seed=3)
    assert ops.mma_gemv_rows[0] <= M <= ops.mma_gemv_rows[1]
    close(ops.linear(x, w, res=r), tops.linear(x, w, res=r))
    nw = rnd(K, scale=0.1, seed=4)
    wg = rnd(2 * N, K, scale=0.03, seed=5)
    close(ops.linear(x, wg, norm_w=nw, eps=1e-6, swiglu=True), tops.linear(x, wg, norm_w=nw, eps=1e-6, swiglu=True), rtol=3e-2, atol=3e-2)
    y32 = ops.linear(x, w, norm_w=nw, eps=1e-6, out_f32=True)
    assert y32.dtype == torch.float32
    close(y32, tops.linear(x, w, norm_w=nw, eps=1e-6, out_f32=True))
    assert torch.equal(ops.linear(x, w, res=r), ops.linear(x, w, res=r))


@pytest.mark.parametrize("M,N,K", [(40, 512, 1024), (300, 512, 2048), (2048, 1000, 512)])
def test_gemm_tcgen05_fp32_out(ops, tops, M, N, K):
    x, w = rnd(M, K, seed=1), rnd(N, K, scale=0.05, seed=2)
    y = ops.linear(x, w, out_f32=True)
    assert y.dtype == torch.float32
    want = tops.linear(x, w, out_f32=True)
    assert (y - want).abs().max().item() < 2e-3 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("nk,nv,dk,dv", [(2, 4, 128, 128), (2, 2, 64, 64)])
def test_gdn_tree_conv_and_recurrence(ops, tops, nk, nv, dk, dv):
    """Verify-tree GDN kernels against the host walk over parent links: two trees in one launch (one branching twice,
    one a plain chain written as a tree), non-zero slot state, and the tree-as-chain equal to the chain kernels."""
    from ferrite_b200.engine.executor import tree_layout
    conv_dim = 2 * nk * dk + nv * dv
    width = conv_dim + nv * dv + 2 * nv
    pa = [-1, 0, 0, 1, 2, 3, 2, 6, 0]
    pb = [-1, 0, 1, 2, 3]
    T = len(pa) + len(pb)
    proj = rnd(T, width, seed=21)
    conv_w = rnd(conv_dim, 4, scale=0.5, seed=2)
    A_log = rnd(nv, scale=0.3, seed=3, dtype=torch.float32)
    dtb = rnd(nv, scale=0.3, seed=4, dtype=torch.float32)
    seg_slot = torch.tensor([1, 2], device=DEV, dtype=torch.int32)
    seg_row0 = torch.tensor([0, len(pa)], device=DEV, dtype=torch.int32)
    seg_n = torch.tensor([len(pa), len(pb)], device=DEV, dtype=torch.int32)
    parent = torch.tensor(pa + pb, device=DEV, dtype=torch.int32)
    flags = torch.tensor(tree_layout(pa)[2] + tree_layout(pb)[2], device=DEV, dtype=torch.int32)
    rec = rnd(3, nv, dk, dv, scale=0.2, seed=6, dtype=torch.float32)
    conv = rnd(3, 3, conv_dim, seed=7)
    rec0, conv0 = rec.clone(), conv.clone()
    qa = ops.gdn_conv_tree(proj, conv_w, conv, seg_slot, seg_row0, seg_n, conv_dim, parent)
    qb = tops.gdn_conv_tree(proj, conv_w, conv, seg_slot, seg_row0, seg_n, conv_dim, parent)
    close(qa, qb)
    ya = ops.gdn_rec_tree(qa, proj, rec, A_log, dtb, seg_slot, seg_row0, seg_n, parent, flags, nk, nv, dk, dv, 1e-6)
    yb = tops.gdn_rec_tree(qa, proj, rec, A_log, dtb, seg_slot, seg_row0, seg_n, parent, flags, nk, nv, dk, dv, 1e-6)
    close(ya, yb, atol=5e-3)
    assert torch.equal(rec, rec0) and torch.equal(conv, conv0)             # read-only
    # the chain segment through the tree kernels equals the chain kernels (the recurrence bit for bit)
    qc = ops.gdn_conv(proj, conv_w, conv, seg_slot[1:], seg_row0[1:], seg_n[1:], conv_dim, max_rows=len(pb))
    close(qc[len(pa):], qa[len(pa):])
    yc = ops.gdn_rec(qa, proj, rec, conv, A_log, dtb, seg_slot[1:], seg_row0[1:], seg_n[1:], nk, nv, dk, dv, 1e-6, commit=False)
    assert torch.equal(yc[len(pa):], ya[len(pa):])


@pytest.mark.parametrize("hd,nq,nkv,gated", [(256, 6, 2, True), (128, 8, 2, False), (64, 4, 4, True)])
def test_attention_prefill_tcgen05_against_mma_sync_and_reference(ops, tops, hd, nq, nkv, gated):
    """The tcgen05/TMEM prompt-attention kernel against the mma.sync kernel and the fp32 reference: two segments of
    different slots in one launch (a 520-row chunk behind a 200-key prefix, and a fresh 333-row prompt whose last
    tiles are ragged), scattered pages."""
    kv_block, n_slots, max_blocks = 64, 2, 16
    nb = n_slots * max_blocks
    width = nq * hd * (2 if gated else 1) + 2 * nkv * hd
    g = torch.Generator().manual_seed(5)
    bt = torch.randperm(nb, generator=g).to(torch.int32).view(n_slots, max_blocks).to(DEV).contiguous()
    rot = 64
    inv = (1e6 ** (-torch.arange(rot // 2, dtype=torch.float64) / (rot // 2))).float().to(DEV)
    qn, kn = rnd(hd, scale=0.1, seed=7), rnd(hd, scale=0.1, seed=8)
    kc = torch.zeros(nb, kv_block, nkv, hd, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    # the prefix of slot 0, then the step's rows: slot 0 continues at 200, slot 1 starts at 0
    pre = rnd(200, width, seed=10)
    ops.attn_prep(pre, qn, kn, inv, torch.zeros(200, device=DEV, dtype=torch.int32),
                  torch.arange(200, device=DEV, dtype=torch.int32), bt, kc, vc, kv_block, nq, nkv, hd, rot, gated, 1e-6)
    T = 520 + 333
    proj = rnd(T, width, seed=11)
    slot = torch.cat([torch.zeros(520), torch.ones(333)]).to(DEV, torch.int32)
    pos = torch.cat([torch.arange(200, 720), torch.arange(333)]).to(DEV, torch.int32)
    q = ops.attn_prep(proj, qn, kn, inv, slot, pos, bt, kc, vc, kv_block, nq, nkv, hd, rot, gated, 1e-6)
    segs = [torch.tensor(v, device=DEV, dtype=torch.int32) for v in ([0, 1], [0, 520], [520, 333], [200, 0])]
    assert ops.attn_tc
    a = ops.attention_prefill(q, proj, kc, vc, *segs, bt, kv_block, nq, nkv, hd, gated, 520)
    ops.attn_tc = False
    try:
        b = ops.attention_prefill(q, proj, kc, vc, *segs, bt, kv_block, nq, nkv, hd, gated, 520)
    finally:
        ops.attn_tc = True
    c = tops.attention_prefill(q, proj, kc, vc, *segs, bt, kv_block, nq, nkv, hd, gated, 520)
    close(b, c, atol=ATT_ATOL)
    close(a, c, atol=ATT_ATOL)
    assert ops.status() == 0


@pytest.mark.parametrize("M,N,K", [(300, 384, 1024), (64, 200, 7168), (1, 128, 512), (513, 2048, 2048 + 64)])
def test_fp8_block_scaled_gemm(ops, M, N, K):
    """Block-scaled e4m3 GEMM (1 x 128 activation blocks, 128 x 128 weight blocks; per-k-block promotion out of TMEM)
    against an fp32 product of the dequantised operands; the quantiser against the torch rounding; ragged M, N and K."""
    x = rnd(M, K, seed=1)
    x[:, :K // 2] *= 8.0                                  # blocks with different scales along k
    w = rnd(N, K, scale=0.05, seed=2)
    w[: N // 2, K // 3:] *= 6.0
    wq, ws = ops.quantize_weight_fp8_block(w)
    xq, xs = ops.quantize_act_fp8_block(x)
    kb = (K + 127) // 128
    assert xq.shape == (M, kb * 128) and xs.shape == (M, kb)
    xp = torch.zeros(M, kb * 128, device=DEV)
    xp[:, :K] = x.float()
    want_s = (xp.view(M, kb, 128).abs().amax(-1) / 448.0)
    want_s = torch.where(want_s > 0, want_s, torch.ones_like(want_s))
    assert torch.allclose(xs, want_s, rtol=1e-6)
    xd = xq.view(torch.float8_e4m3fn).float().view(M, kb, 128) * xs[:, :, None]
    assert (xd.view(M, -1)[:, :K] - x.float()).abs().max().item() <= 0.07 * x.float().abs().max().item()
    nb = (N + 127) // 128
    wd = torch.zeros(nb * 128, kb * 128, device=DEV)
    wd[:N] = wq.view(torch.float8_e4m3fn).float()
    wd = (wd.view(nb, 128, kb, 128) * ws[:, None, :, None]).view(nb * 128, kb * 128)[:N]
    want = xd.view(M, -1) @ wd.t()
    res = rnd(M, N, seed=3)
    for r in (None, res):
        got = ops.linear_fp8_block(x, wq, ws, res=r).float()
        ref = want + (r.float() if r is not None else 0)
        assert (got - ref).abs().max().item() < 1e-2 * ref.abs().max().item() + 1e-2
    # and close to the unquantised product (quantisation noise only)
    full = x.float() @ w.float().t()
    rel = (want - full).norm() / full.norm()
    assert rel < 0.06
    assert ops.status() == 0


def test_drafter_sublayers(ops):
    """Block-drafter kernels against the host statements: grouped dynamic conv (plain and into a residual, coefficients
    as a column slice), merge of per-rank top-16 lists (ties to the lower id), candidate selector walk."""
    from ferrite_b200.ops.torch_ops import TorchOps
    tops = TorchOps("cpu", torch.float32)
    T, H, group, blk = 48, 5120, 16, 16
    G = H // group
    x = rnd(T, H, seed=1)
    wide = rnd(T, 4 * G, scale=0.3, seed=2)
    coef = wide[:, 2 * G:]                                  # one side's two taps out of a wider projection
    base = rnd(2, H, scale=0.5, seed=3)
    got = ops.dynconv(x, coef, base, group, blk)
    want = tops.dynconv(x.cpu(), coef.cpu(), base.cpu(), group, blk)
    assert (got.float().cpu() - want.float()).abs().max().item() < 2e-2 * max(1.0, want.abs().max().item())
    res = rnd(T, H, seed=4)
    want_r = tops.dynconv(x.cpu(), coef.cpu(), base.cpu(), group, blk, res=res.cpu().clone())
    got_r = ops.dynconv(x, coef, base, group, blk, res=res)
    assert got_r.data_ptr() == res.data_ptr()
    assert (got_r.float().cpu() - want_r.float()).abs().max().item() < 3e-2 * max(1.0, want_r.abs().max().item())
    # top-16 merge over 8 ranks with ties
    W, rows = 8, 5
    g = torch.Generator().manual_seed(0)
    vals = torch.randint(0, 40, (W, rows, 16), generator=g).float().sort(-1, descending=True).values
    ids = torch.stack([torch.stack([torch.randperm(1000, generator=g)[:16] + 1000 * w for _ in range(rows)]) for w in range(W)])
    ids = ids.to(torch.int32)
    ov, oi = ops.topk16_merge(vals.to(DEV), ids.to(DEV))
    wv, wi = tops.topk16_merge(vals, ids)
    assert torch.equal(ov.cpu(), wv) and torch.equal(oi.cpu(), wi)
    # selector walk
    V, R, n = 3000, 256, 12
    a_cb, b_cb = rnd(V, R, scale=0.3, seed=5), rnd(V, R, scale=0.3, seed=6)
    gate = rnd(n, R, seed=7)
    cv = torch.randn(n, 16, generator=g).to(DEV)
    ci = torch.stack([torch.randperm(V, generator=g)[:16] for _ in range(n)]).to(torch.int32).to(DEV)
    got = ops.draft_select(cv, ci, gate, a_cb, b_cb, 17)
    want = tops.draft_select(cv.cpu(), ci.cpu(), gate.cpu(), a_cb.cpu(), b_cb.cpu(), 17)
    assert got.cpu().tolist() == want.tolist()


@pytest.mark.parametrize("hd,nq,nkv,gated", [(256, 24, 4, True), (128, 8, 2, False), (64, 4, 4, True), (256, 3, 1, True)])
def test_attention_decode_mma_against_simt_and_reference(ops, tops, hd, nq, nkv, gated):
    """Tensor-core decode attention (rows of a segment packed with the q heads of a GQA group into the MMA's M) against
    the SIMT kernel and the fp32 reference: a 17-row verify segment behind 300 keys, single decode rows of two other
    slots with different lengths, a tree segment with ancestor masks; several split counts."""
    kv_block, n_slots, max_blocks = 64, 4, 8
    nb = n_slots * max_blocks
    width = nq * hd * (2 if gated else 1) + 2 * nkv * hd
    g = torch.Generator().manual_seed(3)
    bt = torch.randperm(nb, generator=g).to(torch.int32).view(n_slots, max_blocks).to(DEV).contiguous()
    rot = 64
    inv = (1e6 ** (-torch.arange(rot // 2, dtype=torch.float64) / (rot // 2))).float().to(DEV)
    qn, kn = rnd(hd, scale=0.1, seed=7), rnd(hd, scale=0.1, seed=8)
    kc = torch.zeros(nb, kv_block, nkv, hd, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    lens = {0: 300, 1: 77, 2: 410, 3: 129}
    for slot, n in lens.items():                               # the committed context of every slot
        ops.attn_prep(rnd(n, width, seed=10 + slot), qn, kn, inv, torch.full((n,), slot, device=DEV, dtype=torch.int32),
                      torch.arange(n, device=DEV, dtype=torch.int32), bt, kc, vc, kv_block, nq, nkv, hd, rot, gated, 1e-6)
    # step rows: 17 verify rows of slot 0, one decode row of slots 1 and 2, a 6-row tree of slot 3
    par = [-1, 0, 0, 1, 2, 2]
    depth = [0, 1, 1, 2, 2, 2]
    amask = [0b1, 0b11, 0b101, 0b1011, 0b10101, 0b100101]
    slot = torch.tensor([0] * 17 + [1, 2] + [3] * 6, device=DEV, dtype=torch.int32)
    pos = torch.tensor(list(range(300, 317)) + [77, 410] + [129 + d for d in depth], device=DEV, dtype=torch.int32)
    cpos = torch.tensor(list(range(300, 317)) + [77, 410] + list(range(129, 135)), device=DEV, dtype=torch.int32)
    kvlen = cpos + 1
    base = torch.tensor([300] * 17 + [77, 410] + [129] * 6, device=DEV, dtype=torch.int32)
    mask = torch.tensor([(1 << (i + 1)) - 1 for i in range(17)] + [1, 1] + amask, device=DEV, dtype=torch.int64)
    T = slot.numel()
    proj = rnd(T, width, seed=30)
    q = ops.attn_prep(proj, qn, kn, inv, slot, pos, bt, kc, vc, kv_block, nq, nkv, hd, rot, gated, 1e-6, row_cpos=cpos)
    segs = (torch.tensor([0, 1, 2, 3], device=DEV, dtype=torch.int32), torch.tensor([0, 17, 18, 19], device=DEV, dtype=torch.int32),
            torch.tensor([17, 1, 1, 6], device=DEV, dtype=torch.int32), 17)
    want = tops.attention(q, proj, kc, vc, slot, kvlen, bt, kv_block, nq, nkv, hd, gated, row_base=base, row_mask=mask)
    assert ops.attn_mma
    for nsplit in (1, 4, 16):
        a = ops.attention(q, proj, kc, vc, slot, kvlen, bt, kv_block, nq, nkv, hd, gated, row_base=base, row_mask=mask,
                          nsplit=nsplit, segs=segs)
        b = ops.attention(q, proj, kc, vc, slot, kvlen, bt, kv_block, nq, nkv, hd, gated, row_base=base, row_mask=mask,
                          nsplit=nsplit)
        close(b, want)
        close(a, want)
    # without masks (plain causal by kvlen)
    a = ops.attention(q, proj, kc, vc, slot, kvlen, bt, kv_block, nq, nkv, hd, gated, nsplit=8, segs=segs)
    close(a, tops.attention(q, proj, kc, vc, slot, kvlen, bt, kv_block, nq, nkv, hd, gated))
    assert ops.status() == 0


def test_hyper_connection_ops(ops):
    """Hyper-connection kernels (per-stream norm, gated mix, injection) against the host statements."""
    from ferrite_b200.ops.torch_ops import TorchOps
    tops = TorchOps("cpu", torch.float32)
    rows, hc, d = 37, 4, 2560
    res = rnd(rows, hc, d, seed=1, dtype=torch.float32)
    w = rnd(hc, d, seed=2, dtype=torch.float32) + 1.0
    gate = rnd(rows, hc, d, seed=3, dtype=torch.float32)
    y, inv = ops.hc_norm(res, w, 1e-6)
    wy, winv = tops.hc_norm(res.cpu(), w.cpu(), 1e-6)
    assert torch.allclose(inv.cpu(), winv, rtol=1e-5)
    assert (y.float().cpu() - wy).abs().max().item() < 2e-2 * wy.abs().max().item()
    m = ops.hc_mix(res, inv, w, gate)
    assert torch.allclose(m.cpu(), tops.hc_mix(res.cpu(), winv, w.cpu(), gate.cpu()), rtol=1e-4, atol=1e-5)
    out = rnd(rows, d, seed=4, dtype=torch.float32)
    wide = rnd(rows, 16, seed=5, dtype=torch.float32)
    inj = wide[:, 8:8 + hc]                                  # a column slice of a wider projection
    want = tops.hc_combine(res.cpu().clone(), out.cpu(), inj.cpu())
    got = ops.hc_combine(res, out, inj)
    assert torch.allclose(got.cpu(), want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("hd,nq,nkv", [(256, 24, 4), (128, 8, 2)])
def test_attention_decode_mma_fp8_cache(ops, hd, nq, nkv):
    """The tensor-core decode kernel over an e4m3 cache (byte tiles expanded in shared memory, per-key scales applied to
    the scores and to P) against the SIMT kernel on the same cache: a 9-row verify segment and two single rows."""
    kv_block, n_slots, max_blocks = 64, 3, 8
    nb = n_slots * max_blocks
    gated = True
    width = nq * hd * 2 + 2 * nkv * hd
    bt = torch.arange(nb, device=DEV, dtype=torch.int32).view(n_slots, max_blocks).flip(0).contiguous()
    rot = 64
    inv = (1e6 ** (-torch.arange(rot // 2, dtype=torch.float64) / (rot // 2))).float().to(DEV)
    qn, kn = rnd(hd, scale=0.1, seed=7), rnd(hd, scale=0.1, seed=8)
    kc = torch.zeros(nb, kv_block, nkv, hd, dtype=torch.uint8, device=DEV)
    vc = torch.zeros_like(kc)
    sc = torch.ones(nb, kv_block, nkv, 2, dtype=torch.float32, device=DEV)
    lens = {0: 200, 1: 333, 2: 70}
    for slot, n in lens.items():
        ops.attn_prep(rnd(n, width, seed=10 + slot), qn, kn, inv, torch.full((n,), slot, device=DEV, dtype=torch.int32),
                      torch.arange(n, device=DEV, dtype=torch.int32), bt, kc, vc, kv_block, nq, nkv, hd, rot, gated, 1e-6,
                      kv_scale=sc)
    slot = torch.tensor([0] * 9 + [1, 2], device=DEV, dtype=torch.int32)
    pos = torch.tensor(list(range(200, 209)) + [333, 70], device=DEV, dtype=torch.int32)
    kvlen = pos + 1
    proj = rnd(11, width, seed=30)
    q = ops.attn_prep(proj, qn, kn, inv, slot, pos, bt, kc, vc, kv_block, nq, nkv, hd, rot, gated, 1e-6, kv_scale=sc)
    i32 = lambda v: torch.tensor(v, device=DEV, dtype=torch.int32)
    segs = (i32([0, 1, 2]), i32([0, 9, 10]), i32([9, 1, 1]), 9)
    for nsplit in (1, 8):
        a = ops.attention(q, proj, kc, vc, slot, kvlen, bt, kv_block, nq, nkv, hd, gated, nsplit=nsplit, kv_scale=sc, segs=segs)
        b = ops.attention(q, proj, kc, vc, slot, kvlen, bt, kv_block, nq, nkv, hd, gated, nsplit=nsplit, kv_scale=sc)
        close(a, b)
    assert ops.status() == 0


def test_determinism_over_cross_cta_hand_offs(capsys):
    """Split-K sums, stream-K slots, split-KV combine and the chunked scan return the same bits run after run."""
    from ferrite_b200.utils.detcheck import main
    rc = main(["--reps", "6"])
    out = capsys.readouterr().out
    assert rc == 0, out


def test_canary_padded_output_buffers_catch_a_stray_write(ops):
    """Debug allocator: guard bytes around every output buffer; a decode-sized forward leaves them intact, a write one
    element past a buffer is reported at the next check."""
    ops.enable_canaries(True)
    try:
        x, w = rnd(3, 1024, seed=1), rnd(768, 1024, scale=0.05, seed=2)
        y = ops.linear(x, w, res=rnd(3, 768, seed=3))
        ops.silu_mul(rnd(3, 2 * 640, seed=4))
        assert ops.check_canaries() >= 2
        y = ops.linear(x, w)
        flat = y.untyped_storage()
        raw = torch.empty(0, dtype=torch.uint8, device=DEV).set_(flat)
        raw[256 + y.numel() * y.element_size()] = 0          # the byte right behind the data
        with pytest.raises(RuntimeError, match="canary"):
            ops.check_canaries()
    finally:
        ops.enable_canaries(False)
