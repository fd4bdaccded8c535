"""MLA kernels on the GPU: latent-cache attention at the 671B-class head shape (latent 512 + rope 64) against the fp32
PyTorch statement, and the tiny MLA + MoE model through the engine against the CPU oracle."""
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


@pytest.mark.parametrize("L,R,nq", [(512, 64, 16), (64, 64, 4)])
@pytest.mark.parametrize("nsplit", [1, 4])
def test_mla_prep_and_attention(ops, L, R, nq, nsplit):
    tops = TorchOps(DEV, torch.float32)
    g = torch.Generator(device=DEV).manual_seed(L + nsplit)
    r = lambda *s, sc=1.0: (torch.randn(*s, generator=g, device=DEV) * sc).to(torch.bfloat16)
    dn, kvb, nslots, ctx = 128 if L == 512 else 32, 64, 2, 200
    nb = (ctx + kvb - 1) // kvb + 1
    cache_a = r(nslots * nb, kvb, L + R)
    cache_b = cache_a.clone().float()
    bt = torch.arange(nslots * nb, device=DEV, dtype=torch.int32).view(nslots, nb)
    T = 6
    q, kva = r(T, nq * (dn + R)), r(T, L + R)
    norm_w, w_uk_t = r(L, sc=0.1), r(nq, L, dn, sc=0.05)
    hr = R // 2
    inv = (1e4 ** (-torch.arange(hr, dtype=torch.float64) / hr)).float().to(DEV)
    slot = torch.tensor([0, 0, 0, 1, 1, 1], device=DEV, dtype=torch.int32)
    pos = torch.tensor([150, 151, 152, 90, 91, 92], device=DEV, dtype=torch.int32)
    qa = ops.mla_prep(q, kva, norm_w, w_uk_t, inv, slot, pos, bt, cache_a, kvb, nq, dn, L, R, 1e-6)
    qb = tops.mla_prep(q, kva, norm_w, w_uk_t, inv, slot, pos, bt, cache_b, kvb, nq, dn, L, R, 1e-6)
    assert (qa.float() - qb.float()).abs().max().item() < 3e-2 * max(1.0, qb.abs().max().item())
    assert (cache_a.float() - cache_b).abs().max().item() < 3e-2
    kvlen = (pos + 1).contiguous()
    scale = 1.0 / math.sqrt(dn + R)
    oa = ops.mla_attention(qa, cache_a, slot, kvlen, bt, kvb, nq, L, R, scale, nsplit=nsplit)
    ob = tops.mla_attention(qa, cache_a, slot, kvlen, bt, kvb, nq, L, R, scale)
    assert (oa.float() - ob.float()).abs().max().item() < 2e-2


@pytest.mark.parametrize("T", [1, 6, 8, 19, 300])
@pytest.mark.parametrize("nh,N,K", [(16, 512, 128), (16, 128, 512), (4, 64, 32), (3, 40, 64)])
def test_head_linear_row_kernel_and_batched_gemm(ops, T, nh, N, K):
    """Per-head linears of the latent attention: <= 8 rows (and shapes the tensor-core tiles do not take) run the row
    kernel, more rows the batched tcgen05 GEMM; x is a strided view (the query's nope part), y a strided slice."""
    tops = TorchOps(DEV, torch.float32)
    g = torch.Generator(device=DEV).manual_seed(T * 131 + N)
    pad = 64
    xfull = (torch.randn(T, nh, K + pad, generator=g, device=DEV)).to(torch.bfloat16)
    W = (torch.randn(nh, N, K, generator=g, device=DEV) * K ** -0.5).to(torch.bfloat16)
    x = xfull[:, :, :K]
    want = tops.head_linear(x, W)
    got = ops.head_linear(x, W)
    err = (got.float() - want).abs().max().item()
    assert err < 2e-2 * max(1.0, want.abs().max().item()), err
    yfull = torch.full((T, nh, N + 24), 7.0, device=DEV, dtype=torch.bfloat16)
    ops.head_linear(x, W, out=yfull[:, :, :N])
    assert torch.equal(yfull[:, :, :N], got) and bool((yfull[:, :, N:] == 7.0).all())
    assert ops.status() == 0


@pytest.mark.parametrize("nq,L,R,dn,dv", [(16, 512, 64, 128, 128), (4, 64, 64, 32, 32)])
def test_mla_expanded_prefill_matches_absorbed(ops, nq, L, R, dn, dv):
    """Prompt segments through the expanded form (kv_b GEMM over the context's latent rows, padded per-head K / V, tcgen05
    flash kernel) against the absorbed-form fp32 statement on the same latent cache: two segments, one of them continuing
    a context that is already in the cache."""
    tops = TorchOps(DEV, torch.float32)
    g = torch.Generator(device=DEV).manual_seed(nq + L)
    r = lambda *s, sc=1.0: (torch.randn(*s, generator=g, device=DEV) * sc).to(torch.bfloat16)
    kvb, nslots, nb = 64, 2, 4
    cache = torch.zeros(nslots * nb, kvb, L + R, dtype=torch.bfloat16, device=DEV)
    bt = torch.randperm(nslots * nb, generator=g, device=DEV).to(torch.int32).view(nslots, nb)
    norm_w, w_uk_t, w_uv = r(L, sc=0.1), r(nq, L, dn, sc=dn ** -0.5), r(nq, dv, L, sc=L ** -0.5)
    kv_b = torch.cat([w_uk_t.transpose(1, 2), w_uv], 1).reshape(nq * (dn + dv), L).contiguous()
    hr = R // 2
    inv = (1e4 ** (-torch.arange(hr, dtype=torch.float64) / hr)).float().to(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    # 70 earlier rows of slot 1
    ops.mla_prep(r(70, nq * (dn + R)), r(70, L + R), norm_w, w_uk_t, inv, i32([1] * 70), i32(list(range(70))), bt, cache, kvb,
                 nq, dn, L, R, 1e-6)
    segs = [(0, 0, 50), (1, 70, 90)]
    T = 140
    slot = i32([0] * 50 + [1] * 90)
    pos = i32(list(range(50)) + list(range(70, 160)))
    q, kva = r(T, nq * (dn + R)), r(T, L + R)
    qabs = ops.mla_prep(q, kva, norm_w, w_uk_t, inv, slot, pos, bt, cache, kvb, nq, dn, L, R, 1e-6)
    scale = 1.0 / math.sqrt(dn + R)
    ol = tops.mla_attention(qabs, cache, slot, (pos + 1).contiguous(), bt, kvb, nq, L, R, scale)
    want = tops.mla_out(ol, w_uv).float()
    got = ops.mla_attention_prefill(q, qabs, cache, kv_b, segs, i32([0, 50]), i32([50, 90]), i32([0, 70]), bt, kvb, nq, dn, dv,
                                    L, R).float()
    assert got.shape == want.shape
    err = (got - want).abs().max().item()
    assert err < 3e-2 * max(1.0, want.abs().max().item()), err
    assert ops.status() == 0


def test_mla_engine_prompt_chunks_gpu(ext):
    """The tiny MLA + MoE model with a 70-row prompt chunk (expanded tensor-core path), a 30-row chunk (absorbed rows) and
    decode steps against the CPU oracle."""
    from ferrite_b200.config import EngineConfig, tiny_mla
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment
    from ferrite_b200.models.weights import init_weights
    cfg = tiny_mla()
    w = init_weights(cfg, seed=0)
    p = torch.randint(0, cfg.vocab, (110,), generator=torch.Generator().manual_seed(2)).tolist()
    ref = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=128), device="cpu")
    want, _, _ = ref.forward([Segment(0, 0, p, "all")])
    eng = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=128), device=DEV)
    a, _, _ = eng.forward([Segment(0, 0, p[:70], "all")])
    b, _, _ = eng.forward([Segment(0, 70, p[70:100], "all")])
    tail = [eng.forward([Segment(0, 100 + i, [p[100 + i]], "last")])[0].clone() for i in range(10)]
    got = torch.cat([a.clone(), b.clone()] + tail).float().cpu()
    kl = torch.nn.functional.kl_div(torch.log_softmax(got, -1), torch.log_softmax(want, -1), log_target=True,
                                    reduction="batchmean").item()
    assert kl < 2e-2, kl
    eng.check()


def test_mla_engine_gpu(ext):
    from ferrite_b200.config import EngineConfig, tiny_mla
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment
    from ferrite_b200.models.weights import init_weights
    cfg = tiny_mla()
    w = init_weights(cfg, seed=0)
    p = torch.randint(0, cfg.vocab, (40,), generator=torch.Generator().manual_seed(1)).tolist()
    ref = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=128), device="cpu")
    want, _, _ = ref.forward([Segment(0, 0, p, "all")])
    eng = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=128), device=DEV)
    got, _, _ = eng.forward([Segment(0, 0, p[:30], "all")])
    tail = [eng.forward([Segment(0, 30 + i, [p[30 + i]], "last")])[0].clone() for i in range(10)]
    got = torch.cat([got] + tail).float().cpu()
    kl = torch.nn.functional.kl_div(torch.log_softmax(got, -1), torch.log_softmax(want, -1), log_target=True,
                                    reduction="batchmean").item()
    assert kl < 2e-2, kl
