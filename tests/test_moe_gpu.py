"""MoE kernels on the GPU: router (both forms, production expert counts), per-pair expert GEMVs, the grouped GEMM path for
prompt-sized batches, and the whole block inside the engine — each against the fp32 PyTorch statement of the op."""
import dataclasses

import pytest
import torch

from ferrite_b200.config import EngineConfig, ModelConfig, tiny_hybrid
from ferrite_b200.models.ref import RefModel, route
from ferrite_b200.ops.torch_ops import TorchOps

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops(ext):
    from ferrite_b200.ops.cuda_ops import CudaOps
    return CudaOps(DEV)


def rnd(*shape, scale=1.0, seed=0, dtype=torch.bfloat16):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=DEV) * scale).to(dtype)


@pytest.mark.parametrize("mode,E,K,ng,tg,scale", [(0, 512, 10, 1, 1, 1.0), (1, 256, 8, 8, 4, 2.5), (0, 32, 4, 1, 1, 1.0),
                                                  (1, 32, 4, 4, 2, 2.5)])
@pytest.mark.parametrize("T", [1, 7])
def test_router(ops, mode, E, K, ng, tg, scale, T):
    logits = rnd(T, E, scale=2.0, seed=T, dtype=torch.float32)
    bias = rnd(E, scale=0.1, seed=3, dtype=torch.float32) if mode == 1 else None
    ids, wts = ops.moe_route(logits, bias, mode, K, ng, tg, scale)
    cfg = ModelConfig(router="softmax" if mode == 0 else "sigmoid_group", top_k=K, n_groups=ng, topk_groups=tg,
                      route_scale=scale, n_experts=E)
    ri, rw = route(cfg, logits.cpu(), None if bias is None else bias.cpu())
    torch.cuda.synchronize()
    for t in range(T):
        got = dict(zip(ids[t].tolist(), wts[t].tolist()))
        want = dict(zip(ri[t].tolist(), rw[t].tolist()))
        assert set(got) == set(want), (t, sorted(got), sorted(want))
        for e in want:
            assert abs(got[e] - want[e]) < 1e-4 * max(1.0, scale)


@pytest.mark.parametrize("mode,E,K,ng,tg,scale", [(0, 512, 10, 1, 1, 1.0), (1, 256, 8, 8, 4, 2.5)])
def test_router_appends_the_shared_expert(ops, mode, E, K, ng, tg, scale):
    """Merged router | shared-gate logits (one more column): the first K picks equal the plain router's, pick K is the
    shared expert's stack entry weighted by the sigmoid of the last column (1 without a gate column)."""
    T = 5
    full = rnd(T, E + 1, scale=2.0, seed=9, dtype=torch.float32)
    bias = rnd(E, scale=0.1, seed=3, dtype=torch.float32) if mode == 1 else None
    ids0, wts0 = ops.moe_route(full[:, :E].contiguous(), bias, mode, K, ng, tg, scale)
    ids1, wts1 = ops.moe_route(full, bias, mode, K, ng, tg, scale, n_exp=E, shared_col=E, shared_id=E)
    assert ids1.shape == (T, K + 1) and torch.equal(ids1[:, :K], ids0) and torch.equal(wts1[:, :K], wts0)
    assert bool((ids1[:, K] == E).all()) and torch.allclose(wts1[:, K], torch.sigmoid(full[:, E]), atol=1e-6)
    _, wts2 = ops.moe_route(full[:, :E].contiguous(), bias, mode, K, ng, tg, scale, n_exp=E, shared_col=-1, shared_id=E)
    assert bool((wts2[:, K] == 1.0).all())


def test_shared_expert_as_a_pair_matches_separate_linears(ext, monkeypatch):
    """Decode rows of the tiny MoE models with the shared expert merged into the expert stacks against the same engine
    with the merge switched off."""
    from ferrite_b200.config import EngineConfig, tiny_mla
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment
    from ferrite_b200.models.weights import init_weights
    cfg = tiny_mla()
    w = init_weights(cfg, seed=0)
    p = torch.randint(0, cfg.vocab, (24,), generator=torch.Generator().manual_seed(5)).tolist()
    outs = []
    for merge in ("1", "0"):
        monkeypatch.setenv("FB_MOE_MERGE_SHARED", merge)
        eng = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=64), device=DEV)
        assert bool(eng.ex.moe_merged) == (merge == "1")
        eng.forward([Segment(0, 0, p[:16], "none")])
        outs.append(torch.cat([eng.forward([Segment(0, 16 + i, [p[16 + i]], "last")])[0].clone() for i in range(8)]).float())
        eng.check()
    kl = torch.nn.functional.kl_div(torch.log_softmax(outs[0], -1), torch.log_softmax(outs[1], -1), log_target=True,
                                    reduction="batchmean").item()
    assert kl < 1e-3, kl


@pytest.mark.parametrize("T", [1, 4, 16, 48])
@pytest.mark.parametrize("ep", [False, True])
def test_experts(ops, T, ep, monkeypatch):
    monkeypatch.setattr(ops, "moe_pair_rows", 16)
    E, K, H, I = 16, 4, 512, 256
    tops = TorchOps(DEV, torch.float32)
    h = rnd(T, H, seed=1)
    w_gu, w_dn = rnd(E, 2 * I, H, scale=0.05, seed=2), rnd(E, H, I, scale=0.05, seed=3)
    g = torch.Generator().manual_seed(T)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(DEV)
    wts = torch.rand(T, K, generator=g).to(DEV)
    shared, sgate, res = rnd(T, H, seed=4), rnd(T, 1, seed=5, dtype=torch.float32), rnd(T, H, seed=6)
    e_lo, e_hi = (8, 16) if ep else (0, 16)
    got = ops.moe_experts(h, ids, wts, w_gu[e_lo:e_hi].contiguous(), w_dn[e_lo:e_hi].contiguous(), e_lo, e_hi, shared, sgate,
                          res)
    want = tops.moe_experts(h, ids, wts, w_gu[e_lo:e_hi], w_dn[e_lo:e_hi], e_lo, e_hi, shared, sgate, res)
    err = (got.float() - want.float()).abs().max().item()
    assert err < 3e-2 * max(1.0, want.abs().max().item()), err


@pytest.mark.parametrize("router", ["softmax", "sigmoid_group"])
def test_moe_engine_gpu(ext, router):
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment
    from ferrite_b200.models.weights import init_weights
    kw = dict(n_groups=4, topk_groups=2, route_scale=2.5) if router == "sigmoid_group" else {}
    cfg = dataclasses.replace(tiny_hybrid(), n_experts=32, top_k=4, expert_inter=64, n_shared=1, router=router, **kw)
    w = init_weights(cfg, seed=0)
    ref = Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=128), device="cpu")
    p = torch.randint(0, cfg.vocab, (88,), generator=torch.Generator().manual_seed(1)).tolist()
    want, _, _ = ref.forward([Segment(0, 0, p, "all")])
    eng = Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=128), device=DEV)
    got, _, _ = eng.forward([Segment(0, 0, p[:80], "all")])          # grouped GEMM path
    tail = [eng.forward([Segment(0, 80 + i, [p[80 + i]], "last")])[0].clone() for i in range(8)]   # pair GEMV path
    got = torch.cat([got] + tail).float().cpu()
    # bf16 weights/activations against the fp32 oracle: compare distributions, not raw logits
    kl = torch.nn.functional.kl_div(torch.log_softmax(got, -1), torch.log_softmax(want, -1), log_target=True,
                                    reduction="batchmean").item()
    assert kl < 2e-2, kl


@pytest.mark.parametrize("T,E,K", [(300, 16, 4), (1000, 64, 8), (5, 16, 4)])
def test_ep_pipeline_one_rank(ops, T, E, K):
    """The expert-parallel kernels with a world of one (dispatch to self): plan, dispatch, grouped tcgen05 GEMMs and
    pulled combine against the pair-by-pair fp32 statement; run twice so flags and counters advance an epoch."""
    from ferrite_b200.parallel.ep import ExpertParallel
    H, I = 512, 256
    tops = TorchOps(DEV, torch.float32)
    ep = ExpertParallel(None, DEV, E, H, cap_rows=T * K)
    h = rnd(T, H, seed=1)
    w_gu, w_dn = rnd(E, 2 * I, H, scale=0.05, seed=2), rnd(E, H, I, scale=0.05, seed=3)
    g = torch.Generator().manual_seed(T)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(DEV)
    wts = torch.rand(T, K, generator=g).to(DEV)
    shared, sgate, res = rnd(T, H, seed=4), rnd(T, 1, seed=5, dtype=torch.float32), rnd(T, H, seed=6)
    want = tops.moe_experts(h, ids, wts, w_gu, w_dn, 0, E, shared, sgate, res)
    for _ in range(2):
        got = ep.moe(ops, h, ids, wts, w_gu, w_dn, shared, sgate, res)
        torch.cuda.synchronize()
        ep.check()
        err = (got.float() - want.float()).abs().max().item()
        assert err < 3e-2 * max(1.0, want.abs().max().item()), err


def test_moe_80b_widths_few_layers(ext):
    """The 80B-A3B layer shapes (hidden 2048, 512 experts, top-10, expert FFN 512, shared expert) on a 4-layer cut:
    a 300-token prompt (grouped tcgen05 expert GEMMs) and decode rows (pair GEMVs) agree with each other through
    the cache: decoding token t after a prompt of t tokens gives the logits of position t in a longer prompt."""
    from ferrite_b200.config import EngineConfig, moe_80b, scaled
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment
    cfg = scaled(moe_80b(), 4)
    eng = Engine(cfg, None, EngineConfig(n_slots=2, max_ctx=512), device=DEV, seed=0)
    p = torch.randint(0, cfg.vocab, (304,), generator=torch.Generator().manual_seed(1)).tolist()
    full, _, _ = eng.forward([Segment(0, 0, p, "all")], greedy=False)
    eng.forward([Segment(1, 0, p[:300], "none")])
    tail = [eng.forward([Segment(1, 300 + i, [p[300 + i]], "last")], greedy=False)[0].clone() for i in range(4)]
    got = torch.cat(tail).float()
    want = full[300:304].float()
    kl = torch.nn.functional.kl_div(torch.log_softmax(got, -1), torch.log_softmax(want, -1), log_target=True,
                                    reduction="batchmean").item()
    assert kl < 2e-2, kl
    assert eng.ex.ep is not None and eng.ex.ep.calls > 0


@pytest.mark.parametrize("T", [1, 4, 16, 48])
@pytest.mark.parametrize("ep", [False, True])
def test_experts_nvfp4(ops, T, ep, monkeypatch):
    """NVFP4 expert stacks: decode rows through the 4-bit pair GEMVs, prompt-sized batches through the dequantiser and
    the grouped GEMM; both against fp32 math on the dequantised weights. 80B-A3B widths (hidden 2048, expert FFN 512)."""
    from ferrite_b200.ops.qweight import quantize_experts
    monkeypatch.setattr(ops, "moe_pair_rows", 16)
    E, K, H, I = 16, 4, 2048, 512
    tops = TorchOps(DEV, torch.float32)
    h = rnd(T, H, seed=1)
    w_gu, w_dn = rnd(E, 2 * I, H, scale=0.05, seed=2), rnd(E, H, I, scale=0.05, seed=3)
    g = torch.Generator().manual_seed(T)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(DEV)
    wts = torch.rand(T, K, generator=g).to(DEV)
    shared, sgate, res = rnd(T, H, seed=4), rnd(T, 1, seed=5, dtype=torch.float32), rnd(T, H, seed=6)
    e_lo, e_hi = (8, 16) if ep else (0, 16)
    q_gu, q_dn = quantize_experts(w_gu[e_lo:e_hi].contiguous()), quantize_experts(w_dn[e_lo:e_hi].contiguous())
    dense = ops.experts_dense(q_gu, 0)
    assert torch.equal(dense.float(), q_gu.dequantize(torch.bfloat16).float())          # the GPU dequantiser, bit for bit
    got = ops.moe_experts(h, ids, wts, q_gu, q_dn, e_lo, e_hi, shared, sgate, res)
    want = tops.moe_experts(h, ids, wts, q_gu, q_dn, e_lo, e_hi, shared, sgate, res)
    err = (got.float() - want.float()).abs().max().item()
    assert err < 3e-2 * max(1.0, want.abs().max().item()), err


def test_moe_engine_nvfp4_experts(ext):
    """The MoE engine with `weight_dtype="nvfp4-a16"`: routed experts are held in NVFP4 only (no dense copy); prompt and
    decode steps agree with the CPU engine quantised the same way."""
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment
    from ferrite_b200.models.weights import init_weights
    from ferrite_b200.ops.qweight import ExpertsFP4
    cfg = dataclasses.replace(tiny_hybrid(), n_experts=32, top_k=4, expert_inter=64, n_shared=1)
    w = init_weights(cfg, seed=0)
    ecfg = EngineConfig(n_slots=2, max_ctx=128, weight_dtype="nvfp4-a16")
    ref = Engine(cfg, w, ecfg, device="cpu")
    p = torch.randint(0, cfg.vocab, (88,), generator=torch.Generator().manual_seed(1)).tolist()
    want, _, _ = ref.forward([Segment(0, 0, p, "all")])
    eng = Engine(cfg, w, ecfg, device=DEV)
    assert isinstance(eng.ex.w["l0.experts_down"], ExpertsFP4)
    got, _, _ = eng.forward([Segment(0, 0, p[:80], "all")], greedy=False)
    tail = [eng.forward([Segment(0, 80 + i, [p[80 + i]], "last")], greedy=False)[0].clone() for i in range(8)]
    got = torch.cat([got] + tail).float().cpu()
    kl = torch.nn.functional.kl_div(torch.log_softmax(got, -1), torch.log_softmax(want.float(), -1), log_target=True,
                                    reduction="batchmean").item()
    assert kl < 2e-2, kl
    eng.check()
