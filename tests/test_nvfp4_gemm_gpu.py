"""Block-scaled NVFP4 tcgen05 GEMM and its activation quantiser against host decodes of the same codes."""
import pytest
import torch

from ferrite_b200.formats import nvfp4

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops(ext):
    from ferrite_b200.ops.cuda_ops import CudaOps
    o = CudaOps(DEV)
    o.fp4_act = True
    o.fp4_prompt = True      # block-scaled kernels for every row count
    o.fp4_terms = 0          # the tests below pin the single-rendering (W4A4) kernels; the few-row kernel has its own
    return o


@pytest.fixture(scope="module")
def ops_tc(ext):
    from ferrite_b200.ops.cuda_ops import CudaOps
    o = CudaOps(DEV)
    o.fp4_act = True
    return o


def rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=DEV) * scale).to(torch.bfloat16)


def untile(sf, rows, K):
    """Tiled activation scales [rt][K/64][32][4][4] back to [rows][K/16]."""
    rt, kt = (rows + 127) // 128, K // 64
    t = sf[:rt * kt * 512].view(rt, kt, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(rt * 128, kt * 4)
    return t[:rows]


def decode_act(codes, sf, rs, rows, K):
    lo = nvfp4.e2m1_to_float(codes & 0xF)
    hi = nvfp4.e2m1_to_float(codes >> 4)
    v = torch.stack([lo, hi], -1).reshape(rows, K)
    sc = untile(sf, rows, K).view(torch.float8_e4m3fn).float().repeat_interleave(16, 1)
    return v * sc * rs[:, None]


@pytest.mark.parametrize("M,K", [(1, 256), (5, 5120), (130, 1024)])
def test_activation_quantiser(ops, M, K):
    x = rnd(M, K, seed=1)
    codes, sf, rs = ops.quant_nvfp4(x)
    got = decode_act(codes, sf, rs, M, K)
    # same recipe on the host (per-row global scale)
    want = torch.stack([nvfp4.quantize(x[i:i + 1].float(), global_scale=float(rs[i])).dequantize()[0] for i in range(M)])
    assert torch.allclose(rs, x.float().abs().amax(1) / (6 * 448), rtol=1e-6)
    mism = (got != want).float().mean().item()
    assert mism < 5e-3, mism                      # identical up to rare rounding ties (device multiplies by 1/scale)
    assert (got - x.float()).abs().max().item() <= 0.3 * x.float().abs().max().item()


@pytest.mark.parametrize("M,N,K", [(1, 256, 256), (4, 5120, 5120), (16, 1024, 2048), (48, 5120, 17408),
                                   (128, 512, 512), (300, 1024, 768), (2048, 6144, 5120)])
def test_gemm_nvfp4(ops, M, N, K):
    from ferrite_b200.ops.qweight import quantize_weight
    x, w = rnd(M, K, seed=1), rnd(N, K, scale=0.05, seed=2)
    q = quantize_weight(w)
    res = rnd(M, N, seed=3)
    codes, sf, rs = ops.quant_nvfp4(x)
    xdq = decode_act(codes, sf, rs, M, K)
    want = xdq @ q.dense.float().t()
    got = ops.linear(x, q)
    err = (got.float() - want).abs().max().item() / want.abs().max().item()
    assert err < 1.5e-2, err
    got = ops.linear(x, q, res=res)
    err = (got.float() - (want + res.float())).abs().max().item() / want.abs().max().item()
    assert err < 1.5e-2, err
    assert ops.status() == 0


@pytest.mark.parametrize("M", [2, 24, 200])
def test_gemm_nvfp4_swiglu_norm(ops, M):
    from ferrite_b200.ops.qweight import quantize_weight
    K, I = 1024, 1536
    x, w, nw = rnd(M, K, seed=1), rnd(2 * I, K, scale=0.05, seed=2), rnd(K, scale=0.1, seed=4)
    q = quantize_weight(w)
    codes, sf, rs = ops.quant_nvfp4(x, nw, 1e-6)
    xdq = decode_act(codes, sf, rs, M, K)
    y = xdq @ q.dense.float().t()
    want = torch.nn.functional.silu(y[:, :I]) * y[:, I:]
    got = ops.linear(x, q, norm_w=nw, eps=1e-6, swiglu=True)
    err = (got.float() - want).abs().max().item() / want.abs().max().item()
    assert err < 2e-2, err
    assert ops.status() == 0


@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("N,K,swiglu", [(5120, 5120, False), (2048, 17408, False), (1536, 1024, True)])
def test_gemm_nvfp4_fused_quantiser(ops, M, N, K, swiglu):
    """Decode form: bf16 rows in, norm + quantisation inside the GEMM kernel; same result as quantise-then-GEMM."""
    from ferrite_b200.ops.qweight import quantize_weight
    x, nw = rnd(M, K, seed=1), rnd(K, scale=0.1, seed=4)
    w = rnd(2 * N if swiglu else N, K, scale=0.05, seed=2)
    q = quantize_weight(w)
    res = None if swiglu else rnd(M, N, seed=3)
    codes, sf, rs = ops.quant_nvfp4(x, nw, 1e-6)
    xdq = decode_act(codes, sf, rs, M, K)
    y = xdq @ q.dense.float().t()
    want = torch.nn.functional.silu(y[:, :N]) * y[:, N:] if swiglu else y + res.float()
    got = ops.linear(x, q, norm_w=nw, eps=1e-6, res=res, swiglu=swiglu)
    err = (got.float() - want).abs().max().item() / want.abs().max().item()
    assert err < 2e-2, err
    if not swiglu:
        got32 = ops.linear(x, q, norm_w=nw, eps=1e-6, out_f32=True)
        assert got32.dtype == torch.float32
        err = (got32 - y).abs().max().item() / y.abs().max().item()
        assert err < 2e-2, err
    # replays give identical bits (split-K partials are summed in split order)
    again = ops.linear(x, q, norm_w=nw, eps=1e-6, res=res, swiglu=swiglu)
    assert torch.equal(got, again)
    assert ops.status() == 0


def _normed(x, nw, eps=1e-6):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (1 + nw.float())
    return y.to(torch.bfloat16).float()


@pytest.mark.parametrize("M", [1, 2, 4, 8])
@pytest.mark.parametrize("N,K,swiglu,norm", [(5120, 5120, False, True), (2048, 17408, False, False), (1536, 1024, True, True),
                                             (1000, 768, False, False), (17408, 5120, True, True)])
def test_few_row_tensor_core_kernel(ops_tc, M, N, K, swiglu, norm):
    """Weights multiplied packed on the block-scaled tensor cores; activations as residual NVFP4 renderings. Against
    fp32 math on the dequantised weights and the un-quantised (normalised) activations: with three renderings the
    activation error is at the level of the bf16 output rounding."""
    from ferrite_b200.ops.qweight import quantize_weight
    ops = ops_tc
    x = rnd(M, K, seed=1)
    x[:, ::7] *= 8.0                                           # outliers, as real hidden states have
    nw = rnd(K, scale=0.1, seed=4) if norm else None
    w = rnd(2 * N if swiglu else N, K, scale=0.05, seed=2)
    q = quantize_weight(w)
    res = None if swiglu else rnd(M, N, seed=3)
    xin = _normed(x, nw) if norm else x.float()
    y = xin @ q.dense.float().t()
    want = torch.nn.functional.silu(y[:, :N]) * y[:, N:] if swiglu else y
    errs = {}
    for terms in (3, 2, 1):
        ops.fp4_terms = terms
        eff = int(ops.C.gemv_nvfp4_tc_terms(M, N, K, swiglu, terms))
        assert eff == min(terms, 8 // M)
        got = ops.linear(x, q, norm_w=nw, eps=1e-6, swiglu=swiglu, out_f32=not swiglu)
        errs[eff] = (got.float() - want).abs().max().item() / want.abs().max().item()
    ops.fp4_terms = 3
    assert errs[1] < 0.3, errs
    if 2 in errs:
        assert errs[2] < 4e-2 and errs[2] < errs[1], errs
    if 3 in errs:
        assert errs[3] < 8e-3 and errs[3] < errs[2], errs
    got = ops.linear(x, q, norm_w=nw, eps=1e-6, res=res, swiglu=swiglu)
    assert got.dtype == torch.bfloat16
    ref = want if swiglu else want + res.float()
    err = (got.float() - ref).abs().max().item() / ref.abs().max().item()
    tol = {1: 0.3, 2: 4e-2, 3: 1.5e-2}[min(3, 8 // M)]
    assert err < tol, err
    # replays give identical bits (partials are summed in CTA order), also with two CTAs per SM
    again = ops.linear(x, q, norm_w=nw, eps=1e-6, res=res, swiglu=swiglu)
    assert torch.equal(got, again)
    ops.fp4_tc_ctas = 2
    two = ops.linear(x, q, norm_w=nw, eps=1e-6, res=res, swiglu=swiglu)
    ops.fp4_tc_ctas = 1
    err = (two.float() - ref).abs().max().item() / ref.abs().max().item()
    assert err < tol, err
    assert ops.status() == 0
    assert int(ops._counters.abs().sum()) == 0                 # every tile's counter went back to zero


def test_few_row_kernel_row_scales(ops_tc):
    """Fused projections of a checkpoint carry one tensor scale per part: per-row alpha in the epilogue."""
    from ferrite_b200.ops.qweight import quantize_weight
    ops = ops_tc
    N, K = 2048, 1024
    x = rnd(2, K, seed=1)
    q = quantize_weight(rnd(N, K, scale=0.05, seed=2))
    alpha = torch.full((N,), float(q.global_scale), device=DEV)
    alpha[N // 2:] *= 3.0
    base = ops.linear(x, q, out_f32=True)
    q.row_alpha = alpha
    got = ops.linear(x, q, out_f32=True)
    want = base.clone()
    want[:, N // 2:] *= 3.0
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-6)
    assert ops.status() == 0


@pytest.mark.parametrize("mode", ["bf16", "nvfp4", "nvfp4-w4a4"])
def test_engine_from_a_modelopt_nvfp4_checkpoint(ext, tmp_path, mode):
    """A ModelOpt NVFP4 checkpoint goes from file to kernels packed: decode rows stream the codes through the NVFP4
    GEMV with one tensor scale per output row (fused q|k|v and gate|up parts bring their own `weight_scale_2`), prompt
    rows take the dequantised copy (or, with weight_dtype nvfp4-w4a4, the block-scaled tensor-core GEMM where a single
    tensor scale allows it); with weight_dtype nvfp4 the decode rows run on the few-row tensor-core kernel. Logits match the fp32 oracle over the dequantised weights."""
    import dataclasses
    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment
    from ferrite_b200.formats import modelopt
    from ferrite_b200.formats.loader import export_hf, load_model_weights
    from ferrite_b200.models.weights import init_weights
    from ferrite_b200.ops.qweight import QWeight
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0)
    hf = export_hf(w, cfg)
    quantised = [k[:-len(".weight")] for k in hf if k.endswith("_proj.weight") or ".in_proj_qkv." in k or ".in_proj_z." in k]
    quantised = [b for b in quantised if hf[b + ".weight"].shape[1] % 32 == 0 and hf[b + ".weight"].shape[0] >= 16]
    modelopt.save_checkpoint(hf, str(tmp_path), "NVFP4", quantised, exclude=["lm_head"])
    packed = load_model_weights(str(tmp_path), cfg, torch.bfloat16)
    dense = load_model_weights(str(tmp_path), cfg, torch.float32, dense=True)
    eng = Engine(cfg, packed, EngineConfig(n_slots=1, max_ctx=128, weight_dtype=mode), device=DEV)
    gu = eng.ex.w["l0.gate_up"]
    assert isinstance(gu, QWeight) and gu.kind == "nvfp4" and gu.row_alpha is not None      # two parts, two tensor scales
    assert isinstance(eng.ex.w["l0.down"], QWeight) and eng.ex.w["l0.down"].row_alpha is None
    ref = Engine(cfg, dense, EngineConfig(n_slots=1, max_ctx=128), device="cpu")
    toks = torch.randint(0, cfg.vocab, (48,), generator=torch.Generator().manual_seed(4)).tolist()
    want, _, _ = ref.forward([Segment(0, 0, toks, "all")])
    got, _, _ = eng.forward([Segment(0, 0, toks[:40], "all")], greedy=False)
    rows = [got.float().cpu().clone()]
    for i in range(40, 48):
        lg, _, _ = eng.forward([Segment(0, i, [toks[i]], "last")], greedy=False)
        rows.append(lg.float().cpu().clone())
    got = torch.cat(rows)
    kl = torch.nn.functional.kl_div(torch.log_softmax(got, -1), torch.log_softmax(want, -1), log_target=True,
                                    reduction="batchmean").item()
    assert kl < (0.3 if mode == "nvfp4-w4a4" else 2e-2), kl     # w4a4 also quantises the activations of prompt rows (one rendering)


@pytest.mark.parametrize("M,H,I", [(65, 512, 256), (300, 1024, 1536), (2048, 5120, 17408)])
def test_ffn_with_requantised_swiglu(ops, M, H, I):
    """gate|up GEMM whose epilogue writes the SwiGLU output as NVFP4 (static global scale) + down GEMM on those codes:
    (1) the codes decode to the SwiGLU of the first GEMM within fp4 rounding, (2) the block equals the down projection of
    the decoded activation, (3) fused and unfused blocks agree within the quantisation noise of the activation."""
    from ferrite_b200.ops.qweight import quantize_weight
    x = rnd(M, H, seed=1)
    norm_w = rnd(H, scale=0.1, seed=5)
    w_gu, w_down = quantize_weight(rnd(2 * I, H, scale=H ** -0.5, seed=2)), quantize_weight(rnd(H, I, scale=I ** -0.5, seed=3))
    res = rnd(M, H, seed=4)
    xq, xsf, rs = ops.quant_nvfp4(x, norm_w, 1e-6)
    codes = torch.empty(M, I // 2, dtype=torch.uint8, device=DEV)
    sf = torch.zeros(int(ops.C.nvfp4_sf_bytes(M, I)), dtype=torch.uint8, device=DEV)
    ars = torch.empty(M, dtype=torch.float32, device=DEV)
    ops.C.gemm_nvfp4_swiglu_q(codes, sf, ars, ops.fp4_act_gscale, xq, xsf, rs, w_gu.packed, w_gu.mma_scales,
                              w_gu.global_scale, ops.status_word)
    act = decode_act(codes, sf, ars, M, I)
    gu = decode_act(xq, xsf, rs, M, H) @ w_gu.dense.float().t()
    want_act = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    assert bool((ars == ops.fp4_act_gscale).all())
    rel = (act - want_act).norm().item() / want_act.norm().item()
    assert rel < 0.12, rel                                           # e2m1 with per-16 scales: about 9 % rms
    y = ops.ffn(x, w_gu, w_down, norm_w, 1e-6, res)
    want = act @ w_down.dense.float().t() + res.float()
    err = (y.float() - want).abs().max().item() / want.abs().max().item()
    assert err < 2e-2, err
    ops.fp4_fuse_requant = False
    try:
        y2 = ops.ffn(x, w_gu, w_down, norm_w, 1e-6, res)
    finally:
        ops.fp4_fuse_requant = True
    d = (y.float() - y2.float() ).norm().item() / (y2.float() - res.float()).norm().item()
    assert d < 0.2, d
    assert ops.status() == 0
