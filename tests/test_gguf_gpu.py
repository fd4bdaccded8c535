"""GGUF block formats on the GPU against the host decoders (`formats/gguf.py::dequantize`): dequantisation of every
supported type, the q8_1 activation quantiser, and the dequantising GEMV."""
import numpy as np
import pytest
import torch

from ferrite_b200.formats.gguf import TYPES, TYPE_ID, dequantize

pytestmark = pytest.mark.gpu
DEV = "cuda"
NAMES = ["Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "IQ4_NL", "MXFP4", "Q4_K", "Q5_K", "Q6_K", "IQ4_XS"]
EXACT = ["Q2_K", "Q3_K", "IQ2_XXS", "IQ2_XS", "IQ2_S", "IQ3_XXS", "IQ3_S", "IQ1_S", "IQ1_M"]     # device == host bit for bit
HALF_FIELDS = {"Q8_0": [0], "Q4_0": [0], "Q4_1": [0, 2], "Q5_0": [0], "Q5_1": [0, 2], "IQ4_NL": [0], "Q4_K": [0, 2],
               "Q5_K": [0, 2], "Q6_K": [208], "IQ4_XS": [0], "Q2_K": [80, 82], "Q3_K": [108], "IQ2_XXS": [0], "IQ2_XS": [0],
               "IQ2_S": [0], "IQ3_XXS": [0], "IQ3_S": [0], "IQ1_S": [0]}


@pytest.fixture(scope="module")
def ops(ext):
    from ferrite_b200.ops.cuda_ops import CudaOps
    return CudaOps(DEV)


def random_blocks(name, n_blocks, seed):
    """Random bytes with the fp16 scale fields (and the MXFP4 exponent) set to finite, moderate values."""
    _, bv, bb = TYPES[TYPE_ID[name]]
    rng = np.random.default_rng(seed)
    raw = rng.integers(0, 256, size=(n_blocks, bb), dtype=np.uint8)
    for off in HALF_FIELDS.get(name, []):
        h = (rng.random(n_blocks).astype(np.float32) * 0.02 + 0.001).astype(np.float16)
        raw[:, off:off + 2] = h.view(np.uint8).reshape(n_blocks, 2)
    if name == "MXFP4":
        raw[:, 0] = rng.integers(118, 126, size=n_blocks, dtype=np.uint8)
    if name == "IQ1_M":
        # the fp16 super-block scale lives in the top nibbles of the four 16-bit scale words
        d = (rng.random(n_blocks).astype(np.float32) * 0.02 + 0.001).astype(np.float16).view(np.uint16)
        sc = raw[:, 48:56].view(np.uint16)
        for j in range(4):
            sc[:, j] = (sc[:, j] & 0x0FFF) | (((d >> (4 * j)) & 0xF) << 12)
    return raw.reshape(-1)


@pytest.mark.parametrize("name", NAMES)
def test_dequant_matches_host(ops, name):
    tid = TYPE_ID[name]
    _, bv, bb = TYPES[tid]
    raw = random_blocks(name, 96, seed=tid)
    want = torch.from_numpy(dequantize(raw, tid))
    got = ops.gguf_dequant(torch.from_numpy(raw).to(DEV), tid, (96 * bv,)).float().cpu()
    assert torch.allclose(got, want.to(torch.bfloat16).float(), rtol=1e-2, atol=1e-6), (got - want).abs().max()


@pytest.mark.parametrize("name", EXACT)
def test_codebook_and_small_k_quants_match_host_bit_for_bit(ops, name):
    """Q2_K, Q3_K and the codebook types: the device decoder rounds every product once, in the host decoder's order, so
    the bf16 results are identical (the host decoder itself is held to the `gguf` package in the CPU tests)."""
    tid = TYPE_ID[name]
    _, bv, bb = TYPES[tid]
    raw = random_blocks(name, 160, seed=100 + tid)
    want = torch.from_numpy(dequantize(raw, tid)).to(torch.bfloat16)
    got = ops.gguf_dequant(torch.from_numpy(raw).to(DEV), tid, (160 * bv,)).cpu()
    assert torch.equal(got, want), (got.float() - want.float()).abs().max()


@pytest.mark.parametrize("name", ["Q8_0", "Q4_0", "Q4_K", "Q6_K", "IQ4_XS", "Q2_K", "Q3_K", "IQ2_XXS", "IQ3_S", "IQ1_M"])
@pytest.mark.parametrize("M", [1, 3, 8])
def test_gemv_matches_dequantised_matmul(ops, name, M):
    tid = TYPE_ID[name]
    _, bv, bb = TYPES[tid]
    N, K = 192, 1024
    raw = random_blocks(name, N * K // bv, seed=tid + M)
    w = torch.from_numpy(dequantize(raw, tid)).view(N, K)
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    res = torch.randn(M, N, generator=g).to(torch.bfloat16)
    want = x.float() @ w.t() + res.float()
    got = ops.gguf_gemv(x.to(DEV), torch.from_numpy(raw).to(DEV), tid, N, res.to(DEV)).float().cpu()
    assert (got - want).abs().max().item() < 2e-2 * max(1.0, want.abs().max().item())


def test_q8_1_quant(ops):
    x = torch.randn(64 * 32, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    out = ops.q8_1_quant(x.to(DEV)).cpu().numpy().reshape(-1, 36)
    d = out[:, 0:2].copy().view(np.float16).astype(np.float32)[:, 0]
    s = out[:, 2:4].copy().view(np.float16).astype(np.float32)[:, 0]
    q = out[:, 4:].view(np.int8).astype(np.float32)
    xf = x.float().numpy().reshape(-1, 32)
    assert np.abs(q * d[:, None] - xf).max() <= np.abs(xf).max() / 127 * 0.51 + 1e-3
    assert np.allclose(s, d * q.sum(1), rtol=2e-3, atol=1e-3)


def test_engine_runs_from_gguf_blocks(ops, tmp_path):
    """A GGUF checkpoint in the engine: decode rows multiply the checkpoint's own Q8_0 blocks (dequantising GEMV), a
    prompt chunk goes through the dequantised scratch on the tensor-core GEMM; logits match the fp32 oracle over the
    dequantised tensors."""
    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment
    from ferrite_b200.formats.gguf_model import export_gguf, load_gguf_weights
    from ferrite_b200.models.weights import init_weights
    from ferrite_b200.ops.qweight import GgufWeight, StackWeight
    cfg = tiny_hybrid()
    path = str(tmp_path / "m.gguf")
    export_gguf(init_weights(cfg, seed=0), cfg, path, "Q8_0")
    eng = Engine(cfg, load_gguf_weights(path, cfg, torch.bfloat16), EngineConfig(n_slots=1, max_ctx=128), device=DEV)
    assert isinstance(eng.ex.w["l0.down"], GgufWeight) and isinstance(eng.ex.w["l0.in_proj"], (GgufWeight, StackWeight))
    ref = Engine(cfg, load_gguf_weights(path, cfg, torch.float32, dense=True), EngineConfig(n_slots=1, max_ctx=128), device="cpu")
    toks = torch.randint(0, cfg.vocab, (48,), generator=torch.Generator().manual_seed(4)).tolist()
    want, _, _ = ref.forward([Segment(0, 0, toks, "all")])
    got, _, _ = eng.forward([Segment(0, 0, toks[:40], "all")], greedy=False)
    rows = [got.float().cpu().clone()]
    for i in range(40, 48):
        lg, _, _ = eng.forward([Segment(0, i, [toks[i]], "last")], greedy=False)
        rows.append(lg.float().cpu().clone())
    kl = torch.nn.functional.kl_div(torch.log_softmax(torch.cat(rows), -1), torch.log_softmax(want, -1), log_target=True,
                                    reduction="batchmean").item()
    assert kl < 2e-2, kl
