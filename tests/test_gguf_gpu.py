"""GGUF block formats on the GPU against the host decoders (`formats/gguf.py::dequantize`): dequantisation of every
supported type, the q8_1 activation quantiser, and the dequantising GEMV."""
import numpy as np
import pytest
import torch

from ferrite_b200.formats.gguf import TYPES, TYPE_ID, dequantize

pytestmark = pytest.mark.gpu
DEV = "cuda"
NAMES = ["Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "IQ4_NL", "MXFP4", "Q4_K", "Q5_K", "Q6_K", "IQ4_XS"]
HALF_FIELDS = {"Q8_0": [0], "Q4_0": [0], "Q4_1": [0, 2], "Q5_0": [0], "Q5_1": [0, 2], "IQ4_NL": [0], "Q4_K": [0, 2],
               "Q5_K": [0, 2], "Q6_K": [208], "IQ4_XS": [0]}


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
    return raw.reshape(-1)


@pytest.mark.parametrize("name", NAMES)
def test_dequant_matches_host(ops, name):
    tid = TYPE_ID[name]
    _, bv, bb = TYPES[tid]
    raw = random_blocks(name, 96, seed=tid)
    want = torch.from_numpy(dequantize(raw, tid))
    got = ops.gguf_dequant(torch.from_numpy(raw).to(DEV), tid, (96 * bv,)).float().cpu()
    assert torch.allclose(got, want.to(torch.bfloat16).float(), rtol=1e-2, atol=1e-6), (got - want).abs().max()


@pytest.mark.parametrize("name", ["Q8_0", "Q4_0", "Q4_K", "Q6_K", "IQ4_XS"])
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
