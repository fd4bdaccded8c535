"""EXL3 kernels against the host float64 statement (`formats/exl3.py`): tile decode, rotations, decode-row GEMV and the
prompt path through the decoded W_hat."""
import numpy as np
import pytest
import torch

from ferrite_b200.formats.exl3 import Exl3Tensor

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops(ext):
    from ferrite_b200.ops.cuda_ops import CudaOps
    return CudaOps(DEV)


@pytest.mark.parametrize("bits", [2, 3, 4, 6, 8])
def test_decode_matches_host(ops, bits):
    from ferrite_b200.ops.exl3_linear import Exl3Linear
    t = Exl3Tensor.random(256, 384, bits, seed=bits)
    lin = Exl3Linear(t, ops)
    want = torch.from_numpy(t.w_hat().astype(np.float32)).t()              # [n, k]
    got = lin.w_hat_t.float().cpu()
    assert torch.equal(got, want.to(torch.bfloat16).float())


@pytest.mark.parametrize("bits", [3, 4])
@pytest.mark.parametrize("M", [1, 5, 8, 40, 200])
def test_linear_matches_host(ops, bits, M):
    from ferrite_b200.ops.exl3_linear import Exl3Linear
    k, n = 1024, 768
    t = Exl3Tensor.random(k, n, bits, seed=10 + bits)
    lin = Exl3Linear(t, ops)
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, k, generator=g).to(torch.bfloat16)
    res = torch.randn(M, n, generator=g).to(torch.bfloat16)
    want = t.linear(x.float()).float() + res.float()
    got = lin.forward(x.to(DEV), res.to(DEV)).float().cpu()
    scale = max(1.0, want.abs().max().item())
    assert (got - want).abs().max().item() < (2e-2 if M <= 8 else 4e-2) * scale
