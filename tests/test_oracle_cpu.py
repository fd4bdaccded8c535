"""The fp32 PyTorch statements of the ops (the oracle of every kernel test) against plain C++ double-precision loops
(`csrc/host_oracle.cpp`): an error in a PyTorch statement cannot hide behind a kernel that reproduces it."""
import math

import pytest
import torch

from ferrite_b200 import _ext
from ferrite_b200.formats import nvfp4
from ferrite_b200.ops.torch_ops import TorchOps

H = _ext.host()
pytestmark = pytest.mark.skipif(H is None or not hasattr(H, "oracle_linear"), reason="extension not built")
OPS = TorchOps("cpu", torch.float32)


def _r(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


@pytest.mark.parametrize("swiglu,norm,res", [(False, False, False), (True, True, False), (False, True, True)])
def test_linear_statement(swiglu, norm, res):
    M, K, N = 5, 96, 40
    x, w = _r(M, K, seed=1), _r(2 * N if swiglu else N, K, seed=2, scale=K ** -0.5)
    nw = _r(K, seed=3, scale=0.1) if norm else None
    rs = _r(M, N, seed=4) if res else None
    got = OPS.linear(x, w, norm_w=nw, eps=1e-6, res=rs, swiglu=swiglu, out_f32=True)
    want = H.oracle_linear(x, w, nw, 1e-6, rs, swiglu)
    assert torch.allclose(got, want, atol=2e-5, rtol=1e-5), (got - want).abs().max()


def test_attention_statement():
    nq, nkv, hd, kvb, T = 6, 2, 32, 16, 7
    nblk = 4
    kc, vc = _r(nblk, kvb, nkv, hd, seed=5), _r(nblk, kvb, nkv, hd, seed=6)
    bt = torch.tensor([[2, 0, 3, 1]], dtype=torch.int32)            # the sequence's pages, out of order
    q = _r(T, nq * hd, seed=7)
    kvlen = torch.tensor([1, 5, 16, 17, 40, 63, 64], dtype=torch.int32)
    slot = torch.zeros(T, dtype=torch.int32)
    got = OPS.attention(q, q, kc, vc, slot, kvlen, bt, kvb, nq, nkv, hd, False).view(T, nq, hd)
    k_seq = kc[bt[0].long()].reshape(nblk * kvb, nkv, hd).contiguous()
    v_seq = vc[bt[0].long()].reshape(nblk * kvb, nkv, hd).contiguous()
    want = H.oracle_attention(q.view(T, nq, hd).contiguous(), k_seq, v_seq, kvlen)
    assert torch.allclose(got, want, atol=2e-5, rtol=1e-5), (got - want).abs().max()


def test_gated_delta_rule_statement():
    nk, nv, dk, dv, T = 2, 4, 16, 8, 9
    conv_dim = 2 * nk * dk + nv * dv
    qkv = _r(T, conv_dim, seed=8)
    proj = torch.cat([_r(T, conv_dim, seed=9), _r(T, nv * dv, seed=10), _r(T, 2 * nv, seed=11)], 1)     # [conv | z | b | a]
    state = _r(1, nv, dk, dv, seed=12, scale=0.3)
    conv_state = torch.zeros(1, 3, conv_dim)
    A_log, dt_bias = _r(nv, seed=13, scale=0.5), _r(nv, seed=14, scale=0.5)
    st = state.clone()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    got = OPS.gdn_rec(qkv, proj, st, conv_state, A_log, dt_bias, i32([0]), i32([0]), i32([T]), nk, nv, dk, dv, 1e-6, commit=True)
    b = proj[:, conv_dim + nv * dv:conv_dim + nv * dv + nv].contiguous()
    a = proj[:, conv_dim + nv * dv + nv:].contiguous()
    want, s_want = H.oracle_gdn(qkv, b, a, state[0].contiguous(), A_log, dt_bias, nk, nv, dk, dv, 1e-6)
    assert torch.allclose(got, want, atol=3e-5, rtol=1e-4), (got - want).abs().max()
    assert torch.allclose(st[0], s_want, atol=3e-5, rtol=1e-4)


def test_nvfp4_decode_statement():
    N, K, M = 24, 64, 3
    w = _r(N, K, seed=15, scale=0.05)
    q = nvfp4.quantize(w)
    x = _r(M, K, seed=16)
    want = H.oracle_nvfp4(x, q.packed.contiguous(), q.scales.view(torch.uint8).contiguous(), float(q.global_scale))
    got = x @ q.dequantize().float().t()
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-5), (got - want).abs().max()
    assert torch.allclose(nvfp4.ref_linear(x, q).float(), want, atol=1e-4, rtol=1e-4)
    # the format itself: every 4-bit code and every finite e4m3 scale decode as the tables say
    codes = torch.arange(16, dtype=torch.uint8)
    vals = nvfp4.e2m1_to_float(codes)
    assert vals.tolist() == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
