"""Codecs and tilings of the quantised formats (CPU)."""
import torch

from ferrite_b200.formats import nvfp4


def test_e2m1_roundtrip_and_rounding():
    codes = torch.arange(16, dtype=torch.uint8)
    vals = nvfp4.e2m1_to_float(codes)
    assert vals.tolist() == [0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6]
    back = nvfp4._e2m1_codes(vals)
    assert (back & 7).tolist() == (codes & 7).tolist()
    # ties go to the even mantissa: 0.25 -> 0, 0.75 -> 1, 1.25 -> 1, 1.75 -> 2, 2.5 -> 2, 3.5 -> 4, 5 -> 4
    x = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0])
    assert nvfp4.e2m1_to_float(nvfp4._e2m1_codes(x)).tolist() == [0, 1, 1, 2, 2, 4, 4, 6]


def test_quantize_error_and_packing():
    g = torch.Generator().manual_seed(0)
    w = torch.randn(64, 256, generator=g) * 0.02
    q = nvfp4.quantize(w)
    assert q.packed.shape == (64, 128) and q.scales.shape == (64, 16)
    d = q.dequantize()
    rel = (d - w).abs().max() / w.abs().max()
    assert rel < 0.27
    # element 2i sits in the low nibble
    lo = nvfp4.e2m1_to_float(q.packed[:, :1] & 0xF)[:, 0] * q.scales[:, 0].float() * q.global_scale
    assert torch.allclose(lo, d[:, 0])


def test_gemv_scale_tiling_is_a_permutation():
    sc = torch.arange(3 * 320, dtype=torch.uint8).view(3, 320) % 200
    t = nvfp4.tile_scales_gemv(sc.view(torch.float8_e4m3fn))
    assert t.shape == (3, 512)
    # lane L, span u, block b of group g sits at g*256 + L*8 + u*2 + b and holds logical block g*256 + u*64 + L*2 + b
    for g, L, u, b in [(0, 0, 0, 0), (0, 5, 3, 1), (1, 31, 0, 1), (0, 17, 2, 0)]:
        logical = g * 256 + u * 64 + L * 2 + b
        want = int(sc[1, logical]) if logical < 320 else 0
        assert int(t[1, g * 256 + L * 8 + u * 2 + b]) == want


def test_mma_scale_tiling_shape():
    sc = torch.ones(200, 40, dtype=torch.uint8).view(torch.float8_e4m3fn)
    t = nvfp4.tile_scales_mma(sc)
    assert t.shape == (2, 10, 512)
