"""The allocation-free decode-attention entry point, called through its exported C symbol (ctypes), against the regular
entry point with caller-provided scratch. Collected last on purpose (file name): it must pass both in a fresh process
and after every other GPU test has used the device."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _lib():
    import ferrite_b200._ext as ext          # loads torch's libraries and the extension first
    ext.load()
    lib = ctypes.CDLL(str(ext.so_path()))
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_long
    lib.fb_attn_decode_static.restype = i32
    lib.fb_attn_decode_static.argtypes = [vp, vp, vp, vp, vp, i64, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32,
                                          i32, i32, vp]
    lib.fb_attn_decode.restype = i32
    lib.fb_attn_decode.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32,
                                   i32, i32, vp]
    lib.fb_attn_decode_static_error.restype = ctypes.c_char_p
    lib.fb_attn_decode_static_scratch_bytes.restype = i64
    lib.fb_attn_decode_static_need_bytes.restype = i64
    lib.fb_attn_decode_static_need_bytes.argtypes = [i32, i32, i32, i32]
    return lib


def _case(rows, ctx, nsplit, seed, nq=8, nkv=2, hd=128, kvb=64):
    g = torch.Generator(device=DEV).manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, device=DEV).to(torch.bfloat16)
    nslots = 2
    nb = (ctx + kvb - 1) // kvb
    kc, vc = r(nslots * nb, kvb, nkv, hd), r(nslots * nb, kvb, nkv, hd)
    bt = torch.arange(nslots * nb, device=DEV, dtype=torch.int32).view(nslots, nb).contiguous()
    q = r(rows, nq, hd)
    proj = r(rows, nq * hd * 2 + 2 * nkv * hd)
    slot = (torch.arange(rows, device=DEV, dtype=torch.int32) % nslots).contiguous()
    kvlen = torch.tensor([ctx - 3 * i for i in range(rows)], device=DEV, dtype=torch.int32)
    return dict(q=q, kc=kc, vc=vc, proj=proj, slot=slot, kvlen=kvlen, bt=bt, nb=nb, kvb=kvb, rows=rows, nq=nq, nkv=nkv,
                hd=hd, nsplit=nsplit)


def _run(lib, c, static, gated=1):
    out = torch.zeros(c["rows"], c["nq"] * c["hd"], dtype=torch.bfloat16, device=DEV)
    s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    common = (c["q"].data_ptr(), c["kc"].data_ptr(), c["vc"].data_ptr(), c["proj"].data_ptr(), c["proj"].stride(0),
              c["slot"].data_ptr(), c["kvlen"].data_ptr(), None, None, c["bt"].data_ptr(), c["nb"], c["kvb"], c["rows"],
              c["nq"], c["nkv"], c["hd"], c["nsplit"], gated, s)
    if static:
        rc = lib.fb_attn_decode_static(out.data_ptr(), *common)
        assert rc == 0, lib.fb_attn_decode_static_error().decode()
    else:
        n = c["rows"] * c["nq"] * c["nsplit"]
        o_part = torch.empty(n * c["hd"], dtype=torch.float32, device=DEV)
        ml_part = torch.empty(n * 2, dtype=torch.float32, device=DEV)
        rc = lib.fb_attn_decode(out.data_ptr(), o_part.data_ptr(), ml_part.data_ptr(), *common)
        assert rc == 0
    torch.cuda.synchronize()
    return out


def test_static_scratch_matches_regular_entry_point(ext):
    lib = _lib()
    assert lib.fb_attn_decode_static_scratch_bytes() == 8 << 20
    # two calls in a row with different shapes: the second finds the first one's partials in the shared array
    for rows, ctx, nsplit, seed in ((4, 700, 8, 1), (2, 300, 4, 2)):
        c = _case(rows, ctx, nsplit, seed)
        want = _run(lib, c, static=False)
        got = _run(lib, c, static=True)
        assert torch.isfinite(got.float()).all()
        assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        assert torch.equal(got, want)            # same kernels, same order of operations


def test_static_scratch_gated_head_dim_256(ext):
    """The 27B attention shape (head_dim 256, sigmoid output gate read from the projection row) and the ungated form."""
    lib = _lib()
    for gated in (1, 0):
        c = _case(3, 500, 8, 5 + gated, nq=6, nkv=1, hd=256)
        want = _run(lib, c, static=False, gated=gated)
        got = _run(lib, c, static=True, gated=gated)
        assert torch.isfinite(got.float()).all() and torch.equal(got, want)


def test_static_scratch_refuses_sizes_that_would_wrap(ext):
    lib = _lib()
    big = 2 ** 31 - 1
    assert lib.fb_attn_decode_static_need_bytes(big, big, 256, big) > lib.fb_attn_decode_static_scratch_bytes()
    assert lib.fb_attn_decode_static_need_bytes(-1, 1, 128, 1) == -1
    rc = lib.fb_attn_decode_static(None, None, None, None, None, 0, None, None, None, None, None, 1, 64, big, big, 8, 128,
                                   big, 1, None)
    assert rc == -1 and "outside" in lib.fb_attn_decode_static_error().decode()


def test_static_scratch_rejects_oversize(ext):
    lib = _lib()
    rows, nq, hd, nsplit = 64, 64, 256, 64
    assert lib.fb_attn_decode_static_need_bytes(rows, nq, hd, nsplit) > lib.fb_attn_decode_static_scratch_bytes()
    rc = lib.fb_attn_decode_static(None, None, None, None, None, 0, None, None, None, None, None, 1, 64, rows, nq, 8, hd,
                                   nsplit, 1, None)
    assert rc == -20                              # refused on the host before anything is launched
    msg = lib.fb_attn_decode_static_error().decode()
    assert "need" in msg and "holds" in msg
