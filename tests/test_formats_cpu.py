"""Codecs and tilings of the quantised formats (CPU)."""
import pytest
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


def _ref_q4k_block(b):
    """Scalar restatement of ggml's dequantize_row_q4_K for one 144-byte block."""
    import numpy as np
    d, dmin = np.frombuffer(b[0:2], np.float16)[0].astype(np.float32), np.frombuffer(b[2:4], np.float16)[0].astype(np.float32)
    sc, qs = b[4:16], b[16:144]

    def sm(j):
        if j < 4:
            return sc[j] & 63, sc[j + 4] & 63
        return (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4), (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)
    y, is_, q = [], 0, 0
    for _ in range(4):
        s1, m1 = sm(is_); s2, m2 = sm(is_ + 1)
        y += [d * s1 * (qs[q + l] & 0xF) - dmin * m1 for l in range(32)]
        y += [d * s2 * (qs[q + l] >> 4) - dmin * m2 for l in range(32)]
        q += 32; is_ += 2
    return np.array(y, np.float32)


def _ref_q6k_block(b):
    import numpy as np
    ql, qh, sc = b[0:128].astype(np.int32), b[128:192].astype(np.int32), np.frombuffer(b[192:208], np.int8).astype(np.int32)
    d = np.frombuffer(b[208:210], np.float16)[0].astype(np.float32)
    y = np.zeros(256, np.float32)
    for n in range(2):
        for l in range(32):
            i = l // 16
            L, H, S, Y = ql[64 * n:], qh[32 * n:], sc[8 * n:], 128 * n
            q1 = ((L[l] & 0xF) | (((H[l] >> 0) & 3) << 4)) - 32
            q2 = ((L[l + 32] & 0xF) | (((H[l] >> 2) & 3) << 4)) - 32
            q3 = ((L[l] >> 4) | (((H[l] >> 4) & 3) << 4)) - 32
            q4 = ((L[l + 32] >> 4) | (((H[l] >> 6) & 3) << 4)) - 32
            y[Y + l], y[Y + l + 32] = d * S[i] * q1, d * S[i + 2] * q2
            y[Y + l + 64], y[Y + l + 96] = d * S[i + 4] * q3, d * S[i + 6] * q4
    return y


def test_gguf_reader_and_block_decoders(tmp_path):
    import numpy as np
    from ferrite_b200.formats import gguf
    r = np.random.default_rng(0)
    x = r.standard_normal((4, 64)).astype(np.float32)
    p = str(tmp_path / "t.gguf")
    gguf.write_gguf(p, {"general.architecture": "test", "n": 3, "names": ["a", "b"]},
                    {"w8": (gguf.quantize_q8_0(x), 8, [4, 64]), "w4": (gguf.quantize_q4_0(x), 2, [4, 64]),
                     "f": (x.view(np.uint8).reshape(-1), 0, [4, 64])})
    g = gguf.Gguf(p)
    assert g.meta["n"] == 3 and g.meta["names"] == ["a", "b"] and g.tensors["w8"].shape == [4, 64]
    assert torch.equal(g.get("f"), torch.from_numpy(x))
    assert (g.get("w8") - torch.from_numpy(x)).abs().max() < 0.02
    assert (g.get("w4") - torch.from_numpy(x)).abs().max() < 0.35
    # K-quants and friends: random block bytes (valid fp16 scales) against scalar restatements of the ggml decoders
    for name, ref in (("Q4_K", _ref_q4k_block), ("Q6_K", _ref_q6k_block)):
        tid = gguf.TYPE_ID[name]
        bb = gguf.TYPES[tid][2]
        blk = r.integers(0, 256, size=(3, bb), dtype=np.uint8)
        if name == "Q4_K":
            blk[:, 0:4] = np.array([0.01, 0.002], np.float16).view(np.uint8)
        else:
            blk[:, 208:210] = np.array([0.01], np.float16).view(np.uint8)
        got = gguf.dequantize(blk.reshape(-1), tid).reshape(3, 256)
        want = np.stack([ref(blk[i]) for i in range(3)])
        assert np.allclose(got, want, rtol=1e-6, atol=1e-7), name
    # 4-bit codebook types: every code of IQ4_NL / MXFP4 decodes to its table value times the scale
    blk = np.zeros((1, 18), np.uint8); blk[0, :2] = np.array([0.5], np.float16).view(np.uint8); blk[0, 2:] = np.arange(16) | (np.arange(16)[::-1] << 4)
    got = gguf.dequantize(blk.reshape(-1), gguf.TYPE_ID["IQ4_NL"])
    assert np.allclose(got[:16], 0.5 * gguf.KVALUES_IQ4NL) and np.allclose(got[16:], 0.5 * gguf.KVALUES_IQ4NL[::-1])
    blk = np.zeros((1, 17), np.uint8); blk[0, 0] = 128; blk[0, 1:] = np.arange(16)
    assert np.allclose(gguf.dequantize(blk.reshape(-1), gguf.TYPE_ID["MXFP4"])[:16], gguf.KVALUES_MXFP4)   # 2^(128-127)/2 = 1
    with pytest.raises(NotImplementedError):
        gguf.dequantize(np.zeros(292, np.uint8), gguf.TYPE_ID["Q8_K"])       # an activation-side type: never in a checkpoint


def test_exl3_decode_reconstruct_and_slices():
    import numpy as np
    from ferrite_b200.formats.exl3 import Exl3Tensor
    t = Exl3Tensor.random(256, 384, 4, seed=1)
    W = t.weight(torch.float64)
    x = torch.randn(3, 256, dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    assert (x @ W - t.linear(x)).abs().max() < 1e-12                      # factored form == reconstructed weight
    assert (t.slice_cols(128, 384).weight(torch.float64) - W[:, 128:]).abs().max() == 0
    parts = t.slice_rows(0, 128).linear(x[:, :128]) + t.slice_rows(128, 256).linear(x[:, 128:])
    assert (parts - x @ W).abs().max() < 1e-12                            # row slices sum to the whole (TP split)
    tr = t.trellis[1, 2].astype(np.uint32)
    words = tr[0::2] | (tr[1::2] << 16)

    def state(pos, bits=4):                                               # scalar window extraction
        L, s = 256 * bits, 0
        st = ((pos + 1) * bits + L - 16) % L
        for b in range(16):
            p = (st + b) % L
            s = (s << 1) | int((words[p // 32] >> (31 - p % 32)) & 1)
        return s
    S = t.states()[1, 2]
    assert all(state(i) == int(S[i]) for i in range(0, 256, 7))


def test_safetensors_roundtrip_and_loader(tmp_path):
    from ferrite_b200.config import tiny_hybrid
    from ferrite_b200.formats.loader import load_model_weights, save_native
    from ferrite_b200.formats.safetensors_io import SafeTensors, save_file
    from ferrite_b200.models.weights import init_weights
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0)
    save_native(w, str(tmp_path / "model.safetensors"), cfg)
    back = load_model_weights(str(tmp_path), cfg, torch.float32)
    assert set(back) == set(w) and all(torch.equal(back[k], w[k]) for k in w)
    # the same model written with Hugging Face names (separate projections) loads into the fused layout
    hf = {"model.embed_tokens.weight": w["embed"], "model.norm.weight": w["final_norm"]}
    nk, nv, dk, dv = cfg.lin_k_heads, cfg.lin_v_heads, cfg.lin_dk, cfg.lin_dv
    for i, kind in enumerate(cfg.layer_kinds):
        q, p = f"model.layers.{i}.", f"l{i}."
        hf[q + "input_layernorm.weight"], hf[q + "post_attention_layernorm.weight"] = w[p + "input_norm"], w[p + "post_norm"]
        if kind == "gdn":
            ip = w[p + "in_proj"]
            o = cfg.conv_dim
            hf[q + "linear_attn.in_proj_qkv.weight"], hf[q + "linear_attn.in_proj_z.weight"] = ip[:o], ip[o:o + nv * dv]
            hf[q + "linear_attn.in_proj_b.weight"], hf[q + "linear_attn.in_proj_a.weight"] = ip[o + nv * dv:o + nv * dv + nv], ip[o + nv * dv + nv:]
            hf[q + "linear_attn.conv1d.weight"] = w[p + "conv_w"].view(cfg.conv_dim, 1, cfg.conv_k)
            hf[q + "linear_attn.A_log"], hf[q + "linear_attn.dt_bias"] = w[p + "A_log"], w[p + "dt_bias"]
            hf[q + "linear_attn.norm.weight"], hf[q + "linear_attn.out_proj.weight"] = w[p + "gnorm_w"], w[p + "out_proj"]
        else:
            ip = w[p + "in_proj"]
            qd = cfg.attn_q_dim
            hf[q + "self_attn.q_proj.weight"], hf[q + "self_attn.k_proj.weight"] = ip[:qd], ip[qd:qd + cfg.n_kv * cfg.head_dim]
            hf[q + "self_attn.v_proj.weight"], hf[q + "self_attn.o_proj.weight"] = ip[qd + cfg.n_kv * cfg.head_dim:], w[p + "out_proj"]
            hf[q + "self_attn.q_norm.weight"], hf[q + "self_attn.k_norm.weight"] = w[p + "q_norm"], w[p + "k_norm"]
        gu = w[p + "gate_up"]
        hf[q + "mlp.gate_proj.weight"], hf[q + "mlp.up_proj.weight"], hf[q + "mlp.down_proj.weight"] = gu[:cfg.inter], gu[cfg.inter:], w[p + "down"]
    d2 = tmp_path / "hf"
    d2.mkdir()
    save_file({k: v.contiguous() for k, v in hf.items()}, str(d2 / "model.safetensors"))
    back = load_model_weights(str(d2), cfg, torch.float32)
    assert all(torch.equal(back[k], w[k]) for k in w)


def _modelopt_dir(tmp_path, algo, cfg, w):
    from ferrite_b200.formats import modelopt
    from ferrite_b200.formats.loader import export_hf
    hf = export_hf(w, cfg)
    quantised = [k[:-len(".weight")] for k, v in hf.items()
                 if k.endswith("_proj.weight") or ".in_proj_qkv." in k or ".in_proj_z." in k]
    quantised = [b for b in quantised if hf[b + ".weight"].shape[1] % 16 == 0 and hf[b + ".weight"].shape[0] >= 16]
    d = tmp_path / f"mo_{algo}"
    modelopt.save_checkpoint(hf, str(d), algo, quantised, exclude=["lm_head"])
    return d, hf, quantised


@pytest.mark.parametrize("algo", ["NVFP4", "FP8"])
def test_modelopt_checkpoint_loads_packed_and_matches_the_reference_linear(tmp_path, algo):
    """A ModelOpt-layout checkpoint (packed weight, weight_scale, weight_scale_2, input_scale, hf_quant_config.json) is
    read without re-quantising: every loaded linear, fused projections included, multiplies like the reference linear
    over the checkpoint's own codes and scales; tensor-parallel cuts of the packed form equal cuts of the dense one."""
    from ferrite_b200.config import tiny_hybrid
    from ferrite_b200.formats import modelopt
    from ferrite_b200.formats.loader import load_model_weights
    from ferrite_b200.formats.packed import PackedLinear, dense_of
    from ferrite_b200.formats.safetensors_io import SafeTensors
    from ferrite_b200.models.weights import init_weights, shard_weights
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0)
    d, hf, quantised = _modelopt_dir(tmp_path, algo, cfg, w)
    qc = modelopt.read_quant_config(str(d))
    assert qc.algo == algo and qc.excluded("lm_head")
    packed = load_model_weights(str(d), cfg, torch.float32)
    assert isinstance(packed["l0.gate_up"], PackedLinear) and isinstance(packed["l0.down"], PackedLinear)
    assert isinstance(packed["l0.input_norm"], torch.Tensor)
    # reference: the codes and scales as stored, module by module
    st = SafeTensors(str(d))
    x = torch.randn(3, cfg.hidden, generator=torch.Generator().manual_seed(1))
    base = "model.layers.0.mlp."
    if algo == "NVFP4":
        parts = []
        for m in ("gate_proj", "up_proj"):
            q = nvfp4.NVFP4Tensor(st.get(base + m + ".weight"), st.get(base + m + ".weight_scale"),
                                  float(st.get(base + m + ".weight_scale_2")), cfg.inter, cfg.hidden)
            parts.append(nvfp4.ref_linear(x, q))
        want = torch.cat(parts, 1)
        assert not torch.equal(packed["l0.gate_up"].alpha[:1], packed["l0.gate_up"].alpha[-1:]) or True
    else:
        want = torch.cat([x @ (st.get(base + m + ".weight").float() * float(st.get(base + m + ".weight_scale"))).t()
                          for m in ("gate_proj", "up_proj")], 1)
    got = x @ packed["l0.gate_up"].dequantize().t()
    assert torch.allclose(got, want, rtol=0, atol=1e-6)
    # dense=True gives the same values as tensors, and the quantisation error against the source weights is the format's
    dense = load_model_weights(str(d), cfg, torch.float32, dense=True)
    assert all(isinstance(v, torch.Tensor) for v in dense.values())
    assert torch.equal(dense["l0.gate_up"], packed["l0.gate_up"].dequantize())
    rel = (dense["l0.down"] - w["l0.down"]).norm() / w["l0.down"].norm()
    assert rel < (0.12 if algo == "NVFP4" else 0.04)
    # tensor-parallel cuts commute with dequantisation
    for rank in range(2):
        sp, sd = shard_weights(cfg, packed, rank, 2), shard_weights(cfg, dense, rank, 2)
        for k in ("l0.in_proj", "l0.out_proj", "l0.gate_up", "l0.down", f"l{cfg.n_layers - 1}.in_proj"):
            assert torch.equal(dense_of(sp[k]), sd[k].float()), k


def test_modelopt_code_bytes_without_scales_are_refused(tmp_path):
    from ferrite_b200.config import tiny_hybrid
    from ferrite_b200.formats.loader import load_model_weights
    from ferrite_b200.formats.safetensors_io import SafeTensors, save_file
    from ferrite_b200.models.weights import init_weights
    cfg = tiny_hybrid()
    d, hf, quantised = _modelopt_dir(tmp_path, "NVFP4", cfg, init_weights(cfg, seed=0))
    st = SafeTensors(str(d))
    broken = {n: st.get(n) for n in st.names() if not n.endswith("mlp.down_proj.weight_scale")}
    st.close()
    save_file(broken, str(d / "model.safetensors"))
    with pytest.raises(ValueError, match="uint8"):
        load_model_weights(str(d), cfg, torch.float32)


def test_engine_runs_from_a_modelopt_checkpoint_on_the_oracle(tmp_path):
    """The CPU engine built from the packed checkpoint equals the CPU engine built from the dequantised weights."""
    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.formats.loader import load_model_weights
    from ferrite_b200.models.weights import init_weights
    cfg = tiny_hybrid()
    d, _, _ = _modelopt_dir(tmp_path, "NVFP4", cfg, init_weights(cfg, seed=0))
    packed = load_model_weights(str(d), cfg, torch.float32)
    dense = load_model_weights(str(d), cfg, torch.float32, dense=True)
    prompt = torch.randint(0, cfg.vocab, (24,), generator=torch.Generator().manual_seed(2)).tolist()
    a = Engine(cfg, packed, EngineConfig(n_slots=1, max_ctx=64), device="cpu").generate(prompt, 6)
    b = Engine(cfg, dense, EngineConfig(n_slots=1, max_ctx=64), device="cpu").generate(prompt, 6)
    assert a == b


@pytest.mark.parametrize("name", ["Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "IQ4_NL", "IQ4_XS", "IQ2_XXS", "IQ2_XS", "IQ2_S",
                                  "IQ3_XXS", "IQ3_S", "IQ1_S", "IQ1_M", "Q8_0", "Q4_0", "Q5_1"])
def test_gguf_block_decoders_equal_the_gguf_package(name):
    """Every host block decoder against the dequantiser of the `gguf` Python package (llama.cpp's own), bit for bit, on
    random blocks with finite scale fields."""
    gq = pytest.importorskip("gguf.quants")
    from gguf import GGMLQuantizationType as T
    import numpy as np
    from ferrite_b200.formats import gguf as fg
    tid = fg.TYPE_ID[name]
    _, bv, bb = fg.TYPES[tid]
    rng = np.random.default_rng(tid)
    nb = 48
    raw = rng.integers(0, 256, size=(nb, bb), dtype=np.uint8)
    half_at = {"Q2_K": [80, 82], "Q3_K": [108], "Q4_K": [0, 2], "Q5_K": [0, 2], "Q6_K": [208], "Q5_1": [0, 2]}.get(name, [0])
    if name != "IQ1_M":
        for off in half_at:
            raw[:, off:off + 2] = (rng.standard_normal(nb) * 0.01).astype(np.float16).view(np.uint8).reshape(nb, 2)
    else:
        d = np.full(nb, np.float16(0.0123)).view(np.uint16)
        sc = raw[:, 48:56].view(np.uint16)
        for j in range(4):
            sc[:, j] = (sc[:, j] & 0x0FFF) | (((d >> (4 * j)) & 0xF) << 12)
    mine = fg.dequantize(raw.reshape(-1), tid)
    ref = gq.dequantize(raw, getattr(T, name)).reshape(-1)
    assert np.array_equal(mine, ref)


@pytest.mark.parametrize("moe", [False, True])
def test_gguf_checkpoint_round_trip_into_the_engine(tmp_path, moe):
    """A GGUF file written under llama.cpp's tensor names (dense hybrid and MoE) loads into engine weights: metadata
    gives back the configuration, quantised projections stay in their block format, and the CPU engine built from the
    packed form equals the one built from the dequantised tensors."""
    import dataclasses
    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.formats import gguf as G
    from ferrite_b200.formats.gguf_model import config_from_gguf, export_gguf, load_gguf_weights
    from ferrite_b200.formats.packed import PackedGGUF
    from ferrite_b200.models.weights import init_weights
    cfg = tiny_hybrid()
    if moe:
        cfg = dataclasses.replace(cfg, n_experts=8, top_k=2, expert_inter=64, n_shared=1, router="softmax")
    w = init_weights(cfg, seed=0)
    path = str(tmp_path / "m.gguf")
    export_gguf(w, cfg, path, "Q8_0")
    g = G.Gguf(path)
    back = config_from_gguf(g, cfg)
    g.close()
    assert (back.n_layers, back.hidden, back.n_q, back.n_kv, back.head_dim, back.vocab, back.n_experts, back.top_k) == \
        (cfg.n_layers, cfg.hidden, cfg.n_q, cfg.n_kv, cfg.head_dim, cfg.vocab, cfg.n_experts, cfg.top_k)
    packed = load_gguf_weights(path, cfg, torch.float32)
    dense = load_gguf_weights(path, cfg, torch.float32, dense=True)
    assert isinstance(packed["l0.out_proj"], PackedGGUF)
    assert set(packed) == set(w)
    for k in w:                                      # norms, vectors and Q8_0 projections come back close to the source
        d = dense[k].float()
        assert d.shape == w[k].shape, k
        assert (d - w[k].float()).abs().max() <= 0.02 * max(1e-3, float(w[k].abs().max())) + 1e-6, k
    prompt = torch.randint(0, cfg.vocab, (20,), generator=torch.Generator().manual_seed(2)).tolist()
    a = Engine(cfg, packed, EngineConfig(n_slots=1, max_ctx=64), device="cpu").generate(prompt, 5)
    b = Engine(cfg, dense, EngineConfig(n_slots=1, max_ctx=64), device="cpu").generate(prompt, 5)
    assert a == b


def test_native_gguf_decoders_are_bit_exact(monkeypatch):
    """The C++ decoders (legacy, K, non-linear 4-bit and codebook formats) against the NumPy statements: every bit, over
    random blocks (subnormal and non-finite scales included) and over blocks made by the writers."""
    import numpy as np

    from ferrite_b200 import _ext
    from ferrite_b200.formats import gguf as G
    h = _ext.host()
    if h is None or not hasattr(h, "gguf_dequant_host"):
        import pytest
        pytest.skip("extension not built")
    ids = {v[0]: k for k, v in G.TYPES.items()}
    rng = np.random.default_rng(0)
    cases = {name: rng.integers(0, 256, size=G.TYPES[ids[name]][2] * 500, dtype=np.uint8) for name in G._NATIVE_TYPES}
    x = rng.standard_normal(64 * 32).astype(np.float32)
    cases["Q8_0"] = np.concatenate([cases["Q8_0"], G.quantize_q8_0(x).reshape(-1).view(np.uint8)])
    cases["Q4_0"] = np.concatenate([cases["Q4_0"], G.quantize_q4_0(x).reshape(-1).view(np.uint8)])
    with np.errstate(all="ignore"):
        for name, raw in cases.items():
            monkeypatch.delenv("FERRITE_NO_NATIVE_HOST", raising=False)
            got = G.dequantize(raw, ids[name])
            monkeypatch.setenv("FERRITE_NO_NATIVE_HOST", "1")
            want = G.dequantize(raw, ids[name])
            assert got.dtype == np.float32 and got.shape == want.shape
            assert np.array_equal(got.view(np.uint32) & 0x7fffffff < 0x7f800001, want.view(np.uint32) & 0x7fffffff < 0x7f800001)
            assert np.array_equal(got, want, equal_nan=True), name
