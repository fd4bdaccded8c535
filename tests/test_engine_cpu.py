"""CPU plumbing tests (fp32): the engine on PyTorch ops against the token-by-token oracle."""
import torch

from ferrite_b200.config import EngineConfig, tiny_hybrid
from ferrite_b200.engine.engine import Engine, prompt_cuts
from ferrite_b200.engine.executor import Segment
from ferrite_b200.models.ref import RefModel
from ferrite_b200.models.weights import init_weights, shard_weights, weight_shapes


def _setup(seed=0):
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=seed)
    return cfg, w, RefModel(cfg, w)


def _prompt(cfg, n, seed=1):
    return torch.randint(0, cfg.vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def test_logits_match_oracle():
    cfg, w, ref = _setup()
    prompt = _prompt(cfg, 48)
    want = ref.forward(prompt, ref.new_state())
    eng = Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=256), device="cpu")
    got, _, rows = eng.forward([Segment(0, 0, prompt, "all")])
    assert rows == list(range(48))
    assert torch.allclose(got, want, atol=2e-5, rtol=1e-4)


def test_greedy_decode_config1():
    """BASELINE config 1: greedy decode of 32 tokens from a 64-token prompt, tiny hybrid, fp32, CPU."""
    cfg, w, ref = _setup()
    prompt = _prompt(cfg, 64)
    eng = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=128, prefill_chunk=32), device="cpu")
    assert eng.generate(prompt, 32) == ref.generate(prompt, 32)


def test_chunked_prefill_equals_whole():
    cfg, w, _ = _setup()
    prompt = _prompt(cfg, 100)
    a = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=256, prefill_chunk=32), device="cpu")
    b = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=256, prefill_chunk=2048), device="cpu")
    la = a.prefill(0, prompt)[0]
    lb = b.prefill(0, prompt)[0]
    assert torch.allclose(la, lb, atol=2e-5, rtol=1e-4)


def test_two_slots_are_independent():
    cfg, w, ref = _setup()
    p0, p1 = _prompt(cfg, 20, 3), _prompt(cfg, 33, 4)
    eng = Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=128), device="cpu")
    got, _, rows = eng.forward([Segment(0, 0, p0, "last"), Segment(1, 0, p1, "last")])
    w0 = ref.forward(p0, ref.new_state())[-1]
    w1 = ref.forward(p1, ref.new_state())[-1]
    assert torch.allclose(got[0], w0, atol=2e-5, rtol=1e-4)
    assert torch.allclose(got[1], w1, atol=2e-5, rtol=1e-4)


def test_verify_rows_do_not_commit_state():
    cfg, w, _ = _setup()
    prompt = _prompt(cfg, 24)
    eng = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=128), device="cpu")
    eng.prefill(0, prompt)
    before = eng.ex.state_save(0)
    eng.forward([Segment(0, 24, [5, 6, 7, 8], "all")], commit=False)
    after = eng.ex.state_save(0)
    assert torch.equal(before["rec"], after["rec"]) and torch.equal(before["conv"], after["conv"])
    assert eng.slot_len[0] == 24
    # committing the accepted prefix afterwards equals decoding it directly
    l1, _, _ = eng.forward([Segment(0, 24, [5, 6], "last")])
    eng2 = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=128), device="cpu")
    eng2.prefill(0, prompt + [5])
    l2, _, _ = eng2.forward([Segment(0, 25, [6], "last")])
    assert torch.allclose(l1, l2, atol=2e-5, rtol=1e-4)


def test_snapshot_restore_and_slot_copy():
    cfg, w, _ = _setup()
    prompt = _prompt(cfg, 40)
    eng = Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=128), device="cpu")
    eng.prefill(0, prompt[:30])
    snap = eng.ex.state_save(0)
    full = eng.prefill(0, prompt[30:])[0]
    eng.ex.state_restore(0, snap)
    eng.slot_len[0] = 30
    again = eng.prefill(0, prompt[30:])[0]
    assert torch.equal(full, again)                       # a cache resume is bitwise the full computation
    eng.ex.state_restore(0, snap)
    eng.ex.copy_slot(0, 1, 30)
    eng.slot_len[1] = 30
    fork = eng.prefill(1, prompt[30:])[0]
    assert torch.equal(full, fork)


def test_prompt_cuts():
    assert prompt_cuts(100, 32, 32) == [32, 32, 36]
    assert prompt_cuts(2048, 2048, 32) == [2048]
    assert prompt_cuts(2060, 2048, 32) == [2060]
    assert prompt_cuts(4100, 2048, 32) == [2048, 2048 + 4]
    assert sum(prompt_cuts(12345, 2048, 32)) == 12345


def test_shard_shapes():
    from ferrite_b200.config import hybrid_27b, scaled
    cfg = scaled(hybrid_27b(), 4)
    shapes = weight_shapes(cfg)
    w = {k: torch.empty(v, dtype=torch.bfloat16, device="meta") for k, v in shapes.items()}
    for world in (2, 4, 8):
        sc = cfg.shard(world)
        want = weight_shapes(sc)
        got = {k: tuple(v.shape) for k, v in shard_weights(cfg, w, 0, world).items()}
        for k, shp in want.items():
            if k == "lm_head":
                assert got[k][0] == (cfg.vocab + world - 1) // world
            elif k in ("embed",):
                assert got[k] == shp
            else:
                assert got[k] == shp, (k, got[k], shp, world)


def test_fp8_kv_cache_stays_close_to_bf16():
    """e4m3 KV cache (one scale per token and kv head): logits stay close to the full-precision cache and decode
    through the cache agrees with a longer prompt."""
    cfg, w, _ = _setup()
    p = _prompt(cfg, 60)
    base = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=128), device="cpu")
    want, _, _ = base.forward([Segment(0, 0, p, "all")])
    eng = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=128, kv_dtype="fp8"), device="cpu")
    got, _, _ = eng.forward([Segment(0, 0, p[:50], "all")])
    tail = [eng.forward([Segment(0, 50 + i, [p[50 + i]], "last")])[0].clone() for i in range(10)]
    got = torch.cat([got] + tail)
    kl = torch.nn.functional.kl_div(torch.log_softmax(got, -1), torch.log_softmax(want, -1), log_target=True,
                                    reduction="batchmean").item()
    assert kl < 1e-3, kl
    assert not torch.equal(got, want)            # the quantisation is really in the path


def test_op_profiler_counts_calls():
    from ferrite_b200.utils.profiler import OpProfiler
    cfg, w, _ = _setup()
    eng = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=64), device="cpu")
    prof = OpProfiler(eng)
    eng.forward([Segment(0, 0, _prompt(cfg, 8), "last")])
    rep = prof.report()
    prof.detach()
    n_layers = cfg.n_layers
    assert rep["linear"]["calls"] + 2 * rep["ffn"]["calls"] >= 4 * n_layers and rep["linear"]["ms"] > 0       # an ffn is two linears
    assert "attention" in rep or "attention_prefill" in rep
    assert eng.ex.profile is None


def test_int4_kv_cache_stays_close_to_the_16bit_cache():
    """4-bit KV cache (groups of 32, scale = amax / 7): next-token distributions stay close to the 16-bit cache, decode
    rows read what prompt rows wrote, and the page accounting shrinks."""
    import torch
    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment
    from ferrite_b200.models.weights import init_weights
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0)
    p = torch.randint(0, cfg.vocab, (70,), generator=torch.Generator().manual_seed(1)).tolist()
    ref = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=128), device="cpu")
    q4 = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=128, kv_dtype="int4"), device="cpu")
    assert q4.ex.kv_block_bytes() < ref.ex.kv_block_bytes() / 3
    a = ref.forward([Segment(0, 0, p, "all")])[0]
    b1 = q4.forward([Segment(0, 0, p[:40], "all")])[0]
    b2 = torch.cat([q4.forward([Segment(0, 40 + i, [p[40 + i]], "last")])[0] for i in range(30)])
    b = torch.cat([b1, b2])
    kl = torch.nn.functional.kl_div(torch.log_softmax(b, -1), torch.log_softmax(a, -1), log_target=True,
                                    reduction="batchmean").item()
    assert kl < 1e-3, kl


def test_host_statements_of_the_small_ops():
    """The fp32 statements the GPU tests compare the drafter and hyper-connection kernels against, checked on values
    worked out by hand."""
    import torch
    from ferrite_b200.ops.torch_ops import TorchOps
    t = TorchOps("cpu", torch.float32)
    g = torch.Generator().manual_seed(0)
    x, c, b = torch.randn(8, 64, generator=g), torch.randn(8, 16, generator=g), torch.randn(2, 64, generator=g)
    y = t.dynconv(x, c, b, 8, 4)
    j, r = 13, 5
    want = (b[0, j] + c[r, j // 8]) * x[r, j] + (b[1, j] + c[r, 8 + j // 8]) * x[r - 1, j]
    assert abs(float(y[r, j]) - float(want)) < 1e-5
    assert abs(float(y[4, j]) - float((b[0, j] + c[4, j // 8]) * x[4, j])) < 1e-5          # first row of a block: one tap
    vals = torch.tensor([[[5.0] + [0.0] * 15], [[5.0] + [1.0] * 15]])                      # two ranks, one row
    ids = torch.stack([torch.arange(100, 116)[None], torch.arange(16)[None]]).to(torch.int32)
    ov, oi = t.topk16_merge(vals, ids)
    assert oi[0, :2].tolist() == [0, 100] and ov[0, :3].tolist() == [5.0, 5.0, 1.0]         # tie goes to the lower id
    a_cb, b_cb, gate = torch.eye(4)[:, :4].repeat(1, 64), torch.eye(4).repeat(1, 64), torch.ones(2, 256)
    cand = torch.tensor([[0, 1, 2, 3] * 4, [3, 2, 1, 0] * 4], dtype=torch.int32)
    out = t.draft_select(torch.zeros(2, 16), cand, gate, a_cb, b_cb, 2)
    assert out.tolist() == [2, 2]                      # <A[pred] * gate, B[c]> peaks at c == pred
    res = torch.ones(3, 4, 8)
    yn, inv = t.hc_norm(res, torch.ones(4, 8), 0.0)
    assert torch.allclose(inv, torch.ones(12)) and torch.allclose(yn, torch.ones(12, 8))
    mixed = t.hc_mix(res, inv, torch.ones(4, 8), torch.zeros(3, 4, 8))
    assert torch.allclose(mixed, torch.full((3, 8), 0.5))
    r2 = t.hc_combine(res.clone(), torch.ones(3, 8), torch.zeros(3, 4))
    assert torch.allclose(r2, torch.full((3, 4, 8), 2.0))


def test_6bit_and_rotated_kv_caches_on_the_oracle():
    """6-bit cache: much closer to the 16-bit cache than the 4-bit one at 1.4x its bytes. Hadamard-rotated keys: q . k is
    unchanged in exact arithmetic, so the rotated caches stay as close as the plain ones."""
    import torch
    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment
    from ferrite_b200.models.weights import init_weights
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0)
    p = torch.randint(0, cfg.vocab, (70,), generator=torch.Generator().manual_seed(1)).tolist()

    def run(kv):
        e = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=128, kv_dtype=kv), device="cpu")
        a = e.forward([Segment(0, 0, p[:40], "all")])[0]
        b = torch.cat([e.forward([Segment(0, 40 + i, [p[40 + i]], "last")])[0] for i in range(30)])
        return e, torch.cat([a, b])

    def kl(x, ref):
        return torch.nn.functional.kl_div(torch.log_softmax(x, -1), torch.log_softmax(ref, -1), log_target=True,
                                          reduction="batchmean").item()
    e16, ref = run("bf16")
    e4, l4 = run("int4")
    e6, l6 = run("int6")
    _, l4h = run("int4h")
    _, l6h = run("int6h")
    assert e4.ex.kv_block_bytes() < e6.ex.kv_block_bytes() < e16.ex.kv_block_bytes() / 2
    assert kl(l6, ref) < kl(l4, ref) / 4 and kl(l6, ref) < 1e-4
    assert kl(l6h, ref) < 1e-4 and kl(l4h, ref) < 1e-3


def test_bounds_checked_debug_mode():
    """Attached, the checker leaves results alone, counts what it looked at, and stops an out-of-range index before the
    op runs, naming op, parameter, element and limit."""
    import pytest
    import torch
    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment
    from ferrite_b200.utils.boundscheck import BoundsChecker
    cfg = tiny_hybrid()
    eng = Engine(cfg, None, EngineConfig(n_slots=2, max_ctx=128), device="cpu")
    want = eng.forward([Segment(0, 0, [1, 2, 3, 4, 5], "last")])[0].clone()
    eng.reset_slot(0)
    chk = BoundsChecker(eng)
    got = eng.forward([Segment(0, 0, [1, 2, 3, 4, 5], "last")])[0]
    assert torch.equal(want, got) and chk.checked["embed"] == 1 and chk.checked["attn_prep"] >= 1
    with pytest.raises(IndexError, match=r"embed: ids\[1\] = 4096 is outside \[0, 4096\)"):
        eng.ex.ops.embed(eng.ex.w["embed"], torch.tensor([1, cfg.vocab], dtype=torch.int32))
    with pytest.raises(IndexError, match=r"gdn_conv: seg_slot\[0\] = 7 is outside \[0, 2\) \(slots\)"):
        eng.ex.ops.gdn_conv(None, None, None, torch.tensor([7], dtype=torch.int32), None, None, 0)
    bad_table = eng.ex.block_table.clone()
    bad_table[1, 0] = 10 ** 6
    with pytest.raises(IndexError, match="block_table"):
        eng.ex.ops.attention(None, None, None, None, torch.tensor([0], dtype=torch.int32),
                             torch.tensor([1], dtype=torch.int32), bad_table, 64, 1, 1, 64, False)
    chk.detach()
    assert type(eng.ex.ops).__name__ == "TorchOps" and eng.ex.profile is None
