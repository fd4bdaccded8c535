"""The engine on the CUDA kernels against the fp32 oracle (bf16 tolerance), eager and through CUDA graphs."""
import pytest
import torch

from ferrite_b200.config import EngineConfig, hybrid_27b, scaled, tiny_hybrid
from ferrite_b200.engine.engine import Engine
from ferrite_b200.engine.executor import Segment
from ferrite_b200.models.ref import RefModel
from ferrite_b200.models.weights import init_weights

pytestmark = pytest.mark.gpu


def _prompt(cfg, n, seed=1):
    return torch.randint(0, cfg.vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def test_tiny_logits_vs_oracle(ext):
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0)
    w = {k: v.to(torch.bfloat16).float() if v.dtype == torch.float32 and not k.endswith(("A_log", "dt_bias")) else v
         for k, v in w.items()}
    ref = RefModel(cfg, w)
    prompt = _prompt(cfg, 40)
    want = ref.forward(prompt + [7, 8, 9], ref.new_state())
    eng = Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=256), device="cuda")
    got, _, _ = eng.forward([Segment(0, 0, prompt, "all")])
    err = (got.cpu() - want[:40]).abs().max().item()
    assert err < 0.05 * want.abs().max().item() + 0.02, err
    # decode rows through the graph path (twice the same key: capture, then replay)
    for i, t in enumerate([7, 8, 9]):
        lg, picks, _ = eng.forward([Segment(0, 40 + i, [t], "last")])
        err = (lg[0].cpu() - want[40 + i]).abs().max().item()
        assert err < 0.05 * want.abs().max().item() + 0.02, (i, err)
        assert int(picks[0][0]) == int(lg[0].argmax())
    eng.check()


def test_27b_width_layers_decode_matches_prefill(ext):
    """Real 27B widths (4 layers): logits of a decode row equal the same row computed inside a prompt chunk."""
    cfg = scaled(hybrid_27b(), 4)
    eng = Engine(cfg, None, EngineConfig(n_slots=2, max_ctx=512), device="cuda", seed=3)
    prompt = _prompt(cfg, 130)
    a, _, _ = eng.forward([Segment(0, 0, prompt, "last")])
    eng.forward([Segment(1, 0, prompt[:-1], "none")])
    b, _, _ = eng.forward([Segment(1, 129, prompt[-1:], "last")])
    err = (a - b).abs().max().item()
    assert err < 0.03 * a.abs().max().item() + 0.02, err
    eng.check()


def test_nvfp4_engine_matches_dequantised_oracle(ext):
    """NVFP4 weights: the decode path (fp4 GEMV) and the oracle run on the same dequantised weights."""
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0)
    eng = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=256, weight_dtype="nvfp4-a16"), device="cuda")
    wq = {k: (v.dense.float().cpu() if hasattr(v, "dense") else v.float().cpu()) for k, v in eng.ex.w.items()}
    ref = RefModel(cfg, wq)
    prompt = _prompt(cfg, 20)
    want = ref.forward(prompt + [3, 4], ref.new_state())
    eng.forward([Segment(0, 0, prompt, "none")])
    for i, t in enumerate([3, 4]):
        lg, _, _ = eng.forward([Segment(0, 20 + i, [t], "last")])
        err = (lg[0].cpu() - want[20 + i]).abs().max().item()
        assert err < 0.05 * want.abs().max().item() + 0.02, (i, err)
    eng.check()


def test_nvfp4_w4a4_engine_tracks_the_16bit_activation_path(ext):
    """Weights and activations in NVFP4 (block-scaled tcgen05 GEMM): next-token distributions stay close to the
    NVFP4-weight / 16-bit-activation engine on the same weights (activation quantisation noise only)."""
    cfg = scaled(hybrid_27b(), 2)
    a = Engine(cfg, None, EngineConfig(n_slots=1, max_ctx=256, weight_dtype="nvfp4-a16"), device="cuda", seed=5)
    b = Engine(cfg, None, EngineConfig(n_slots=1, max_ctx=256, weight_dtype="nvfp4-w4a4"), device="cuda", seed=5)
    prompt = _prompt(cfg, 40)
    la, _, _ = a.forward([Segment(0, 0, prompt, "last")])
    lb, _, _ = b.forward([Segment(0, 0, prompt, "last")])
    for i in range(3):
        la, _, _ = a.forward([Segment(0, 40 + i, [11 + i], "last")])
        lb, _, _ = b.forward([Segment(0, 40 + i, [11 + i], "last")])
        pa, pb = torch.log_softmax(la[0].float(), -1), torch.log_softmax(lb[0].float(), -1)
        kl = (pa.exp() * (pa - pb)).sum().item()
        assert kl < 0.5, kl           # random-init logits are nearly flat: quantisation noise shows up amplified
    a.check(); b.check()


def test_fp8_kv_cache_gpu(ext):
    """e4m3 KV cache on the GPU (quantising attn-prep, decode kernel reading codes + scales, prompt attention over
    the decoded scratch) against the CPU oracle with the same cache quantisation."""
    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment
    from ferrite_b200.models.weights import init_weights
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0)
    p = torch.randint(0, cfg.vocab, (120,), generator=torch.Generator().manual_seed(1)).tolist()
    ref = Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=256, kv_dtype="fp8"), device="cpu")
    want, _, _ = ref.forward([Segment(1, 0, p, "all")])
    eng = Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=256, kv_dtype="fp8"), device="cuda")
    assert eng.ex.k_cache[3].dtype == torch.uint8 if 3 in eng.ex.k_cache else True
    a, _, _ = eng.forward([Segment(1, 0, p[:64], "all")], greedy=False)          # prompt chunk 1 (flash over scratch)
    b, _, _ = eng.forward([Segment(1, 64, p[64:110], "all")], greedy=False)      # chunk 2 sees chunk 1 through the cache
    tail = [eng.forward([Segment(1, 110 + i, [p[110 + i]], "last")], greedy=False)[0].clone() for i in range(10)]
    got = torch.cat([a, b] + tail).float().cpu()
    kl = torch.nn.functional.kl_div(torch.log_softmax(got, -1), torch.log_softmax(want, -1), log_target=True,
                                    reduction="batchmean").item()
    assert kl < 2e-2, kl


def test_mixed_decode_and_prompt_rows_in_one_step(ext):
    """27B layer widths (2 layers): a decode row of one slot and a 100-row prompt chunk of another in ONE forward give
    the logits of the two separate forwards (chunked GDN scan with a one-row segment, flash attention with a one-row
    tile, one GEMM for all rows)."""
    from ferrite_b200.config import EngineConfig, hybrid_27b, scaled
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment
    cfg = scaled(hybrid_27b(), 4)
    g = torch.Generator().manual_seed(3)
    pa = torch.randint(0, cfg.vocab, (70,), generator=g).tolist()
    pb = torch.randint(0, cfg.vocab, (100,), generator=g).tolist()

    def fresh():
        e = Engine(cfg, None, EngineConfig(n_slots=2, max_ctx=512), device="cuda", seed=0)
        e.forward([Segment(0, 0, pa[:69], "none")])
        return e
    e1 = fresh()
    da = e1.forward([Segment(0, 69, [pa[69]], "last")], greedy=False)[0].clone()
    db = e1.forward([Segment(1, 0, pb, "last")], greedy=False)[0].clone()
    e2 = fresh()
    both = e2.forward([Segment(0, 69, [pa[69]], "last"), Segment(1, 0, pb, "last")], greedy=False)[0]
    assert both.shape[0] == 2
    scale = max(1.0, da.abs().max().item())
    assert (both[0] - da[0]).abs().max().item() < 3e-2 * scale
    assert (both[1] - db[0]).abs().max().item() < 3e-2 * scale
    # and the states they leave behind continue identically
    n1 = e1.forward([Segment(0, 70, [5], "last")], greedy=False)[0].clone()
    n2 = e2.forward([Segment(0, 70, [5], "last")], greedy=False)[0].clone()
    assert (n1 - n2).abs().max().item() < 3e-2 * scale


def test_verify_then_commit_at_27b_widths(ext):
    """Speculative verification at the 27B layer widths: 1 + 8 rows scored without committing, the first 5 accepted
    (replay of the GDN state from the saved projections, KV rows kept), then the next decode row must match the plain
    path that fed the same 5 tokens normally."""
    cfg = scaled(hybrid_27b(), 4)
    p = _prompt(cfg, 90)
    draft = _prompt(cfg, 9, seed=7)
    eng = Engine(cfg, None, EngineConfig(n_slots=1, max_ctx=512), device="cuda", seed=3)
    eng.forward([Segment(0, 0, p, "none")])
    before = eng.ex.state_save(0)
    eng.forward([Segment(0, 90, draft, "all")], commit=False)
    after = eng.ex.state_save(0)
    assert torch.equal(before["rec"], after["rec"]) and torch.equal(before["conv"], after["conv"])
    eng.commit_verified([5])
    assert eng.slot_len[0] == 95
    a = eng.forward([Segment(0, 95, [11], "last")], greedy=False)[0].clone()
    ref = Engine(cfg, None, EngineConfig(n_slots=1, max_ctx=512), device="cuda", seed=3)
    ref.forward([Segment(0, 0, p + draft[:5], "none")])
    b = ref.forward([Segment(0, 95, [11], "last")], greedy=False)[0].clone()
    err = (a - b).abs().max().item()
    assert err < 0.03 * b.abs().max().item() + 0.02, err
    eng.check()


def test_mtp_chain_drafter_on_the_gpu(ext):
    """The MTP head (one attention layer over [embedding | target hidden] rows) drafting for the scheduler at the 27B
    layer widths: drafts are produced and verified, the first token equals the plain engine's (later ones may differ at
    near-ties of random-weight logits between the one-row and the many-row kernels; exact equality is asserted by the
    CPU test of the same path)."""
    from ferrite_b200.engine.scheduler import Sampling, SchedOptions, Scheduler, generate
    from ferrite_b200.models.mtp import MtpDrafter
    cfg = scaled(hybrid_27b(), 4)
    cfg.tap_layers = [cfg.n_layers - 1]
    prompt = _prompt(cfg, 70)
    plain = Engine(cfg, None, EngineConfig(n_slots=1, max_ctx=512), device="cuda", seed=3)
    want = generate(Scheduler(plain, SchedOptions(spec=0)), [prompt], Sampling(max_tokens=12))[0]
    eng = Engine(cfg, None, EngineConfig(n_slots=1, max_ctx=512), device="cuda", seed=3)
    dr = MtpDrafter(eng, n_slots=1, max_ctx=512, depth=3)
    sched = Scheduler(eng, SchedOptions(spec=3, copy_rows=False), drafter=dr)
    got = generate(sched, [prompt], Sampling(max_tokens=12))[0]
    assert got[0] == want[0] and len(got) == len(want)
    assert sched.stats["drafted"] > 0
    eng.check(); dr.eng.check()


def test_verify_tree_on_the_gpu(ext):
    """A verify tree (ancestor-masked attention, GDN conv / recurrence along parent links) scores every path like the
    chain verify of that path, and `commit_tree` (GDN replay of the kept path, KV rows moved into place) leaves the
    slot as if the path had been fed row by row: tiny model, then the 27B layer widths, then an e4m3 KV cache."""
    from ferrite_b200.utils.selftest import tree_test
    tree_test("cuda", 3e-2)
    tree_test("cuda", 3e-2, cfg=scaled(hybrid_27b(), 4), n_prompt=70)
    tree_test("cuda", 6e-2, kv_dtype="fp8")


def test_fp8_block_engine_matches_dequantised_oracle(ext):
    """Block-scaled e4m3 weights (128 x 128 blocks): the prompt path multiplies the codes on the f8f6f4 tensor path with
    activations quantised per 1 x 128 block, decode rows stream the dequantised copy; both against the fp32 oracle on
    the dequantised weights (the prompt path differs by the activation quantisation only)."""
    cfg = scaled(hybrid_27b(), 2)
    eng = Engine(cfg, None, EngineConfig(n_slots=1, max_ctx=256, weight_dtype="fp8-block"), device="cuda", seed=5)
    assert eng.ex.w["l0.in_proj"].kind == "fp8b"
    dense = Engine(cfg, {k: (v.dense if hasattr(v, "dense") else v) for k, v in eng.ex.w.items()},
                   EngineConfig(n_slots=1, max_ctx=256), device="cuda", seed=5)
    prompt = _prompt(cfg, 100)
    a = eng.forward([Segment(0, 0, prompt, "last")], greedy=False)[0].clone()
    b = dense.forward([Segment(0, 0, prompt, "last")], greedy=False)[0].clone()
    pa, pb = torch.log_softmax(a[0].float(), -1), torch.log_softmax(b[0].float(), -1)
    assert (pb.exp() * (pb - pa)).sum().item() < 0.05
    a = eng.forward([Segment(0, 100, [7], "last")], greedy=False)[0].clone()
    b = dense.forward([Segment(0, 100, [7], "last")], greedy=False)[0].clone()
    pa, pb = torch.log_softmax(a[0].float(), -1), torch.log_softmax(b[0].float(), -1)
    assert (pb.exp() * (pb - pa)).sum().item() < 0.05
    eng.check()


def test_int4_kv_cache_gpu(ext):
    """4-bit KV cache on the GPU (quantising attn-prep, decode kernel reading nibbles + group scales, prompt attention
    over the decoded scratch, a verify tree on top) against the CPU oracle with the same cache quantisation."""
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0)
    p = torch.randint(0, cfg.vocab, (120,), generator=torch.Generator().manual_seed(1)).tolist()
    ref = Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=256, kv_dtype="int4"), device="cpu")
    want, _, _ = ref.forward([Segment(1, 0, p, "all")])
    eng = Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=256, kv_dtype="int4"), device="cuda")
    kc = next(iter(eng.ex.k_cache.values()))
    assert kc.dtype == torch.uint8 and kc.shape[-1] == cfg.head_dim // 2
    a, _, _ = eng.forward([Segment(1, 0, p[:64], "all")], greedy=False)
    b, _, _ = eng.forward([Segment(1, 64, p[64:110], "all")], greedy=False)
    tail = [eng.forward([Segment(1, 110 + i, [p[110 + i]], "last")], greedy=False)[0].clone() for i in range(10)]
    got = torch.cat([a.clone(), b.clone()] + tail).float().cpu()
    kl = torch.nn.functional.kl_div(torch.log_softmax(got, -1), torch.log_softmax(want, -1), log_target=True,
                                    reduction="batchmean").item()
    assert kl < 2e-2, kl
    from ferrite_b200.utils.selftest import tree_test
    tree_test("cuda", 8e-2, kv_dtype="int4")
    eng.check()


@pytest.mark.parametrize("kv", ["int6", "int4h", "int6h", "fp8h"])
def test_6bit_and_rotated_kv_caches_gpu(ext, kv):
    """6-bit codes (4 per 3 bytes) and Hadamard-rotated keys on the GPU: quantising attn-prep, the decode kernel reading
    the packed codes, prompt attention over the decoded scratch, a verify tree, against the CPU oracle of the same form."""
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0)
    p = torch.randint(0, cfg.vocab, (120,), generator=torch.Generator().manual_seed(1)).tolist()
    ref = Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=256, kv_dtype=kv), device="cpu")
    want, _, _ = ref.forward([Segment(1, 0, p, "all")])
    eng = Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=256, kv_dtype=kv), device="cuda")
    kc = next(iter(eng.ex.k_cache.values()))
    bits = {"int6": 6, "int6h": 6, "int4h": 4, "fp8h": 8}[kv]
    assert kc.dtype == torch.uint8 and kc.shape[-1] == cfg.head_dim * bits // 8
    a, _, _ = eng.forward([Segment(1, 0, p[:64], "all")], greedy=False)
    b, _, _ = eng.forward([Segment(1, 64, p[64:110], "all")], greedy=False)
    tail = [eng.forward([Segment(1, 110 + i, [p[110 + i]], "last")], greedy=False)[0].clone() for i in range(10)]
    got = torch.cat([a.clone(), b.clone()] + tail).float().cpu()
    kl = torch.nn.functional.kl_div(torch.log_softmax(got, -1), torch.log_softmax(want, -1), log_target=True,
                                    reduction="batchmean").item()
    assert kl < 2e-2, kl
    from ferrite_b200.utils.selftest import tree_test
    tree_test("cuda", 8e-2, kv_dtype=kv)
    eng.check()


@pytest.mark.parametrize("hd", [64, 128, 256])
def test_6bit_kv_kernels_at_every_head_width(ext, hd):
    """attn-prep writing 6-bit rows and the decode kernel reading them, per head width (2, 4 and 8 codes per lane pack
    differently), with rotated keys, against the fp32 statement of the same cache."""
    from ferrite_b200.ops.cuda_ops import CudaOps
    from ferrite_b200.ops.torch_ops import TorchOps
    ops, tops = CudaOps("cuda"), TorchOps("cuda", torch.float32)
    g = torch.Generator(device="cuda").manual_seed(hd)
    nq, nkv, kvb, nblk, T, rot = 4, 2, 64, 6, 5, 32
    proj = torch.randn(T, (nq + 2 * nkv) * hd, generator=g, device="cuda").bfloat16()
    qn = (torch.randn(hd, generator=g, device="cuda") * 0.1).bfloat16()
    kn = (torch.randn(hd, generator=g, device="cuda") * 0.1).bfloat16()
    inv = (1e4 ** (-torch.arange(rot // 2, dtype=torch.float64) / (rot // 2))).float().cuda()
    slot = torch.tensor([0, 0, 1, 1, 1], dtype=torch.int32, device="cuda")
    pos = torch.tensor([5, 6, 70, 71, 72], dtype=torch.int32, device="cuda")
    bt = torch.arange(2 * nblk, dtype=torch.int32, device="cuda").view(2, nblk)
    # fill the caches with earlier rows first so the decode reads more than the five new rows
    kc = torch.zeros(2 * nblk, kvb, nkv, hd * 3 // 4, dtype=torch.uint8, device="cuda")
    vc = torch.zeros_like(kc)
    sc = torch.ones(2 * nblk, kvb, nkv, 2 * (hd // 32), dtype=torch.float32, device="cuda")
    kf = torch.zeros(2 * nblk, kvb, nkv, hd, dtype=torch.float32, device="cuda")
    vf = torch.zeros_like(kf)
    for s0, n in ((0, 5), (1, 70)):
        pj = torch.randn(n, (nq + 2 * nkv) * hd, generator=g, device="cuda").bfloat16()
        sl = torch.full((n,), s0, dtype=torch.int32, device="cuda")
        ps = torch.arange(n, dtype=torch.int32, device="cuda")
        ops.attn_prep(pj, qn, kn, inv, sl, ps, bt, kc, vc, kvb, nq, nkv, hd, rot, False, 1e-6, kv_scale=sc, hrot=True)
        tops.attn_prep(pj, qn, kn, inv, sl, ps, bt, kf, vf, kvb, nq, nkv, hd, rot, False, 1e-6, kv_scale=sc, hrot=True, kv_bits=6)
    qa = ops.attn_prep(proj, qn, kn, inv, slot, pos, bt, kc, vc, kvb, nq, nkv, hd, rot, False, 1e-6, kv_scale=sc, hrot=True)
    qb = tops.attn_prep(proj, qn, kn, inv, slot, pos, bt, kf, vf, kvb, nq, nkv, hd, rot, False, 1e-6, kv_scale=sc, hrot=True,
                        kv_bits=6)
    assert (qa.float() - qb.float()).abs().max().item() < 5e-2
    kvlen = (pos + 1).contiguous()
    for nsplit in (1, 3):
        oa = ops.attention(qa, proj, kc, vc, slot, kvlen, bt, kvb, nq, nkv, hd, False, nsplit=nsplit, kv_scale=sc)
        ob = tops.attention(qb, proj, kf, vf, slot, kvlen, bt, kvb, nq, nkv, hd, False)
        assert (oa.float() - ob.float()).abs().max().item() < 6e-2, (hd, nsplit)
    assert ops.status() == 0


def test_commit_after_replayed_verify_graphs(ext):
    """Verify steps of two slots with different context lengths are different CUDA graphs; replaying the first one again
    and committing must replay THAT graph's saved projections (and its captured commit graph), not those of the graph
    captured last. Against an engine without graphs."""
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0)
    pa, pb = _prompt(cfg, 40, 1), _prompt(cfg, 300, 2)
    da, db = _prompt(cfg, 6, 3), _prompt(cfg, 6, 4)

    def run(use_graphs):
        e = Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=512, use_graphs=use_graphs), device="cuda")
        e.forward([Segment(0, 0, pa, "none")])
        e.forward([Segment(1, 0, pb, "none")])
        outs = []
        for rnd_ in range(2):                                  # second round replays both verify graphs
            for slot, d in ((0, da), (1, db)):
                p0 = e.slot_len[slot]
                e.forward([Segment(slot, p0, d, "all")], commit=False)
                e.commit_verified([4])
                outs.append(e.forward([Segment(slot, p0 + 4, [9], "last")], greedy=False)[0].clone())
        e.check()
        return torch.cat(outs).float()
    a, b = run(True), run(False)
    assert (a - b).abs().max().item() < 2e-2 * max(1.0, b.abs().max().item())


def test_scheduler_samples_on_the_device(ext):
    """Sampled requests without penalties draw their decode tokens with the device sampler: seeded requests repeat, a
    different seed changes the text, a near-zero temperature reproduces greedy decoding, and the host path (switched on
    through the option) stays available."""
    from ferrite_b200.engine.scheduler import Sampling, SchedOptions, Scheduler, generate
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0)
    eng = Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=256), device="cuda")
    sched = Scheduler(eng, SchedOptions(spec=0))
    p = _prompt(cfg, 30)
    calls = []
    orig = eng.ops.sample
    eng.ops.sample = lambda *a, **k: (calls.append(1), orig(*a, **k))[1]
    s1 = Sampling(temperature=0.9, top_k=40, top_p=0.95, seed=11, max_tokens=12)
    a = generate(sched, [p], s1)[0]
    b = generate(sched, [p], s1)[0]
    c = generate(sched, [p], Sampling(temperature=0.9, top_k=40, top_p=0.95, seed=12, max_tokens=12))[0]
    assert a == b and len(a) == 12 and a != c and len(calls) > 0
    greedy = generate(sched, [p], Sampling(max_tokens=8))[0]
    cold = generate(sched, [p], Sampling(temperature=1e-3, top_k=1, seed=3, max_tokens=8))[0]
    assert cold == greedy
    n = len(calls)
    host = Scheduler(eng, SchedOptions(spec=0, device_sampling=False))
    h = generate(host, [p], s1)[0]
    assert len(h) == 12 and len(calls) == n


@pytest.mark.parametrize("streams", [1, 3])
def test_persistent_decode_layer_matches_the_separate_kernels(ext, streams):
    """One persistent kernel per layer (grid barriers between its phases) against the separate-launch path: same
    weights, same prompts, decode rows compared step by step (logits to bf16 rounding of the norms' sums, greedy
    picks equal), eager first and then through the CUDA graph."""
    cfg = scaled(hybrid_27b(), 8)                              # 6 Gated DeltaNet layers, 2 attention layers
    engs = [Engine(cfg, None, EngineConfig(n_slots=streams, max_ctx=256, fused_layers=f), device="cuda", seed=3)
            for f in (False, True)]
    prompts = [_prompt(cfg, 30 + 5 * s, seed=10 + s) for s in range(streams)]
    for e in engs:
        for s, p in enumerate(prompts):
            e.prefill(s, p)
    feed = [[int(t) for t in _prompt(cfg, 12, seed=50 + s)] for s in range(streams)]
    for i in range(12):
        outs = []
        for e in engs:
            segs = [Segment(s, len(prompts[s]) + i, [feed[s][i]], "last") for s in range(streams)]
            lg, picks, _ = e.forward(segs, commit=True, greedy=True)
            outs.append((lg.float().cpu(), picks[0].cpu()))
        err = (outs[0][0] - outs[1][0]).abs().max().item()
        # (with several rows the separate path multiplies through mma.sync fragments: another summation order)
        assert err < 0.05 * outs[0][0].abs().max().item() + 1e-3, (i, err)
        if streams == 1:
            assert torch.equal(outs[0][1], outs[1][1]), i
    assert engs[1].ops.launches < engs[0].ops.launches
    for e in engs:
        e.check()


def test_128k_context_prefill_and_decode(ext):
    """131072 tokens of context on one GPU (27B widths, 4 layers): chunked prefill, then decode rows whose attention
    reads the whole cache through 64 key splits. The decode row at position 128K must agree with the same row computed
    as the last row of a prompt chunk, and stay finite."""
    cfg = scaled(hybrid_27b(), 4)
    ctx = 131072
    eng = Engine(cfg, None, EngineConfig(n_slots=2, max_ctx=ctx + 64, prefill_chunk=4096), device="cuda", seed=3)
    prompt = _prompt(cfg, ctx + 1, seed=9)
    for s in range(2):
        eng.prefill(s, prompt[:ctx])
    a, _, _ = eng.forward([Segment(0, ctx, prompt[ctx:], "last")])                       # one decode row
    b, _, _ = eng.forward([Segment(1, ctx, prompt[ctx:] + [5, 6, 7, 8, 9, 10, 11, 12, 13], "all")], commit=False)   # first row of a verify segment
    assert torch.isfinite(a).all() and torch.isfinite(b).all()
    err = (a[0] - b[0]).abs().max().item()
    assert err < 0.03 * a.abs().max().item() + 0.02, err
    for i in range(3):
        lg, picks, _ = eng.forward([Segment(0, ctx + 1 + i, [int(picks[0][0]) if i else 3], "last")])
        assert torch.isfinite(lg).all()
    assert eng.slot_len[0] == ctx + 4
    eng.check()
