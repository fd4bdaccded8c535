"""Tensor-parallel plumbing on CPU ranks (gloo): sharded weights + process-group reductions reproduce the
single-rank logits; a rank that never joins is detected by a short process-group timeout, not by a hang."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ferrite_b200.config import PRESETS, EngineConfig, tiny_hybrid
from ferrite_b200.engine.engine import Engine
from ferrite_b200.engine.executor import Segment
from ferrite_b200.models.weights import init_weights


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, prompt, q, preset="tiny"):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    from ferrite_b200.parallel.tp import TensorParallel
    tp = TensorParallel(dist.group.WORLD, "cpu", fused=False)
    cfg = PRESETS[preset]()
    w = init_weights(cfg, seed=0)
    eng = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=128), device="cpu", tp=tp)
    logits, picks, _ = eng.forward([Segment(0, 0, prompt, "all")])
    l2, p2, _ = eng.forward([Segment(0, len(prompt), [int(picks[0][-1])], "last")])
    q.put((rank, logits, picks[0], l2))
    dist.destroy_process_group()


@pytest.mark.parametrize("world,plen", [(2, 24), (2, 97)])
def test_tp_matches_single_rank(world, plen):
    """24 rows: replicated rows + all-reduce; 97 rows: the sequence-parallel prompt path (row-sharded residual stream,
    all-gather before column-parallel and reduce-scatter after row-parallel projections) with a ragged last shard."""
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0)
    prompt = torch.randint(0, cfg.vocab, (plen,), generator=torch.Generator().manual_seed(5)).tolist()
    eng = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=128), device="cpu")
    want, wp, _ = eng.forward([Segment(0, 0, prompt, "all")])
    want2, _, _ = eng.forward([Segment(0, len(prompt), [int(wp[0][-1])], "last")])
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, prompt, q)) for r in range(world)]
    for p in procs:
        p.start()
    outs = sorted([q.get(timeout=120) for _ in range(world)], key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
    for rank, logits, ids, l2 in outs:
        assert torch.allclose(logits, want, atol=3e-5, rtol=1e-4), rank
        assert ids.tolist() == wp[0].tolist()
        assert torch.allclose(l2, want2, atol=3e-5, rtol=1e-4)
    # every rank holds identical bits
    assert torch.equal(outs[0][1], outs[1][1])


@pytest.mark.parametrize("plen", [20, 70])
def test_moe_latent_attention_model_under_tp2(plen):
    """The tiny latent-attention + MoE model on two gloo ranks (heads and experts split over the ranks, expert partial
    sums reduced): prompt logits, picks and a decode step equal the single-rank run, and both ranks hold the same bits."""
    cfg = PRESETS["tiny-mla"]()
    w = init_weights(cfg, seed=0)
    prompt = torch.randint(0, cfg.vocab, (plen,), generator=torch.Generator().manual_seed(6)).tolist()
    eng = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=128), device="cpu")
    want, wp, _ = eng.forward([Segment(0, 0, prompt, "all")])
    want2, _, _ = eng.forward([Segment(0, len(prompt), [int(wp[0][-1])], "last")])
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, prompt, q, "tiny-mla")) for r in range(2)]
    for p in procs:
        p.start()
    outs = sorted([q.get(timeout=180) for _ in range(2)], key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
    for rank, logits, ids, l2 in outs:
        assert torch.allclose(logits, want, atol=5e-5, rtol=1e-4), (rank, (logits - want).abs().max())
        assert ids.tolist() == wp[0].tolist()
        assert torch.allclose(l2, want2, atol=5e-5, rtol=1e-4)
    assert torch.equal(outs[0][1], outs[1][1]) and torch.equal(outs[0][3], outs[1][3])


def _lonely(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    if rank == 1:
        q.put((rank, "left"))            # leaves between steps, nothing in flight
        return
    try:
        t = torch.ones(4)
        dist.all_reduce(t)
        q.put((rank, "no error"))
    except Exception as e:                # the survivor's collective ends with an error instead of hanging
        q.put((rank, "error:" + type(e).__name__))


def test_missing_rank_is_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_lonely, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=60) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.terminate()
    assert got[1] == "left"
    assert got[0].startswith("error")


def _selftest_worker(rank, world, port, corrupt, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    if corrupt:
        os.environ["FE_TEST_P2P_CORRUPT"] = corrupt
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    from ferrite_b200.parallel.tp import TensorParallel
    tp = TensorParallel(dist.group.WORLD, "cpu", fused=False)
    try:
        tp.selftest()
        q.put((rank, "ok"))
    except RuntimeError as e:
        q.put((rank, str(e)))
    dist.destroy_process_group()


@pytest.mark.parametrize("corrupt", ["", "2,0"])
def test_p2p_selftest_checks_every_ordered_pair(corrupt):
    """Three CPU ranks: the clean run passes on every rank; a word flipped on the receiving side of the pair 2 -> 0
    (host-side injection) makes EVERY rank refuse, naming the pair."""
    from ferrite_b200.parallel.selftest import expected_pattern, verify
    assert verify([expected_pattern(s, 1, 64) for s in range(3)], 1) == []
    bad = [expected_pattern(s, 1, 64) for s in range(3)]
    bad[2][5] ^= 1
    assert verify(bad, 1) == [(2, 1, 5)]
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_selftest_worker, args=(r, world, port, corrupt, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    if not corrupt:
        assert all(v == "ok" for v in got.values()), got
    else:
        assert all("2->0" in v and "refusing" in v for v in got.values()), got
