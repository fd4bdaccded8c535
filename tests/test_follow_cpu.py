"""Leader / follower tensor parallelism on two gloo ranks: the leader runs the scheduler (prompt cache, snapshots,
chunked prefill, decode) over a mirrored engine, the follower only replays the call stream; the generated tokens must be
those of a single-rank run."""
import datetime
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ferrite_b200.config import EngineConfig, tiny_hybrid
from ferrite_b200.engine.engine import Engine
from ferrite_b200.engine.sampler import Sampling
from ferrite_b200.engine.scheduler import SchedOptions, Scheduler, generate
from ferrite_b200.models.weights import init_weights


def _prompts(cfg):
    g = torch.Generator().manual_seed(11)
    base = torch.randint(0, cfg.vocab, (90,), generator=g).tolist()
    return [base[:70], base[:70] + torch.randint(0, cfg.vocab, (12,), generator=g).tolist(), base[:33]]


def _run(eng):
    sched = Scheduler(eng, SchedOptions(spec=0))
    out = []
    for p in _prompts(eng.full_cfg):          # one after the other, so later prompts resume from cached prefixes
        out.append(generate(sched, [p], Sampling(max_tokens=12))[0])
    return out


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
        from ferrite_b200.engine.follow import Leader, follow
        from ferrite_b200.parallel.tp import TensorParallel
        tp = TensorParallel(dist.group.WORLD, "cpu", fused=False)
        cfg = tiny_hybrid()
        eng = Engine(cfg, init_weights(cfg, seed=0), EngineConfig(n_slots=2, max_ctx=256, prefill_chunk=64), device="cpu", tp=tp)
        if rank == 0:
            lead = Leader(eng, tp)
            toks = _run(lead)
            lead.stop_followers()
            q.put((rank, toks))
        else:
            q.put((rank, follow(eng, tp)))
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, "ERR " + repr(e) + traceback.format_exc()[-800:]))


def test_follower_replays_the_leaders_calls():
    cfg = tiny_hybrid()
    want = _run(Engine(cfg, init_weights(cfg, seed=0), EngineConfig(n_slots=2, max_ctx=256, prefill_chunk=64), device="cpu"))
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    outs = dict(q.get(timeout=180) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert not isinstance(outs[0], str), outs[0]
    assert not isinstance(outs[1], str), outs[1]
    assert outs[0] == want
    assert outs[1] > 10          # calls replayed by the follower


# ---- a draft model under tensor parallelism: mirrored at the Drafter interface ------------------------------------
def _spec_cfg(kind="block"):
    cfg = tiny_hybrid()
    if kind == "mtp":
        cfg.tap_layers = [cfg.n_layers - 1]
        cfg.tie_embeddings = False            # the head then borrows the target's output matrix: one vocabulary shard per rank
    else:
        cfg.tap_layers = sorted({max(0, cfg.n_layers * (i + 1) // 4 - 1) for i in range(3)})
    return cfg


def _spec_run(eng, tp=None, tree=False, kind="block"):
    from ferrite_b200.models.drafter import BlockDrafter, drafter_config_for
    cfg = eng.full_cfg
    if kind == "mtp":
        from ferrite_b200.models.mtp import MtpDrafter
        drafter = MtpDrafter(eng, n_slots=2, max_ctx=256, depth=4)
    else:
        drafter = BlockDrafter(drafter_config_for(cfg), target_hidden=cfg.hidden, n_taps=len(cfg.tap_layers), n_slots=2,
                               max_ctx=256, device="cpu", block=8, tp=tp)
    if tp is not None and tp.rank != 0:
        from ferrite_b200.engine.follow import follow
        return follow(eng, tp, drafter)
    if tp is not None:
        from ferrite_b200.engine.follow import Leader
        eng = Leader(eng, tp)
        drafter = eng.attach_drafter(drafter)
    sched = Scheduler(eng, SchedOptions(spec=4, tree_rows=6 if tree else 0), drafter=drafter)
    out = []
    for p in _prompts(cfg):
        out.append(generate(sched, [p], Sampling(max_tokens=12))[0])
    stats = (sched.stats["drafted"], sched.stats["accepted"])
    if tp is not None:
        eng.stop_followers()
    return out, stats


def _spec_worker(rank, world, port, q, tree, kind="block"):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
        from ferrite_b200.parallel.tp import TensorParallel
        tp = TensorParallel(dist.group.WORLD, "cpu", fused=False)
        cfg = _spec_cfg(kind)
        eng = Engine(cfg, init_weights(cfg, seed=0), EngineConfig(n_slots=2, max_ctx=256, prefill_chunk=64), device="cpu", tp=tp)
        q.put((rank, _spec_run(eng, tp, tree, kind)))
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, "ERR " + repr(e) + traceback.format_exc()[-1200:]))


def _spec_case(tree, kind="block"):
    cfg = _spec_cfg(kind)
    mk = lambda: Engine(cfg, init_weights(cfg, seed=0), EngineConfig(n_slots=2, max_ctx=256, prefill_chunk=64), device="cpu")
    plain = _run(mk())
    want, want_stats = _spec_run(mk(), None, tree, kind)
    assert want == plain                      # speculation does not change greedy output
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_spec_worker, args=(r, 2, port, q, tree, kind)) for r in range(2)]
    for p in procs:
        p.start()
    outs = dict(q.get(timeout=240) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert not isinstance(outs[0], str), outs[0]
    assert not isinstance(outs[1], str), outs[1]
    got, stats = outs[0]
    assert got == want
    # the sharded drafter drafts what the whole one drafts: same proposals, same acceptance
    assert stats == want_stats and stats[0] > 0
    assert outs[1] > 20                       # engine and drafter calls replayed by the follower


def test_block_drafter_is_mirrored_under_tensor_parallelism():
    _spec_case(tree=False)


def test_block_drafter_tree_is_mirrored_under_tensor_parallelism():
    _spec_case(tree=True)


def test_mtp_head_is_mirrored_under_tensor_parallelism():
    _spec_case(tree=False, kind="mtp")
