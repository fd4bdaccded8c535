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
