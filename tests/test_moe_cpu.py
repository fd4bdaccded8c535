"""Mixture-of-experts FFN on CPU: the engine's routed + shared expert block against the token-by-token oracle, for both
router forms, and expert parallelism over two gloo ranks (each rank owns half of the experts; partial sums reduce)."""
import dataclasses
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ferrite_b200.config import EngineConfig, tiny_hybrid
from ferrite_b200.engine.engine import Engine
from ferrite_b200.engine.executor import Segment
from ferrite_b200.models.ref import RefModel, route
from ferrite_b200.models.weights import init_weights

ROUTERS = {"softmax": {}, "sigmoid_group": dict(n_groups=4, topk_groups=2, route_scale=2.5)}


def tiny_moe(router):
    return dataclasses.replace(tiny_hybrid(), name="tiny-moe", n_experts=32, top_k=4, expert_inter=64, n_shared=1,
                               router=router, **ROUTERS[router])


def weights(cfg):
    w = init_weights(cfg, seed=0)
    g = torch.Generator().manual_seed(9)
    for k in w:
        if k.endswith("router_bias"):
            w[k] = torch.randn(w[k].shape, generator=g) * 0.1
    return w


def prompt_of(cfg, n=20):
    return torch.randint(0, cfg.vocab, (n,), generator=torch.Generator().manual_seed(1)).tolist()


@pytest.mark.parametrize("router", list(ROUTERS))
def test_moe_engine_matches_oracle(router):
    cfg = tiny_moe(router)
    w = weights(cfg)
    ref = RefModel(cfg, w)
    p = prompt_of(cfg)
    want = ref.forward(p, ref.new_state())
    eng = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=64), device="cpu")
    got, _, _ = eng.forward([Segment(0, 0, p, "all")])
    assert torch.allclose(got, want, atol=3e-5, rtol=1e-4)


def test_router_group_limit():
    cfg = tiny_moe("sigmoid_group")
    logits = torch.randn(5, cfg.n_experts, generator=torch.Generator().manual_seed(2))
    idx, wt = route(cfg, logits, torch.zeros(cfg.n_experts))
    per = cfg.n_experts // cfg.n_groups
    for t in range(5):
        assert len({int(e) // per for e in idx[t]}) <= cfg.topk_groups
        assert abs(float(wt[t].sum()) - cfg.route_scale) < 1e-5


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q, plen=20):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
        from ferrite_b200.parallel.tp import TensorParallel
        tp = TensorParallel(dist.group.WORLD, "cpu", fused=False)
        cfg = tiny_moe("softmax")
        eng = Engine(cfg, weights(cfg), EngineConfig(n_slots=1, max_ctx=128), device="cpu", tp=tp)
        logits, _, _ = eng.forward([Segment(0, 0, prompt_of(cfg, plen), "all")])
        q.put((rank, logits))
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        q.put((rank, repr(e)))


@pytest.mark.parametrize("plen", [20, 75])
def test_expert_parallel_two_ranks(plen):
    """20 rows: replicated rows, owners' partial sums reduced. 75 rows: tokens sharded by rows, routed pairs dispatched
    to the expert owners and combined back (process-group statement of the fused kernels)."""
    cfg = tiny_moe("softmax")
    eng = Engine(cfg, weights(cfg), EngineConfig(n_slots=1, max_ctx=128), device="cpu")
    want, _, _ = eng.forward([Segment(0, 0, prompt_of(cfg, plen), "all")])
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, plen)) for r in range(2)]
    for p in procs:
        p.start()
    outs = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
    for rank, logits in outs:
        assert not isinstance(logits, str), logits
        assert torch.allclose(logits, want, atol=5e-5, rtol=1e-4), rank


def test_expert_heat_counters(tmp_path, monkeypatch):
    """FE_EXPERT_HEAT: every routed pick of every MoE layer is counted (top_k per token and layer), read through the
    engine and written to the file when the engine is closed."""
    import json

    import torch

    from ferrite_b200.config import EngineConfig, tiny_mla
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment
    path = tmp_path / "heat.json"
    monkeypatch.setenv("FE_EXPERT_HEAT", str(path))
    cfg = tiny_mla()
    eng = Engine(cfg, None, EngineConfig(n_slots=1, max_ctx=64), device="cpu")
    toks = torch.randint(0, cfg.vocab, (21,), generator=torch.Generator().manual_seed(0)).tolist()
    eng.forward([Segment(0, 0, toks[:20], "none")])
    eng.forward([Segment(0, 20, toks[20:], "last")])
    heat = eng.expert_heat()
    moe_layers = [i for i in range(cfg.n_layers) if cfg.is_moe(i)]
    assert sorted(heat) == moe_layers
    for i in moe_layers:
        assert sum(heat[i]) == 21 * cfg.top_k and len(heat[i]) == cfg.n_experts + 1 and max(heat[i]) > 0
    eng.close()
    assert json.loads(path.read_text())["layers"][str(moe_layers[0])] == heat[moe_layers[0]]
    monkeypatch.delenv("FE_EXPERT_HEAT")
    assert Engine(cfg, None, EngineConfig(n_slots=1, max_ctx=64), device="cpu").expert_heat() == {}
