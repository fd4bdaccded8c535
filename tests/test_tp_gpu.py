"""Fused compute + collective kernels on 2+ GPUs of one box (child processes, NVLS off, plain peer loads/stores).
Skipped on a single GPU."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    try:
        _worker_body(rank, world, port, q)
    except Exception as e:                       # report instead of leaving the parent waiting
        import traceback
        q.put((rank, False, {"exception": repr(e), "trace": traceback.format_exc()[-1500:]}))


def _worker_body(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    from ferrite_b200.ops.cuda_ops import CudaOps
    from ferrite_b200.parallel.tp import TensorParallel
    tp = TensorParallel(dist.group.WORLD, dev, fused=True)
    ops = CudaOps(dev)
    res = {}
    g = torch.Generator(device=dev).manual_seed(1)          # same seed: every rank draws the same tensors
    N, Kfull = 5120, 17408
    Kr = Kfull // world
    wfull = (torch.randn(N, Kfull, generator=g, device=dev) * 0.03).to(torch.bfloat16)
    ok = True
    for M in (1, 4, 8, 48):
        x = torch.randn(M, Kfull, generator=g, device=dev).to(torch.bfloat16)
        r = torch.randn(M, N, generator=g, device=dev).to(torch.bfloat16)
        want = x.float() @ wfull.float().t() + r.float()
        xs = x[:, rank * Kr:(rank + 1) * Kr].contiguous()
        ws = wfull[:, rank * Kr:(rank + 1) * Kr].contiguous()
        outs = [tp.linear_allreduce(ops, xs, ws, r) for _ in range(3)]       # epochs advance, buffers alternate
        err = (outs[-1].float() - want).abs().max().item() / want.abs().max().item()
        same = all(torch.equal(outs[0], o) for o in outs)
        gathered = [torch.empty_like(outs[0]) for _ in range(world)]
        dist.all_gather(gathered, outs[0])
        identical = all(torch.equal(gathered[0], t) for t in gathered)
        res[f"M{M}"] = (err, same, identical)
        ok = ok and err < 2e-2 and same and identical
    # vocabulary-parallel argmax
    V = 151936
    per = (V + world - 1) // world
    full = torch.randn(3, V, generator=g, device=dev)
    full[1, 140000] = 99.0
    shard = full[:, rank * per:min(V, (rank + 1) * per)].contiguous()
    _, (ids, fin) = tp.gather_logits(ops, shard, True, rank * per, V)
    res["argmax"] = (ids.tolist(), full.argmax(-1).tolist())
    ok = ok and ids.tolist() == full.argmax(-1).tolist()
    # the same step inside a CUDA graph (device-side epochs make the kernels replayable)
    x = torch.randn(1, Kfull, generator=g, device=dev).to(torch.bfloat16)
    r = torch.randn(1, N, generator=g, device=dev).to(torch.bfloat16)
    xs = x[:, rank * Kr:(rank + 1) * Kr].contiguous()
    ws = wfull[:, rank * Kr:(rank + 1) * Kr].contiguous()
    eager = tp.linear_allreduce(ops, xs, ws, r).clone()
    torch.cuda.synchronize()
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        y = tp.linear_allreduce(ops, xs, ws, r)
    for _ in range(4):
        gr.replay()
    torch.cuda.synchronize()
    res["graph"] = torch.equal(y, eager)
    ok = ok and res["graph"]
    tp.check()
    # timing of the fused decode reduction, max over ranks (device events)
    e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
    dist.barrier(); torch.cuda.synchronize()
    e0.record()
    for _ in range(50):
        gr.replay()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / 50], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res["fused_gemv_allreduce_us"] = t.item() * 1e3
    q.put((rank, ok, res))
    dist.barrier()
    dist.destroy_process_group()


def test_fused_collectives(ext):
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs 2+ GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    import queue as _queue
    import time
    outs, deadline = [], time.time() + 240
    while len(outs) < world and time.time() < deadline:
        try:
            outs.append(q.get(timeout=2))
        except _queue.Empty:
            if any(p.exitcode not in (None, 0) for p in procs):
                break
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()
    assert len(outs) == world, f"only {len(outs)} of {world} ranks reported: {outs}"
    for rank, ok, res in outs:
        print(rank, res)
        assert ok, (rank, res)


def test_peer_wait_times_out_cleanly(ext):
    """A wait on a flag nobody sets runs out after its limit, sets the status word and returns: the context
    stays usable (no trap, no hang)."""
    from ferrite_b200._ext import load
    C = load()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    C.comm_wait_probe(flag, 7, 1 << 16, status)
    torch.cuda.synchronize()
    assert status.item() == 2
    assert torch.ones(4, device="cuda").sum().item() == 4.0
