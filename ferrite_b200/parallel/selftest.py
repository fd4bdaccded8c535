"""Start-up self-test of the peer-to-peer paths: before serving, every ordered pair (source GPU, destination GPU) moves
a 64 KB pattern that names the pair and the word, and the destination checks it on the host. A mismatch refuses to
start: a link that corrupts data would otherwise surface as wrong tokens much later. The reference does this for its
expert cards (`p2p_selftest`, `crates/fe-dsc/src/engine.rs:2500-2529`: a 64 KB pattern per ordered pair by peer copy,
"refuses to run on mismatch").

On GPUs the pattern travels by the same plain peer stores the fused collective kernels use (`p2p_pattern_kernel`,
`csrc/comm.cu`) into the symmetric workspace; on CPU ranks (gloo) it travels through the process group, which lets the
checking logic and the refusal be tested without GPUs. `FE_TEST_P2P_CORRUPT="src,dst"` flips one received word of that
pair on the destination (host-side fault injection)."""
from __future__ import annotations

import os
from typing import List, Tuple

import numpy as np
import torch
import torch.distributed as dist

N_WORDS = 16384          # 64 KB per ordered pair


def expected_pattern(src: int, dst: int, n: int = N_WORDS, seed: int = 0x5EED) -> np.ndarray:
    """The words source `src` writes for destination `dst` (the kernel computes the same)."""
    i = np.arange(n, dtype=np.uint64)
    v = (np.uint64(seed) ^ (np.uint64(src) * np.uint64(0x9E3779B1)) ^ (np.uint64(dst) * np.uint64(0x85EBCA77))
         ^ (i * np.uint64(0xC2B2AE3D))) & np.uint64(0xFFFFFFFF)
    v ^= v >> np.uint64(15)
    v = (v * np.uint64(0x2C1B3C6D)) & np.uint64(0xFFFFFFFF)
    v ^= v >> np.uint64(12)
    return v.astype(np.uint32)


def verify(received: List[np.ndarray], rank: int, seed: int = 0x5EED) -> List[Tuple[int, int, int]]:
    """received[src] = words that arrived from `src`. Returns (src, dst, first bad word) for every pair that differs."""
    bad = []
    for src, got in enumerate(received):
        want = expected_pattern(src, rank, len(got), seed)
        diff = np.nonzero(got != want)[0]
        if diff.size:
            bad.append((src, rank, int(diff[0])))
    return bad


def _inject(received: List[np.ndarray], rank: int) -> None:
    spec = os.environ.get("FE_TEST_P2P_CORRUPT", "")
    if spec:
        s, d = (int(x) for x in spec.split(","))
        if d == rank and 0 <= s < len(received):
            received[s] = received[s].copy()
            received[s][7] ^= 0x10


def p2p_selftest(tp, seed: int = 0x5EED) -> None:
    """Collective: every rank calls it. Raises RuntimeError on every rank when any ordered pair failed."""
    world, rank = tp.world, tp.rank
    if world == 1:
        return
    if tp.fused:
        n = N_WORDS
        tp.C.p2p_pattern(tp.comm, 0, n, seed)
        torch.cuda.synchronize(tp.device)
        dist.barrier(tp.group)                                   # every source has finished writing
        words = tp.ws[tp.data_offset:].view(torch.int32)
        slot = tp.slot_floats
        received = [words[src * slot:src * slot + n].cpu().numpy().view(np.uint32) for src in range(world)]
    else:
        send = [torch.from_numpy(expected_pattern(rank, d, N_WORDS, seed).view(np.int32).copy()) for d in range(world)]
        recv = [torch.empty(N_WORDS, dtype=torch.int32) for _ in range(world)]
        if tp.device.type == "cuda":
            send = [t.to(tp.device) for t in send]
            recv = [t.to(tp.device) for t in recv]
            dist.all_to_all(recv, send, group=tp.group)
        else:
            # gloo has no all_to_all on CPU tensors in every build: gather every rank's outbox and pick this rank's lane
            box = [None] * world
            dist.all_gather_object(box, [t.numpy() for t in send], group=tp.ctrl_group())
            recv = [torch.from_numpy(box[src][rank]) for src in range(world)]
        received = [t.cpu().numpy().view(np.uint32) for t in recv]
    _inject(received, rank)
    bad = verify(received, rank, seed)
    flags = [None] * world
    dist.all_gather_object(flags, bad, group=tp.ctrl_group())
    if tp.fused:
        # leave the workspace as the kernels expect it: zero pairs, then nobody proceeds before everyone has cleaned up
        words[: world * tp.slot_floats].view(world, tp.slot_floats)[:, :N_WORDS].zero_()
        torch.cuda.synchronize(tp.device)
        dist.barrier(tp.group)
    allbad = [b for f in flags for b in f]
    if allbad:
        pairs = ", ".join(f"{s}->{d} (word {w})" for s, d, w in allbad)
        raise RuntimeError(f"peer-to-peer self-test failed for {len(allbad)} ordered pair(s): {pairs}; refusing to serve")
