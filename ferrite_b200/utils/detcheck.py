"""Determinism check: every kernel whose result passes through a cross-CTA (or cross-GPU) hand-off is run repeatedly on
the same inputs and must return the same bits every time.

    python -m ferrite_b200.utils.detcheck [--reps 20]

Hand-offs covered: split-K partial sums of the tcgen05 GEMMs (few-row "swapped" form), stream-K slots of the NVFP4
few-row kernel, split-K of the few-row mma GEMV, split-KV partials + combine of decode attention, the chunked Gated
DeltaNet scan (state handed from chunk to chunk), MoE pair GEMVs + fixed-order combine, the EXL3 cross-warp sum. Arrival
order differs from run to run; the sums are taken in a fixed order, which is what this checks. Prints one JSON line;
exit code 1 if any case changed a bit. The role of the reference's `exl3-detcheck` (`crates/fe-exl3/src/bin/exl3-detcheck.rs`),
widened to every family.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def cases(ops, dev):
    from ..ops.qweight import quantize_weight
    g = torch.Generator(device=dev).manual_seed(5)
    rnd = lambda *s, scale=1.0, dtype=torch.bfloat16: (torch.randn(*s, generator=g, device=dev) * scale).to(dtype)
    out = {}
    x1, x4, x17 = rnd(1, 5120), rnd(4, 5120), rnd(17, 5120)
    w = rnd(5120, 5120, scale=0.03)
    wk = rnd(2048, 17408, scale=0.02)
    xk = rnd(17, 17408)
    out["gemv 1 row"] = lambda: ops.linear(x1, w)
    out["gemv_mma 4 rows (split k)"] = lambda: ops.linear(x4, w)
    out["tcgen05 gemm 17 rows, K 17408 (split k)"] = lambda: ops.linear(xk, wk)
    out["tcgen05 gemm 17 rows fp32 out"] = lambda: ops.linear(x17, w, out_f32=True)
    q = quantize_weight(w)
    fp4 = type(ops)(dev)
    fp4.fp4_act = True
    out["nvfp4 few-row tcgen05 kernel (stream-k slots)"] = lambda: fp4.linear(x1, q)
    out["nvfp4 few-row kernel, 4 rows"] = lambda: fp4.linear(x4, q)
    # decode attention: split-KV partials + combine
    hd, nq, nkv, kvb, ctx = 256, 8, 2, 64, 1500
    nb = (ctx + kvb - 1) // kvb + 1
    bt = torch.arange(nb, device=dev, dtype=torch.int32).view(1, nb)
    kc, vc = rnd(nb, kvb, nkv, hd), rnd(nb, kvb, nkv, hd)
    qv = rnd(1, nq * hd)
    proj = rnd(1, nq * hd * 2 + 2 * nkv * hd)
    i32 = lambda *v: torch.tensor(list(v), device=dev, dtype=torch.int32)
    out["decode attention, 8 key splits"] = lambda: ops.attention(qv, proj, kc, vc, i32(0), i32(ctx), bt, kvb, nq, nkv, hd, True, nsplit=8,
                                                                  segs=(i32(0), i32(0), i32(1), 1))
    # chunked Gated DeltaNet scan
    nk, nv, dk, dv, T = 4, 8, 128, 128, 300
    conv_dim = 2 * nk * dk + nv * dv
    gproj = rnd(T, conv_dim + nv * dv + 2 * nv)
    qkv = rnd(T, conv_dim)
    A_log, dtb = rnd(nv, scale=0.3, dtype=torch.float32), rnd(nv, scale=0.3, dtype=torch.float32)
    rec0, conv0 = rnd(1, nv, dk, dv, scale=0.2, dtype=torch.float32), rnd(1, 3, conv_dim)

    def gdn():
        rec, conv = rec0.clone(), conv0.clone()
        y = ops.gdn_rec(qkv, gproj, rec, conv, A_log, dtb, i32(0), i32(0), i32(T), nk, nv, dk, dv, 1e-6, commit=True, chunked=True, max_rows=T)
        return torch.cat([y.flatten().float(), rec.flatten()])
    out["gdn chunked scan, 300 rows"] = gdn
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reps", type=int, default=20)
    a = ap.parse_args(argv)
    from ..ops.cuda_ops import CudaOps
    dev = torch.device("cuda", 0)
    ops = CudaOps(dev)
    report, bad = {}, 0
    for name, fn in cases(ops, dev).items():
        first = fn().clone()
        torch.cuda.synchronize(dev)
        same = all(torch.equal(first, fn()) for _ in range(a.reps))
        report[name] = "same bits" if same else "CHANGED"
        bad += 0 if same else 1
    report["status_word"] = ops.status()
    print(json.dumps({"reps": a.reps, "cases": report}))
    return 1 if bad or report["status_word"] else 0


if __name__ == "__main__":
    sys.exit(main())
