"""Kernel micro-benchmarks with roofline fractions (the role of the reference's `exl3-bench`, `fp4-bench`,
`fabric-bench` and `ferrite gemm-bench` binaries, `crates/fe-exl3/src/bin`, `crates/fe-fp4/src/bin`).

    python -m ferrite_b200.utils.microbench gemv --m 1 --n 34816 --k 5120 --swiglu
    python -m ferrite_b200.utils.microbench gemm --m 2048 --n 5120 --k 17408
    python -m ferrite_b200.utils.microbench layer           # every linear of one 27B decode step

Timing: CUDA events on the launching stream, `--warmup` untimed launches (>= 3), an L2 flush (a write larger
than L2) before every timed launch, median over `--iters`. Fractions are of the measured copy bandwidth / cuBLAS
bf16 rate in MEASURED_PEAKS.json when that file is present ("of measured"), else of 6.65 TB/s / 1.59 PFLOP/s
("of fallback").
"""
from __future__ import annotations

import argparse
import json
import statistics
from pathlib import Path

import torch


def peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"], d["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


class Timer:
    def __init__(self, dev, warmup=3, iters=20, flush=True, graph=False, trace=False, hot=False):
        self.dev, self.warmup, self.iters, self.flush, self.graph, self.trace, self.hot = dev, max(3, warmup), iters, flush, graph, trace, hot
        # flush = write a buffer larger than L2, then read another one so the cache is left full of CLEAN lines
        # (dirty lines would be written back during the timed kernel and charged to it)
        self.junk = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if flush else None
        self.junk2 = torch.zeros(64 << 20, dtype=torch.float32, device=dev) if flush else None

    def run(self, fn):
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize(self.dev)
        ts = []
        for _ in range(self.iters):
            if self.flush:
                self.junk.fill_(1)
                self.junk2.sum()
            e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
            torch.cuda.synchronize(self.dev)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize(self.dev)
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)


def rnd(*shape, scale=1.0, dtype=torch.bfloat16, dev="cuda"):
    return (torch.randn(*shape, device=dev) * scale).to(dtype)


def report(name, ms, nbytes, flops, extra=None):
    hbm, tf, tag = peaks()
    gbs = nbytes / ms / 1e6
    tfl = flops / ms / 1e9
    out = {"kernel": name, "ms": round(ms, 5), "GB/s": round(gbs, 1), "TFLOP/s": round(tfl, 2),
           "frac_hbm": round(gbs / hbm, 3), "frac_bf16": round(tfl / tf, 3), "peaks": tag}
    if extra:
        out.update(extra)
    print(json.dumps(out), flush=True)
    return out


def bench_linear(ops, t, m, n, k, swiglu=False, norm=False, res=False, label=None, fp4=False):
    rows = 2 * n if swiglu else n
    x, w = rnd(m, k), rnd(rows, k, scale=0.02)
    wbytes = rows * k * 2
    if fp4:
        from ..ops.qweight import quantize_weight
        w = quantize_weight(w)
        wbytes = rows * k // 2 + rows * k // 16
    nw = rnd(k, scale=0.1) if norm else None
    r = rnd(m, n) if res else None
    if t.graph:
        # device time inside a stream of such calls, as in a decode step: R calls over R copies of the weight (together
        # larger than L2, so every call streams from HBM) captured in one CUDA graph; time of a replay / R. A lone
        # call timed from an idle GPU also measures the host's launch path, which is longer than these kernels.
        import copy
        reps = max(2, min(24, -(-(600 << 20) // wbytes)))
        ws = [w] * reps if t.hot else [w] + [copy.deepcopy(w) if fp4 else w.clone() for _ in range(reps - 1)]
        if fp4:
            for i, wi in enumerate(ws):                      # each call prefetches the weight of the one after it
                wi.pair, wi.next = swiglu, ws[(i + 1) % reps]

        def chain():
            for wi in ws:
                ops.linear(x, wi, norm_w=nw, res=r, swiglu=swiglu)
        chain()
        trace = None
        if t.trace and fp4 and ops.fp4_act:
            trace = torch.zeros(8 * 1024 * 8, dtype=torch.int64, device=x.device)
            ops.C.gemv_nvfp4_tc_trace_set(trace)
            reps = 8
            ws = ws[:8] if len(ws) >= 8 else (ws * 8)[:8]
            if fp4 and not t.hot:
                for i, wi in enumerate(ws):
                    wi.next = ws[(i + 1) % reps]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            chain()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                chain()
        torch.cuda.current_stream().wait_stream(side)
        flush, t.flush = t.flush, False
        ms = t.run(g.replay) / reps
        t.flush = flush
        if trace is not None:
            # the capture stamped calls 0..7 into regions (0..7 + eager calls before it) % 8: the last two calls of the
            # graph are the regions with the two latest end times
            ops.C.gemv_nvfp4_tc_trace_set(None)
            tr = trace.view(8, 1024, 8).cpu()
            used = tr[:, :, 0] > 0
            ends = [int(tr[c, :, 7][used[c]].max()) if used[c].any() else 0 for c in range(8)]
            order = sorted(range(8), key=lambda c: ends[c])
            last, prev = order[-1], order[-2]
            names = ["entry", "set-up done", "dependency met", "row statistics", "quantised", "first stage landed",
                     "last MMA issued", "epilogue done"]
            rel = tr[last][used[last]].double() - ends[prev]
            print(json.dumps({"trace_us_after_previous_kernel_end": {
                n: {"median": round(float(rel[:, i].median()) / 1e3, 2), "max": round(float(rel[:, i].max()) / 1e3, 2)}
                for i, n in enumerate(names)}, "ctas": int(used[last].sum())}), flush=True)
    else:
        ms = t.run(lambda: ops.linear(x, w, norm_w=nw, res=r, swiglu=swiglu))
    nbytes = wbytes + m * k * 2 + m * n * 2 * (2 if res else 1)
    return report(label or f"linear m{m} n{n} k{k}{' swiglu' if swiglu else ''}", ms, nbytes, 2.0 * m * rows * k,
                  {"m": m, "n": n, "k": k})


def graph_time(t, chain, reps):
    """ms per call of `chain` (which issues `reps` calls over distinct buffers) replayed as one CUDA graph: device time in
    a stream of such calls, without the host's launch path."""
    chain()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        chain()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            chain()
    torch.cuda.current_stream().wait_stream(side)
    flush, t.flush = t.flush, False
    ms = t.run(g.replay) / reps
    t.flush = flush
    return ms


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemv", "gemm", "layer", "attn_decode", "attn_prefill", "gdn", "moe", "exl3",
                                     "head_linear", "ffn_fp4", "select"])
    ap.add_argument("--kv", default="bf16", help="attn_decode: cache form (bf16 | fp8 | int6 | int4)")
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--n", type=int, default=5120)
    ap.add_argument("--k", type=int, default=5120)
    ap.add_argument("--bits", type=int, default=4, help="exl3: bits per weight")
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--splits", type=int, default=0, help="attn_decode: key splits (0 = by context length)")
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--norm", action="store_true")
    ap.add_argument("--res", action="store_true")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--hot", action="store_true", help="with --graph: every call uses the same weight (L2-resident when it fits)")
    ap.add_argument("--trace", action="store_true",
                    help="with --graph --fp4: print where the few-row tensor-core kernel's time goes (%%globaltimer stamps)")
    ap.add_argument("--graph", action="store_true",
                    help="gemv/gemm: time the call inside a CUDA graph of back-to-back calls over weight copies larger than L2")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--fp4", action="store_true", help="NVFP4 weights and activations (block-scaled tcgen05 GEMM)")
    ap.add_argument("--fp8b", action="store_true", help="gemm: block-scaled e4m3 (1x128 activations, 128x128 weights)")
    ap.add_argument("--terms", type=int, default=3, help="with --fp4, few rows: NVFP4 renderings per activation row (0 = older fused kernel)")
    ap.add_argument("--prefetch", type=int, default=48, help="with --fp4 --graph, few rows: MB of the next call's weight asked into L2")
    ap.add_argument("--ctas", type=int, default=1, help="with --fp4, few rows: CTAs per SM of the tensor-core kernel")
    ap.add_argument("--a16", action="store_true", help="with --fp4: keep 16-bit activations (W4A16 GEMV)")
    a = ap.parse_args()
    from ..ops.cuda_ops import CudaOps
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    ops = CudaOps(dev)
    ops.fp4_act = a.fp4 and not a.a16
    ops.fp4_terms, ops.fp4_tc_ctas, ops.fp4_prefetch_mb = a.terms, a.ctas, a.prefetch
    t = Timer(dev, a.warmup, a.iters, flush=not a.no_flush, graph=a.graph, trace=a.trace, hot=a.hot)
    if a.what == "exl3":
        # the three kernels of an EXL3 linear for few rows: input rotation, trellis GEMV, output rotation (+ residual)
        from ..formats.exl3 import Exl3Tensor
        from ..ops.exl3_linear import HAD, Exl3Linear
        nbytes = a.k * a.n * a.bits // 8
        reps = max(2, min(12, -(-(300 << 20) // nbytes)))
        lins = [Exl3Linear(Exl3Tensor.random(a.k, a.n, a.bits, seed=i), dev) for i in range(reps)]
        x = rnd(a.m, a.k)
        xh = torch.empty(a.m, a.k, dtype=torch.float32, device=dev)
        z = torch.empty(a.m, a.n, dtype=torch.float32, device=dev)
        y = torch.empty(a.m, a.n, dtype=torch.bfloat16, device=dev)
        t.flush = False
        C = ops.C
        state = [0]

        def gemv():
            state[0] = (state[0] + 1) % reps                       # weight copies larger than L2 together
            C.exl3_gemv(z, xh, lins[state[0]].trellis, a.bits)
        report(f"exl3 input rotation m{a.m} k{a.k}", t.run(lambda: C.exl3_had(xh, x, lins[0].suh, None, None, HAD)), a.m * a.k * 6, 0)
        report(f"exl3 trellis gemv m{a.m} n{a.n} k{a.k} {a.bits}bpw", t.run(gemv), nbytes, 2.0 * a.m * a.n * a.k)
        report(f"exl3 output rotation m{a.m} n{a.n}", t.run(lambda: C.exl3_had(y, z, None, lins[0].svh, None, HAD)), a.m * a.n * 6, 0)
        return
    if a.what == "gemm" and a.fp8b:
        x = rnd(a.m, a.k)
        wq, ws = ops.quantize_weight_fp8_block(rnd(a.n, a.k, scale=0.05))
        ms = t.run(lambda: ops.linear_fp8_block(x, wq, ws))
        xq, xs = ops.quantize_act_fp8_block(x)
        y = torch.empty(a.m, a.n, dtype=torch.bfloat16, device=dev)
        ms_g = t.run(lambda: ops.C.gemm_fp8_block(y, xq, xs, wq, ws, None, a.k, ops.status_word))
        report(f"fp8 block-scaled linear (quantise + gemm) m{a.m} n{a.n} k{a.k}", ms, a.n * a.k + a.m * a.k * 3 + a.m * a.n * 2,
               2.0 * a.m * a.n * a.k)
        report(f"fp8 block-scaled gemm only m{a.m} n{a.n} k{a.k}", ms_g, a.n * a.k + a.m * a.k + a.m * a.n * 2, 2.0 * a.m * a.n * a.k)
    elif a.what in ("gemv", "gemm"):
        bench_linear(ops, t, a.m, a.n, a.k, a.swiglu, a.norm, a.res, fp4=a.fp4)
    elif a.what == "layer":
        from ..config import hybrid_27b
        c = hybrid_27b()
        tot_ms = tot_b = 0.0
        for m in (a.m,):
            for label, n, k, sw, nm, rs in (
                    ("gdn in_proj", c.gdn_in_dim, c.hidden, False, True, False),
                    ("gdn out_proj", c.hidden, c.lin_v_heads * c.lin_dv, False, False, True),
                    ("attn in_proj", c.attn_in_dim, c.hidden, False, True, False),
                    ("attn out_proj", c.hidden, c.n_q * c.head_dim, False, False, True),
                    ("mlp gate_up", c.inter, c.hidden, True, True, False),
                    ("mlp down", c.hidden, c.inter, False, False, True),
                    ("lm_head", c.vocab, c.hidden, False, True, False)):
                r = bench_linear(ops, t, m, n, k, sw, nm, rs, label=f"{label} m{m}", fp4=a.fp4)
                tot_ms += r["ms"]
                tot_b += r["GB/s"] * r["ms"]
        print(json.dumps({"sum_ms": round(tot_ms, 4), "mean_GB/s": round(tot_b / tot_ms, 1)}))
    elif a.what == "head_linear":
        # per-head up-projections of latent attention at the 671B-class shape: 128 heads, latent 512, head width 128
        nh, L, dn = 128, 512, 128
        for N, K, label in ((L, dn, "key up-projection into the query"), (dn, L, "value up-projection")):
            wbytes = nh * N * K * 2
            reps = max(2, min(24, -(-(400 << 20) // wbytes)))
            Ws = [rnd(nh, N, K, scale=K ** -0.5) for _ in range(reps)]
            x = rnd(a.m, nh, K)
            ms = graph_time(t, lambda: [ops.head_linear(x, W) for W in Ws], reps)
            report(f"head_linear rows{a.m} {nh} heads N{N} K{K} ({label})", ms, wbytes + a.m * nh * (N + K) * 2,
                   2.0 * a.m * nh * N * K)
    elif a.what == "ffn_fp4":
        # dense FFN block of the 27B model on prompt rows, NVFP4 weights and activations: gate|up + SwiGLU + down with the
        # activation re-quantised in the first GEMM's epilogue, against the same block through a bf16 activation
        from ..ops.qweight import quantize_weight
        H, I, M = 5120, 17408, max(a.m, 65)
        ops.fp4_act = ops.fp4_prompt = True
        x, nw, res = rnd(M, H), rnd(H, scale=0.1), rnd(M, H)
        w_gu, w_dn = quantize_weight(rnd(2 * I, H, scale=H ** -0.5)), quantize_weight(rnd(H, I, scale=I ** -0.5))
        flops = 2.0 * M * 3 * H * I
        wbytes = 3 * H * I // 2 + 3 * H * I // 16
        for fused in (True, False):
            ops.fp4_fuse_requant = fused
            ms = t.run(lambda: ops.ffn(x, w_gu, w_dn, nw, 1e-6, res))
            act_bytes = M * I // 2 + M * I // 16 if fused else M * I * 2 * 2 + M * I // 2 + M * I // 16
            report(f"ffn nvfp4 rows{M} {'SwiGLU output written as NVFP4' if fused else 'bf16 activation + quantiser'}", ms,
                   wbytes + M * H * 2 * 3 + act_bytes, flops)
        ops.fp4_fuse_requant = True
    elif a.what == "select":
        # sparse-attention selection of decode rows: indexer scores over --ctx entries (32 heads x 128 dims), exact top-2048
        rows, n, nh, D, k = a.m, a.ctx, 32, 128, 2048
        q, w = rnd(rows, nh, D, scale=0.3), torch.rand(rows, nh, device=dev)
        keys = rnd(1, n, D)
        slot = torch.zeros(rows, dtype=torch.int32, device=dev)
        length = torch.full((rows,), n, dtype=torch.int32, device=dev)
        ms = t.run(lambda: ops.index_score(q, w, 0.0, keys, slot, length, n))
        report(f"index_score rows{rows} entries{n}", ms, n * D * 2 + rows * n * 4, 2.0 * rows * n * nh * D)
        score = ops.index_score(q, w, 0.0, keys, slot, length, n)
        ms = t.run(lambda: ops.topk_select(score, k))
        report(f"topk_select rows{rows} entries{n} k{k}", ms, rows * n * 4 * 5, 0.0)
    elif a.what in ("attn_decode", "attn_prefill"):
        nq, nkv, hd, kvb = 24, 4, 256, 64
        nslots = 4 if a.what == "attn_decode" else 1
        rows = a.m if a.what == "attn_decode" else a.ctx
        nb = (a.ctx + kvb - 1) // kvb
        kc = rnd(nslots * nb, kvb, nkv, hd)
        vc = rnd(nslots * nb, kvb, nkv, hd)
        bt = torch.arange(nslots * nb, device=dev, dtype=torch.int32).view(nslots, nb)
        proj = rnd(rows, nq * hd * 2 + 2 * nkv * hd)
        q = rnd(rows, nq, hd)
        if a.what == "attn_decode":
            slot = (torch.arange(rows, device=dev, dtype=torch.int32) % nslots).contiguous()
            kvlen = torch.full((rows,), a.ctx, device=dev, dtype=torch.int32)
            ns = a.splits or max(1, min(64, 1 << ((a.ctx + 255) // 256 - 1).bit_length()))
            if a.kv != "bf16":
                # quantised caches (random codes, unit-range scales: the timing does not depend on the values)
                bits = {"fp8": 8, "int6": 6, "int4": 4}[a.kv]
                kq = torch.randint(0, 255, (nslots * nb, kvb, nkv, hd * bits // 8), device=dev, dtype=torch.uint8)
                vq = torch.randint(0, 255, (nslots * nb, kvb, nkv, hd * bits // 8), device=dev, dtype=torch.uint8)
                if bits == 8:
                    kq, vq = kq.clamp(max=119), vq.clamp(max=119)               # finite e4m3 codes
                sc = torch.rand(nslots * nb, kvb, nkv, 2 if bits == 8 else 2 * (hd // 32), device=dev) * 0.1
                ms = t.run(lambda: ops.attention(q, proj, kq, vq, slot, kvlen, bt, kvb, nq, nkv, hd, True, nsplit=ns, kv_scale=sc))
                qbytes = rows * a.ctx * nkv * 2 * (hd * bits // 8 + sc.shape[-1] * 2)
                report(f"attn_decode (SIMT, {a.kv} cache) rows{rows} ctx{a.ctx} splits{ns}", ms, qbytes, 4.0 * rows * a.ctx * nq * hd)
                return 0
            ms = t.run(lambda: ops.attention(q, proj, kc, vc, slot, kvlen, bt, kvb, nq, nkv, hd, True, nsplit=ns))
            nbytes = rows * a.ctx * nkv * hd * 2 * 2
            report(f"attn_decode (SIMT) rows{rows} ctx{a.ctx} splits{ns}", ms, nbytes, 4.0 * rows * a.ctx * nq * hd)
            i32 = lambda v: torch.tensor(v, device=dev, dtype=torch.int32)
            # tensor-core kernel: independent streams (one row per segment), then one verify segment of all rows
            segs = (slot, i32(list(range(rows))), i32([1] * rows), 1)
            ms = t.run(lambda: ops.attention(q, proj, kc, vc, slot, kvlen, bt, kvb, nq, nkv, hd, True, nsplit=ns, segs=segs))
            report(f"attn_decode (mma) {rows} streams ctx{a.ctx} splits{ns}", ms, nbytes, 4.0 * rows * a.ctx * nq * hd)
            if rows > 1:
                slot0 = torch.zeros(rows, device=dev, dtype=torch.int32)
                segs = (i32([0]), i32([0]), i32([rows]), rows)
                ms = t.run(lambda: ops.attention(q, proj, kc, vc, slot0, kvlen, bt, kvb, nq, nkv, hd, True, nsplit=ns, segs=segs))
                report(f"attn_decode (mma) verify {rows} rows ctx{a.ctx} splits{ns}", ms, a.ctx * nkv * hd * 2 * 2,
                       4.0 * rows * a.ctx * nq * hd)
        else:
            i32 = lambda v: torch.tensor([v], device=dev, dtype=torch.int32)
            ms = t.run(lambda: ops.attention_prefill(q, proj, kc, vc, i32(0), i32(0), i32(rows), i32(0), bt, kvb, nq,
                                                     nkv, hd, True, rows))
            report(f"attn_prefill ctx{a.ctx}", ms, 2 * a.ctx * nkv * hd * 2, 4.0 * a.ctx * a.ctx / 2 * nq * hd)
    elif a.what == "gdn":
        nk = nv = 16
        dk = dv = 128
        conv_dim = 2 * nk * dk + nv * dv
        rows = a.m
        proj = rnd(rows, conv_dim + nv * dv + 2 * nv)
        conv_w = rnd(conv_dim, 4, scale=0.5)
        rec = rnd(4, nv, dk, dv, scale=0.1, dtype=torch.float32)
        cst = rnd(4, 3, conv_dim)
        A, dtb = rnd(nv, dtype=torch.float32), rnd(nv, dtype=torch.float32)
        i32 = lambda v: torch.tensor(v, device=dev, dtype=torch.int32)
        nseg = min(4, rows)
        per = rows // nseg
        ss, r0, nr = i32(list(range(nseg))), i32([i * per for i in range(nseg)]), i32([per] * nseg)

        def fn():
            qkv = ops.gdn_conv(proj, conv_w, cst, ss, r0, nr, conv_dim, max_rows=per)
            ops.gdn_rec(qkv, proj, rec, cst, A, dtb, ss, r0, nr, nk, nv, dk, dv, 1e-6, commit=True,
                        chunked=per >= 24, max_rows=per)
        ms = t.run(fn)
        report(f"gdn conv+rec rows{rows} segs{nseg}", ms, nseg * nv * dk * dv * 4 * 2, 0.0)
    elif a.what == "moe":
        # routed-expert block of one decode step at the 80B-A3B shapes: 512 experts, top-10, hidden 2048, expert FFN 512
        E, K, H, I = 512, 10, 2048, 512
        rows = a.m
        h = rnd(rows, H)
        w_gu, w_dn = rnd(E, 2 * I, H, scale=0.02), rnd(E, H, I, scale=0.02)
        logits = rnd(rows, E, dtype=torch.float32)
        res = rnd(rows, H)

        def fn():
            ids, wts = ops.moe_route(logits, None, 0, K, 1, 1, 1.0)
            ops.moe_experts(h, ids, wts, w_gu, w_dn, 0, E, None, None, res)
        ms = t.run(fn)
        ids, _ = ops.moe_route(logits, None, 0, K, 1, 1, 1.0)
        distinct = int(ids.unique().numel())
        report(f"moe route+experts rows{rows} (distinct experts {distinct})", ms, distinct * 3 * H * I * 2,
               2.0 * rows * K * 3 * H * I)
        if a.fp4:
            from ..ops.qweight import quantize_experts
            q_gu, q_dn = quantize_experts(w_gu), quantize_experts(w_dn)

            def fn4():
                ids, wts = ops.moe_route(logits, None, 0, K, 1, 1, 1.0)
                ops.moe_experts(h, ids, wts, q_gu, q_dn, 0, E, None, None, res)
            ms4 = t.run(fn4)
            report(f"moe fp4 route+experts rows{rows} (distinct experts {distinct})", ms4,
                   distinct * 3 * H * I * 9 // 16, 2.0 * rows * K * 3 * H * I)


if __name__ == "__main__":
    main()
