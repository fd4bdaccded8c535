"""`python -m ferrite_b200.server`: the serving binary (reference `crates/fe-server/src/main.rs` flags, `scripts/serve.sh`
environment). Binds the port, builds the engine, serves; exits with code 70 when the engine dies so a supervisor
restarts the process."""
from __future__ import annotations

import argparse
import asyncio
import os
import sys

from aiohttp import web

from ..config import PRESETS, EngineConfig, ModelConfig, SiteConfig, scaled


def build_engine(args, tok):
    from .engine_api import MockEngine, SchedulerEngine
    if args.mock or args.engine == "mock":
        return MockEngine(tok, args.served_model_name, max_batch=args.slots, max_len=args.max_model_len)
    if args.engine == "fake":
        # the deterministic CPU step model behind the real batching loop (protocol and load tests without weights)
        from .batch import BatchConfig, BatchEngine, FakeModel
        return BatchEngine(BatchConfig("fake", args.prefill_chunk),
                           lambda: FakeModel(args.slots, args.max_model_len, min(args.prefill_chunk, 2048), vocab=tok.vocab_size
                                             if hasattr(tok, "vocab_size") else 4096), args.served_model_name)
    import torch

    from ..engine.engine import Engine
    from ..engine.scheduler import SchedOptions, Scheduler
    cfg_path = os.path.join(args.model_dir, "config.json") if args.model_dir else ""
    if cfg_path and os.path.exists(cfg_path):
        cfg = ModelConfig.from_hf(cfg_path)
    else:
        cfg = PRESETS[args.preset]()
        if args.layers:
            cfg = scaled(cfg, args.layers)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    kind = getattr(args, "drafter", "none")
    if kind != "none":
        # the drafters read hidden rows of the target: the MTP head the last layer's, the block drafter three evenly
        # spaced ones (the preset's own tap list when it has one)
        if kind == "mtp":
            cfg.tap_layers = [cfg.n_layers - 1]
        elif not cfg.tap_layers:
            cfg.tap_layers = sorted({max(0, cfg.n_layers * (i + 1) // 4 - 1) for i in range(3)})
    ecfg = EngineConfig.from_env(n_slots=args.slots, max_ctx=args.max_model_len, prefill_chunk=args.prefill_chunk,
                                 weight_dtype=args.weights)
    weights = None
    if args.model_dir and any(f.endswith(".safetensors") for f in os.listdir(args.model_dir)):
        from ..formats.loader import load_model_weights
        weights = load_model_weights(args.model_dir, cfg)
    tp = None
    if world > 1:
        # launched with torch.distributed.run: every rank builds its shard; rank 0 schedules and serves, the others
        # replay its engine calls (leader / follower control, `engine/follow.py`)
        import torch.distributed as dist

        from ..parallel.tp import TensorParallel
        local = int(os.environ.get("LOCAL_RANK", "0"))
        on_gpu = torch.cuda.is_available() and args.device != "cpu"
        if on_gpu:
            torch.cuda.set_device(local)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if on_gpu else "gloo",
                                **({"device_id": torch.device("cuda", local)} if on_gpu else {}))
        tp = TensorParallel(dist.group.WORLD, f"cuda:{local}" if on_gpu else "cpu")
        tp.selftest()                      # refuse to serve over a peer path that corrupts data
        args.device = f"cuda:{local}" if on_gpu else "cpu"
    if args.model_dir and weights is None:
        ggufs = sorted(f for f in os.listdir(args.model_dir) if f.endswith(".gguf"))
        if ggufs:
            from ..formats import gguf as G
            from ..formats.gguf_model import config_from_gguf, load_gguf_weights
            path = os.path.join(args.model_dir, ggufs[0])
            g = G.Gguf(path)
            cfg = config_from_gguf(g, cfg)
            g.close()
            weights = load_gguf_weights(path, cfg)
    if args.engine == "ferrite-batch":
        # the small engine: plain continuous batching over the step-model surface (no speculation, no parking)
        from .batch import BatchConfig, BatchEngine, EngineStepModel
        return BatchEngine(BatchConfig("ferrite-batch", args.prefill_chunk),
                           lambda: EngineStepModel(Engine(cfg, weights, ecfg, device=args.device or None, seed=0)),
                           args.served_model_name)
    eng = Engine(cfg, weights, ecfg, device=args.device or None, seed=0, tp=tp)
    opts = SchedOptions.from_env()
    drafter = None
    if kind != "none":
        # speculative decoding with a draft model (reference: the drafter `factory`, `crates/fe-dflash/src/lib.rs:1381`,
        # and the MTP head of the checkpoint). Under tensor parallelism every rank builds the drafter over its shard of
        # the draft engine and the leader mirrors the drafter's calls (reference: DFlash2 at TP2)
        if kind == "mtp":
            from ..models.mtp import MtpDrafter
            drafter = MtpDrafter(eng, n_slots=args.slots, max_ctx=args.max_model_len, depth=max(1, min(opts.spec or 4, 8)))
        else:
            from ..models.drafter import BlockDrafter, drafter_config_for
            # the drafter's own context is bounded (window / ring) once the served context is longer than the ring
            dw = int(getattr(args, "draft_window", 2048))
            win = dw if args.max_model_len > 2 * dw else 0
            drafter = BlockDrafter(drafter_config_for(cfg), target_hidden=cfg.hidden, n_taps=len(cfg.tap_layers),
                                   n_slots=args.slots, max_ctx=args.max_model_len, device=str(eng.device), block=16,
                                   window=win, ring=2 * win, weight_dtype=getattr(args, "draft_weights", "bf16"), tp=tp)
        if opts.spec == 0:
            opts.spec = 4 if kind == "mtp" else 8
    if tp is not None:
        from ..engine.follow import Leader, follow
        if tp.rank != 0:
            follow(eng, tp, drafter)
            raise SystemExit(0)
        eng = Leader(eng, tp)
        if drafter is not None:
            drafter = eng.attach_drafter(drafter)
    return SchedulerEngine(Scheduler(eng, opts, drafter=drafter), args.served_model_name)


def main(argv=None) -> int:
    site = SiteConfig.from_env()
    ap = argparse.ArgumentParser(prog="ferrite-server")
    ap.add_argument("--model-dir", default=os.environ.get("FERRITE_MODEL_DIR", ""))
    ap.add_argument("--host", default=site.host)
    ap.add_argument("--port", type=int, default=site.port)
    ap.add_argument("--served-model-name", default=site.served_model_name)
    ap.add_argument("--engine", default="ferrite", choices=["ferrite", "ferrite-batch", "fake", "mock"])
    ap.add_argument("--preset", default="tiny", choices=sorted(PRESETS))
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--weights", default=os.environ.get("FERRITE_WEIGHTS", "bf16"))
    ap.add_argument("--device", default="")
    ap.add_argument("--slots", type=int, default=int(os.environ.get("FERRITE_SLOTS", "4")))
    ap.add_argument("--prefill-chunk", type=int, default=int(os.environ.get("FERRITE_CHUNK", "2048")))
    ap.add_argument("--max-concurrent", type=int, default=site.max_concurrent)
    ap.add_argument("--max-model-len", type=int, default=int(os.environ.get("FERRITE_CTX", "8192")))
    ap.add_argument("--profile", default=os.environ.get("FERRITE_PROFILE", "default"))
    ap.add_argument("--mock", action="store_true")
    ap.add_argument("--drafter", default=os.environ.get("FERRITE_DRAFTER", "none"), choices=["none", "block", "mtp"],
                    help="draft model for speculative decoding (FE_SPEC sets the depth, FE_TREE the rows of a verify tree)")
    ap.add_argument("--draft-window", type=int, default=int(os.environ.get("FERRITE_DRAFT_WINDOW", "2048")),
                    help="block drafter: tokens of its own context (its cache ring holds twice as many); 0 = the whole context")
    ap.add_argument("--draft-weights", default=os.environ.get("FERRITE_DRAFT_WEIGHTS", "bf16"),
                    help="block drafter: its weight format (bf16, nvfp4, ...)")
    args = ap.parse_args(argv)

    from .app import AppState, make_app
    from .profiles import GenDefaults
    from .template import ChatTemplate
    from .tokenizer import load_tokenizer

    vocab = PRESETS[args.preset]().vocab
    tok = load_tokenizer(args.model_dir or None, vocab)
    engine_box = {}

    def factory():
        engine_box["e"] = build_engine(args, tok)
        return AppState(engine_box["e"], tok, ChatTemplate.from_dir(args.model_dir or None),
                        GenDefaults.from_dir(args.model_dir or None, args.profile), args.served_model_name,
                        args.max_concurrent)

    if int(os.environ.get("RANK", "0")) > 0:          # tensor-parallel follower: no HTTP side, replay until told to stop
        build_engine(args, tok)
        return 0

    app = make_app(factory)

    async def watch(app):
        async def loop():
            while True:
                await asyncio.sleep(1.0)
                e = engine_box.get("e")
                if e is not None and e.dead():
                    print(f"engine dead: {e.dead()}", file=sys.stderr, flush=True)
                    os._exit(70)
        app["watch"] = asyncio.create_task(loop())

    app.on_startup.append(watch)
    web.run_app(app, host=args.host, port=args.port, print=lambda *a: print(*a, file=sys.stderr))
    return 0


if __name__ == "__main__":
    sys.exit(main())
