"""`BatchEngine` over the deterministic fake model and over the real CPU engine, through the HTTP surface: usage
accounting, prompt-cache hits, slot release, more streams than slots (reference `crates/fe-server/tests/e2e_batch.rs`)."""
import asyncio
import json
import threading

import torch
from aiohttp.test_utils import TestClient, TestServer

from ferrite_b200.engine.sampler import Sampling
from ferrite_b200.server.app import AppState, make_app
from ferrite_b200.server.batch import BatchConfig, BatchEngine, EngineStepModel, FakeModel, fake_reference
from ferrite_b200.server.engine_api import GenRequest
from ferrite_b200.server.profiles import GenDefaults
from ferrite_b200.server.template import ChatTemplate
from ferrite_b200.server.tokenizer import ByteTokenizer


def _collect(engine, ids, sampling):
    out, fin, done = [], {}, threading.Event()

    def sink(ev):
        if ev.kind == "tokens":
            out.extend(ev.tokens)
        else:
            fin.update(kind=ev.kind, reason=ev.reason, timings=ev.timings, message=ev.message)
            done.set()
    engine.submit(GenRequest(list(ids), sampling), sink)
    return out, fin, done


def test_fake_model_streams_equal_the_solo_reference_with_more_streams_than_slots():
    models = []

    def factory():
        models.append(FakeModel(n_slots=4, max_rows=64))
        return models[0]
    eng = BatchEngine(BatchConfig("fake", prefill_chunk=16), factory, "fake-model")
    assert eng.info().max_batch_size == 4
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(2, 256, (int(n),), generator=g).tolist() for n in (5, 40, 90, 17, 33, 64)]   # 6 streams, 4 slots
    runs = [_collect(eng, p, Sampling(max_tokens=60, stop_ids=[1])) for p in prompts]
    for (out, fin, done), p in zip(runs, prompts):
        assert done.wait(20)
        want, reason = fake_reference(p, 60, 256, 1, 97)
        assert out == want and fin["reason"] == reason
        assert fin["timings"]["prompt_n"] == len(p) and fin["timings"]["predicted_n"] == len(out)
    # every forward stayed inside the row budget, and prompts were cut into chunks
    assert all(rows <= 64 for rows, _ in models[0].log)
    assert eng.load() == {"running": 0, "queued": 0}
    # second turn on the same conversation: the slot's history is a prefix of the new prompt -> cached tokens
    turn1 = prompts[2]
    out1 = runs[2][0]
    turn2 = turn1 + out1 + [7, 8, 9]
    out, fin, done = _collect(eng, turn2, Sampling(max_tokens=10, stop_ids=[1]))
    assert done.wait(20)
    assert fin["timings"]["cache_n"] >= len(turn1) and out == fake_reference(turn2, 10, 256, 1, 97)[0]
    # sampled requests go through the host sampler: the fake's logits are a point mass, so the text is the same
    out, fin, done = _collect(eng, prompts[0], Sampling(temperature=0.8, top_p=0.9, seed=1, max_tokens=12, stop_ids=[1]))
    assert done.wait(20) and out == fake_reference(prompts[0], 12, 256, 1, 97)[0]
    eng.shutdown()


def test_real_cpu_engine_behind_the_step_model_surface_and_http():
    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.models.weights import init_weights
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0)

    def model():
        return EngineStepModel(Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=256, prefill_chunk=32), device="cpu"))

    async def go():
        tok = ByteTokenizer(cfg.vocab)
        app = make_app(lambda: AppState(BatchEngine(BatchConfig("ferrite-batch"), model, "tiny"), tok, ChatTemplate(), GenDefaults(), "tiny"))
        c = TestClient(TestServer(app))
        await c.start_server()
        h = await (await c.get("/health")).json()
        assert h["engine"] == "ferrite-batch" and h["max_batch_size"] == 2
        body = {"model": "tiny", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 8, "temperature": 0}
        rs = await asyncio.gather(*[c.post("/v1/chat/completions", json=body) for _ in range(3)])    # 3 requests, 2 slots
        js = [await r.json() for r in rs]
        assert all(j["usage"]["completion_tokens"] <= 8 and j["usage"]["prompt_tokens"] > 5 for j in js)
        assert js[0]["choices"][0]["message"]["content"] == js[1]["choices"][0]["message"]["content"]
        # the plain engine gives the same greedy tokens
        ids = tok.encode(ChatTemplate().render(body["messages"], None, True))
        want = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=256), device="cpu").generate(ids, js[0]["usage"]["completion_tokens"])
        assert tok.decode(want).strip() == js[0]["choices"][0]["message"]["content"].strip()
        h = await (await c.get("/health")).json()
        assert h["running"] == 0 and h["queued"] == 0
        await c.close()
    asyncio.run(go())
