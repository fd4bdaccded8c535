"""Multi-head latent attention through the engine on CPU (absorbed form over the paged latent cache) against the
token-by-token oracle (explicit key/value up-projection), with the grouped-sigmoid MoE and leading dense layers of the
671B-class family in a tiny configuration."""
import torch

from ferrite_b200.config import EngineConfig, tiny_mla
from ferrite_b200.engine.engine import Engine
from ferrite_b200.engine.executor import Segment
from ferrite_b200.models.ref import RefModel
from ferrite_b200.models.weights import init_weights


def test_mla_engine_matches_oracle():
    cfg = tiny_mla()
    w = init_weights(cfg, seed=0)
    ref = RefModel(cfg, w)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=torch.Generator().manual_seed(1)).tolist()
    want = ref.forward(prompt, ref.new_state())
    eng = Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=128), device="cpu")
    got, _, _ = eng.forward([Segment(1, 0, prompt[:30], "all")])                      # prompt rows, causal
    tail = [eng.forward([Segment(1, 30 + i, [prompt[30 + i]], "last")])[0].clone() for i in range(10)]   # decode rows
    got = torch.cat([got] + tail)
    assert torch.allclose(got, want, atol=3e-5, rtol=1e-4)


def test_mla_cache_is_one_latent_row_per_token():
    cfg = tiny_mla(moe=False)
    eng = Engine(cfg, init_weights(cfg, seed=0), EngineConfig(n_slots=1, max_ctx=128), device="cpu")
    k = eng.ex.k_cache[0]
    assert k.shape[-1] == cfg.kv_lora + cfg.rope_head_dim and k.shape[-2] == 1
    assert eng.ex.v_cache[0].numel() == 0
