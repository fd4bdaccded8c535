"""Typed configuration: model shapes, engine options and operator-tier site settings.

The reference keeps three tiers (operator env `FERRITE_*`, server flags, engine env knobs `FE_*`;
`scripts/serve.sh:14-43`, `crates/fe-model/src/config.rs:6-107`, `crates/fe-model/src/sched.rs:14-48`).
Here one set of dataclasses is filled from file + env + CLI, and model dimensions are run-time values
instead of recompiled kernel crates (`kernels/k-core/src/dims.rs`).
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import List, Optional


@dataclass
class ModelConfig:
    """Dense hybrid decoder (Gated DeltaNet + gated GQA attention), optionally with MoE FFN or MLA attention."""

    name: str = "tiny-hybrid"
    hidden: int = 256
    inter: int = 768
    n_layers: int = 4
    # layer i is full attention when (i % full_attn_every) == full_attn_every - 1, else Gated DeltaNet
    full_attn_every: int = 4
    head_dim: int = 64
    n_q: int = 4
    n_kv: int = 2
    rotary_dim: int = 64
    rope_theta: float = 1e6
    attn_gate: bool = True          # q_proj carries a per-head sigmoid output gate
    lin_k_heads: int = 4
    lin_v_heads: int = 4
    lin_dk: int = 64
    lin_dv: int = 64
    conv_k: int = 4
    eps: float = 1e-6
    vocab: int = 4096
    tie_embeddings: bool = True
    eos: int = 0
    # ---- MoE FFN (0 experts = dense SwiGLU) ----
    n_experts: int = 0
    top_k: int = 0
    expert_inter: int = 0
    n_shared: int = 0
    router: str = "softmax"         # "softmax" (top-k, renormalised) | "sigmoid_group" (grouped top-k with bias)
    n_groups: int = 1
    topk_groups: int = 1
    route_scale: float = 1.0
    first_dense: int = 0            # leading layers that keep a dense FFN
    dense_inter: int = 0
    # ---- MLA attention (kv_lora > 0 switches every layer to MLA; no GDN layers) ----
    kv_lora: int = 0
    q_lora: int = 0
    rope_head_dim: int = 0
    nope_head_dim: int = 0
    v_head_dim: int = 0
    # ---- drafter taps ----
    tap_layers: List[int] = field(default_factory=list)

    # derived -----------------------------------------------------------------------------------
    def is_attn(self, i: int) -> bool:
        if self.kv_lora > 0:
            return True
        return (i % self.full_attn_every) == self.full_attn_every - 1

    @property
    def layer_kinds(self) -> List[str]:
        if self.kv_lora > 0:
            return ["mla"] * self.n_layers
        return ["attn" if self.is_attn(i) else "gdn" for i in range(self.n_layers)]

    @property
    def n_attn(self) -> int:
        return sum(1 for k in self.layer_kinds if k != "gdn")

    @property
    def n_gdn(self) -> int:
        return self.n_layers - self.n_attn

    @property
    def conv_dim(self) -> int:
        return 2 * self.lin_k_heads * self.lin_dk + self.lin_v_heads * self.lin_dv

    @property
    def gdn_in_dim(self) -> int:
        """Rows of the fused GDN input projection: qkv | z | b | a."""
        return self.conv_dim + self.lin_v_heads * self.lin_dv + 2 * self.lin_v_heads

    @property
    def attn_q_dim(self) -> int:
        return self.n_q * self.head_dim * (2 if self.attn_gate else 1)

    @property
    def attn_in_dim(self) -> int:
        """Rows of the fused attention input projection: per head [q|gate], then k, then v."""
        return self.attn_q_dim + 2 * self.n_kv * self.head_dim

    def is_moe(self, i: int) -> bool:
        return self.n_experts > 0 and i >= self.first_dense

    def param_count(self) -> int:
        h = self.hidden
        n = self.vocab * h * (1 if self.tie_embeddings else 2)
        for i, kind in enumerate(self.layer_kinds):
            if kind == "gdn":
                n += h * self.gdn_in_dim + self.lin_v_heads * self.lin_dv * h + self.conv_dim * self.conv_k
            elif kind == "attn":
                n += h * self.attn_in_dim + self.n_q * self.head_dim * h
            else:
                qd = self.n_q * (self.nope_head_dim + self.rope_head_dim)
                n += h * self.q_lora + self.q_lora * qd + h * (self.kv_lora + self.rope_head_dim)
                n += self.kv_lora * self.n_q * (self.nope_head_dim + self.v_head_dim) + self.n_q * self.v_head_dim * h
            if self.is_moe(i):
                n += (self.n_experts + self.n_shared) * 3 * h * self.expert_inter + self.n_experts * h
            else:
                n += 3 * h * (self.dense_inter if (self.n_experts > 0 and self.dense_inter) else self.inter)
        return n

    def shard(self, world: int) -> "ModelConfig":
        """Per-rank shapes of a `world`-way tensor-parallel split (reference `Config::shard`,
        `crates/fe-model/src/config.rs:80`): whole heads and FFN columns per rank; KV heads are
        replicated when there are fewer of them than ranks."""
        c = dataclasses.replace(self)
        if world == 1:
            return c
        assert self.n_q % world == 0 and self.inter % world == 0
        c.n_q = self.n_q // world
        c.n_kv = max(1, self.n_kv // world)
        if self.kv_lora == 0:
            assert self.lin_k_heads % world == 0 and self.lin_v_heads % world == 0
            c.lin_k_heads = self.lin_k_heads // world
            c.lin_v_heads = self.lin_v_heads // world
        c.inter = self.inter // world
        if self.dense_inter:
            c.dense_inter = self.dense_inter // world
        return c

    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self), indent=1)

    @staticmethod
    def from_hf(path: str | os.PathLike) -> "ModelConfig":
        """Read a Hugging Face `config.json` (the `text_config` block when present), the way the
        reference does in `crates/fe-model/src/config.rs:44-78`."""
        v = json.loads(Path(path).read_text())
        t = v.get("text_config", v)
        rp = t.get("rope_parameters") or {}
        head_dim = int(t["head_dim"])
        prf = float(rp.get("partial_rotary_factor", t.get("partial_rotary_factor", 0.25)))
        lt = t.get("layer_types")
        every = 4
        if lt:
            idx = [i for i, x in enumerate(lt) if x == "full_attention"]
            every = (idx[0] + 1) if idx else len(lt) + 1
        return ModelConfig(
            name=str(v.get("model_type", "hf")),
            hidden=int(t["hidden_size"]), inter=int(t["intermediate_size"]), n_layers=int(t["num_hidden_layers"]),
            full_attn_every=every, head_dim=head_dim, n_q=int(t["num_attention_heads"]),
            n_kv=int(t["num_key_value_heads"]), rotary_dim=int(head_dim * prf),
            rope_theta=float(rp.get("rope_theta", t.get("rope_theta", 1e7))),
            lin_k_heads=int(t.get("linear_num_key_heads", 16)), lin_v_heads=int(t.get("linear_num_value_heads", 16)),
            lin_dk=int(t.get("linear_key_head_dim", 128)), lin_dv=int(t.get("linear_value_head_dim", 128)),
            conv_k=int(t.get("linear_conv_kernel_dim", 4)), eps=float(t.get("rms_norm_eps", 1e-6)),
            vocab=int(t["vocab_size"]), tie_embeddings=bool(v.get("tie_word_embeddings", False)),
            eos=int(t.get("eos_token_id", 0) if not isinstance(t.get("eos_token_id"), list) else t["eos_token_id"][0]),
        )


# ---- presets: the five benchmark configurations ----------------------------------------------------

def tiny_hybrid() -> ModelConfig:
    """4 layers (3 GDN + 1 GQA), hidden 256, vocab 4096, tied embeddings: the fp32 CPU plumbing model and oracle."""
    return ModelConfig()


def hybrid_27b() -> ModelConfig:
    """27B-class dense hybrid: 64 layers 3:1 GDN:GQA, hidden 5120, FFN 17408, vocab 151936."""
    return ModelConfig(
        name="hybrid-27b", hidden=5120, inter=17408, n_layers=64, full_attn_every=4, head_dim=256, n_q=24, n_kv=4,
        rotary_dim=64, rope_theta=1e7, lin_k_heads=16, lin_v_heads=16, lin_dk=128, lin_dv=128, vocab=151936,
        tie_embeddings=False, tap_layers=[15, 31, 47],
    )


def drafter_block() -> ModelConfig:
    """5-layer block drafter conditioned on tapped target hidden states (reference `crates/fe-dflash/src/lib.rs:1-66`)."""
    return ModelConfig(
        name="block-drafter", hidden=5120, inter=17408, n_layers=5, full_attn_every=1, head_dim=128, n_q=32, n_kv=8,
        rotary_dim=128, rope_theta=1e7, attn_gate=False, vocab=151936, tie_embeddings=False,
    )


def moe_80b() -> ModelConfig:
    """80B-A3B-class hybrid MoE: 48 layers 3:1, hidden 2048, 512 experts (FFN 512) top-10 + 1 shared."""
    return ModelConfig(
        name="moe-80b-a3b", hidden=2048, inter=512, n_layers=48, full_attn_every=4, head_dim=256, n_q=16, n_kv=2,
        rotary_dim=64, rope_theta=1e7, lin_k_heads=16, lin_v_heads=32, lin_dk=128, lin_dv=128, vocab=151936,
        tie_embeddings=False, n_experts=512, top_k=10, expert_inter=512, n_shared=1, router="softmax",
    )


def mla_671b() -> ModelConfig:
    """671B-class MLA MoE: 61 layers (3 dense), hidden 7168, 256 experts (FFN 2048) sigmoid top-8 in 4 of 8 groups."""
    return ModelConfig(
        name="mla-671b", hidden=7168, inter=18432, n_layers=61, head_dim=192, n_q=128, n_kv=128, rotary_dim=64,
        rope_theta=1e4, attn_gate=False, vocab=129280, tie_embeddings=False, n_experts=256, top_k=8,
        expert_inter=2048, n_shared=1, router="sigmoid_group", n_groups=8, topk_groups=4, route_scale=2.5,
        first_dense=3, dense_inter=18432, kv_lora=512, q_lora=1536, rope_head_dim=64, nope_head_dim=128,
        v_head_dim=128,
    )


def tiny_mla(moe: bool = True) -> ModelConfig:
    """3-layer MLA model (latent 64 + rope 64) with the grouped-sigmoid MoE and a leading dense layer: the plumbing
    model of the 671B-class family."""
    kw = dict(n_experts=16, top_k=4, expert_inter=64, n_shared=1, router="sigmoid_group", n_groups=4, topk_groups=2,
              route_scale=2.5, first_dense=1, dense_inter=512) if moe else {}
    return ModelConfig(name="tiny-mla", hidden=256, inter=512, n_layers=3, head_dim=96, n_q=4, n_kv=4, rotary_dim=64,
                       vocab=1024, tie_embeddings=True, kv_lora=64, q_lora=128, rope_head_dim=64, nope_head_dim=32,
                       v_head_dim=32, **kw)


PRESETS = {
    "tiny": tiny_hybrid, "tiny-mla": tiny_mla, "27b": hybrid_27b, "drafter": drafter_block, "moe80b": moe_80b, "mla671b": mla_671b,
}


def scaled(cfg: ModelConfig, n_layers: int) -> ModelConfig:
    """Same architecture with fewer layers (for tests that need real widths but little memory)."""
    c = dataclasses.replace(cfg)
    c.n_layers = n_layers
    c.tap_layers = [t for t in cfg.tap_layers if t < n_layers]
    return c


@dataclass
class EngineConfig:
    """Engine-tier options (reference `LoadOpts::from_env` `crates/fe-model/src/model.rs:585-597`,
    `SchedOptions` `crates/fe-model/src/sched.rs:14-48`)."""

    n_slots: int = 4
    max_ctx: int = 4096
    kv_block: int = 64                 # tokens per KV page
    kv_dtype: str = "bf16"             # "bf16" | "fp8"
    weight_dtype: str = "bf16"         # "bf16" | "nvfp4" | "nvfp4-w4a4" | "nvfp4-a16" | "fp8-block" (e4m3, 128 x 128 blocks) | "exl3[-bits]"
    prefill_chunk: int = 2048          # rows per prompt forward (reference FERRITE_CHUNK)
    prompt_align: int = 32             # chunk cuts land on this grid (reference PROMPT_ALIGN)
    max_step_rows: int = 4096
    decode_rows_max: int = 64          # rows routed to the small-M (GEMV) kernels
    attn_splits: int = 0               # 0 = pick from context length
    use_graphs: bool = True
    fused_layers: Optional[bool] = None   # plain decode rows: one persistent kernel per layer (None = when tensor parallel)
    # "bf16" | "fp8" (e4m3, one scale per (token, kv head)) | "int6" | "int4" (integer codes, one scale per 32 elements);
    # "fp8h" / "int6h" / "int4h": the same with keys stored in a Walsh-Hadamard rotated basis
    kv_dtype: str = "bf16"
    seq_parallel: bool = True          # TP prompts: row-sharded residual stream, all-gather/reduce-scatter fused into the GEMMs
    graph_max: int = 128               # LRU size of the CUDA-graph cache (reference GRAPH_MAX)
    spec_depth: int = 0
    park_gb: float = 0.0
    park_host: bool = False
    finite_check: bool = True
    step_timeout_s: float = 120.0
    seed: int = 0

    @staticmethod
    def from_env(**over) -> "EngineConfig":
        e = os.environ
        c = EngineConfig()
        def geti(name, cur):
            return int(e[name]) if name in e and e[name] != "" else cur
        c.n_slots = geti("FERRITE_SLOTS", c.n_slots)
        c.max_ctx = geti("FERRITE_CTX", c.max_ctx)
        c.prefill_chunk = geti("FERRITE_CHUNK", c.prefill_chunk)
        c.spec_depth = geti("FE_SPEC", c.spec_depth)
        c.graph_max = geti("FE_GRAPH_MAX", c.graph_max)
        if "FE_KVQ" in e:
            c.kv_dtype = "fp8" if e["FE_KVQ"] not in ("", "0") else "bf16"
        if "FERRITE_WEIGHTS" in e:
            c.weight_dtype = e["FERRITE_WEIGHTS"]
        if "FE_PARK_GB" in e:
            c.park_gb = float(e["FE_PARK_GB"])
        c.park_host = e.get("FE_PARK_HOST", "0") not in ("", "0")
        c.use_graphs = e.get("FE_NO_GRAPHS", "0") in ("", "0")
        c.seq_parallel = e.get("FE_NO_SEQ_PARALLEL", "0") in ("", "0")
        c.kv_dtype = e.get("FE_KV_DTYPE", c.kv_dtype)
        c.step_timeout_s = float(e.get("FE_STEP_TIMEOUT", c.step_timeout_s))
        for k, v in over.items():
            if v is not None:
                setattr(c, k, v)
        return c


@dataclass
class SiteConfig:
    """Operator tier: the `FERRITE_*` names of `tools/site.sh:1-40` / `crates/fe-site`."""

    models_dir: str = ""
    state_dir: str = ""
    host: str = "127.0.0.1"
    port: int = 8080
    served_model_name: str = "ferrite"
    max_concurrent: int = 16

    @staticmethod
    def from_env() -> "SiteConfig":
        e = os.environ
        return SiteConfig(
            models_dir=e.get("FERRITE_MODELS", ""), state_dir=e.get("FERRITE_STATE", ""),
            host=e.get("FERRITE_HOST", "127.0.0.1"), port=int(e.get("FERRITE_PORT", "8080")),
            served_model_name=e.get("FERRITE_NAME", "ferrite"),
            max_concurrent=int(e.get("FERRITE_MAX_CONCURRENT", "16")),
        )
