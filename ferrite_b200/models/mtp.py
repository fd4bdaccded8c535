"""Multi-token-prediction (MTP) head as a chain drafter.

The head is one full-attention layer that runs over rows built from two halves: the embedding of the token AFTER a
position, and the target model's final hidden state AT that position (reference `MtpW`,
`crates/fe-model/src/model.rs:428-439`: `fc` over [norm(embed(next token)) | norm(final hidden)], one layer, a norm,
and the target's own head; `mtp_forward`, `crates/fe-model/src/model.rs:2617`, with rows whose hidden half comes
either from the target (`MtpSrc::Tap`) or from the head's own previous output (`MtpSrc::Out`) for chained drafts).

Here the layer, its KV cache and its position bookkeeping are an `Engine` over a one-layer attention-only
`ModelConfig` that shares the target's embedding table and output head (same tensors, no copy); the engine is asked
to take its input rows from the caller (`Executor.input_rows`) instead of embedding tokens. A row of the head at
position p holds the target hidden of position p and the token of position p + 1 and predicts the token of p + 2:

  absorb(tokens t_0..t_{n-1} at pos0..)   rows (pos0-1+j): hidden H_j, token t_j   (H_0 = hidden kept from last time)
  draft(last_token at pos, n)             row pos-1: kept hidden + last_token -> draft 1; then the head's own output
                                          and draft j feed row pos-1+j -> draft j+1 (chain, one row per forward)

Draft rows are run without committing, so the accepted ones are recomputed by the next `absorb` from the target's
hidden states, as the reference does ("MTP absorb").
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Sequence

import torch

from ..config import EngineConfig, ModelConfig
from ..engine.engine import Engine
from ..engine.executor import Segment
from ..engine.scheduler import Drafter
from .weights import init_weights


def mtp_config(target: ModelConfig) -> ModelConfig:
    """One full-attention layer with the target's widths (its attention geometry, dense FFN, vocabulary)."""
    return ModelConfig(
        name=target.name + "-mtp", hidden=target.hidden, inter=target.inter or target.dense_inter or 4 * target.hidden,
        n_layers=1, full_attn_every=1, head_dim=target.head_dim, n_q=target.n_q, n_kv=target.n_kv,
        rotary_dim=target.rotary_dim, rope_theta=target.rope_theta, attn_gate=target.attn_gate, vocab=target.vocab,
        tie_embeddings=target.tie_embeddings, eps=target.eps)


class MtpDrafter(Drafter):
    """Chain drafter over the target's last-layer hidden rows. The target must tap its last layer
    (`cfg.tap_layers` ends with `n_layers - 1`); `taps[-1]` is read as the hidden source."""

    def __init__(self, target: Engine, n_slots: int, max_ctx: int, seed: int = 1, weights=None, depth: int = 4):
        tcfg = target.full_cfg
        assert tcfg.tap_layers and tcfg.tap_layers[-1] == tcfg.n_layers - 1, "the target must tap its last layer"
        self.target = target
        self.depth = depth
        cfg = mtp_config(tcfg)
        dev, dt = target.device, target.dtype
        if weights is None:
            weights = init_weights(dataclasses.replace(cfg, vocab=8), seed=seed, dtype=dt, device=dev)
            g = torch.Generator().manual_seed(seed + 5)
            weights["mtp.fc"] = (torch.randn(cfg.hidden, 2 * cfg.hidden, generator=g) * 0.02).to(dev, dt)
            weights["mtp.pre_e"] = torch.zeros(cfg.hidden, device=dev, dtype=dt)
            weights["mtp.pre_h"] = torch.zeros(cfg.hidden, device=dev, dtype=dt)
        weights = dict(weights)
        tw = target.ex.w
        tp = getattr(target, "tp", None)
        sharded = tp is not None and tp.world > 1
        weights["embed"] = tw["embed"]                       # shared with the target: the same storage (replicated)
        if not cfg.tie_embeddings and not sharded:
            weights["lm_head"] = tw["lm_head"]
        self.fc = weights.pop("mtp.fc")
        self.pre_e = weights.pop("mtp.pre_e")
        self.pre_h = weights.pop("mtp.pre_h")
        self.tnorm = tw["final_norm"]
        # under tensor parallelism the head's own layer is cut like the target's layers (every rank builds it from the same
        # full weights); the target's output matrix is already this rank's vocabulary rows, so it goes in after the cut
        self.eng = Engine(cfg, weights, EngineConfig(n_slots=n_slots, max_ctx=max_ctx, use_graphs=False), device=str(dev),
                          seed=seed, tp=tp if sharded else None)
        if not cfg.tie_embeddings and sharded:
            self.eng.ex.w["lm_head"] = tw["lm_head"]
        self.eng.ex.input_rows = True
        self.cfg = cfg
        self.base: List[Optional[int]] = [None] * n_slots    # target position of the head's cache row 0
        self.kept: List[Optional[tuple]] = [None] * n_slots  # (position, target hidden row) awaiting its next token
        self.gen = [0] * n_slots                             # bumped when a slot's cache starts over: dates window snapshots

    # ---- the head's input rows -------------------------------------------------------------------------
    def _rows(self, tokens: Sequence[int], hidden: torch.Tensor, src_norm: torch.Tensor) -> torch.Tensor:
        """fc([norm(embed(token)) | norm(norm_src(hidden))]) for n rows."""
        ops, eps = self.eng.ops, self.cfg.eps
        ids = torch.tensor(list(tokens), dtype=torch.int32, device=self.eng.device)
        e = ops.rmsnorm(ops.embed(self.eng.ex.w["embed"], ids), self.pre_e, eps)[0]
        h = ops.rmsnorm(hidden.to(self.eng.device, self.eng.dtype).contiguous(), src_norm, eps)[0]
        h = ops.rmsnorm(h, self.pre_h, eps)[0]
        return ops.linear(torch.cat([e, h], -1).contiguous(), self.fc)

    def _forward(self, slot: int, pos: int, rows: torch.Tensor, commit: bool, want: str):
        n = rows.shape[0]
        if self.base[slot] is None:
            self.base[slot] = pos
        seg = Segment(slot, pos - self.base[slot], [0] * n, want)
        return self.eng.forward([seg], commit=commit, greedy=True, x_add=rows)

    # ---- Drafter interface --------------------------------------------------------------------------
    def reset(self, slot: int) -> None:
        self.eng.reset_slot(slot)
        self.base[slot] = None
        self.kept[slot] = None
        self.gen[slot] += 1

    def absorb(self, slot: int, tokens: Sequence[int], pos0: int, taps) -> None:
        n = len(tokens)
        if n == 0 or not taps:
            return
        hid = taps[-1][:n]
        kept = self.kept[slot]
        if kept is not None and kept[0] == pos0 - 1:
            hs, toks, p = torch.cat([kept[1], hid[:n - 1]], 0), list(tokens), pos0 - 1
        else:
            if kept is not None or (self.base[slot] is not None):
                self.reset(slot)                             # a gap in the positions: start the head's cache over
            hs, toks, p = hid[:n - 1], list(tokens[1:]), pos0
        if toks:
            self._forward(slot, p, self._rows(toks, hs, self.tnorm), commit=True, want="none")
        self.kept[slot] = (pos0 + n - 1, hid[n - 1:n].clone())

    def draft(self, slot: int, last_token: int, pos: int, taps, n: int) -> List[int]:
        kept = self.kept[slot]
        n = min(n, self.depth)
        if n <= 0 or kept is None or kept[0] != pos - 1:
            return []
        out: List[int] = []
        hidden, norm, tok = kept[1], self.tnorm, last_token
        for j in range(n):
            rows = self._rows([tok], hidden, norm)
            _, picks, _ = self._forward(slot, pos - 1 + j, rows, commit=False, want="last")
            tok = int(picks[0][0])
            out.append(tok)
            hidden, norm = self.eng.ex.last_hidden[-1:].clone(), self.eng.ex.w["final_norm"]
        return out

    def draft_many(self, reqs, taps) -> List[List[int]]:
        """The chains of several requests, one head pass per depth for all of them (reqs[i] = (slot, last_token, pos, n))."""
        out: List[List[int]] = [[] for _ in reqs]
        live = []
        for i, (slot, tok, pos, n) in enumerate(reqs):
            kept = self.kept[slot]
            n = min(n, self.depth)
            if n > 0 and kept is not None and kept[0] == pos - 1:
                live.append({"i": i, "slot": slot, "pos": pos, "n": n, "hidden": kept[1], "tok": int(tok)})
        if len(live) <= 1:
            for x in live:
                out[x["i"]] = self.draft(x["slot"], x["tok"], x["pos"], taps, x["n"])
            return out
        norm = self.tnorm
        for j in range(max(x["n"] for x in live)):
            act = [x for x in live if j < x["n"]]
            rows = self._rows([x["tok"] for x in act], torch.cat([x["hidden"] for x in act], 0), norm)
            segs = []
            for x in act:
                if self.base[x["slot"]] is None:
                    self.base[x["slot"]] = x["pos"] - 1
                segs.append(Segment(x["slot"], x["pos"] - 1 + j - self.base[x["slot"]], [0], "last"))
            _, picks, _ = self.eng.forward(segs, commit=False, greedy=True, x_add=rows)
            ids = picks[0].tolist()
            hid = self.eng.ex.last_hidden
            for k, x in enumerate(act):
                x["tok"] = int(ids[k])
                x["hidden"] = hid[k:k + 1].clone()
                out[x["i"]].append(x["tok"])
            norm = self.eng.ex.w["final_norm"]
        return out

    def save_window(self, slot: int):
        return {"len": self.eng.slot_len[slot], "base": self.base[slot], "kept": self.kept[slot], "slot": slot,
                "gen": self.gen[slot]}

    def restore_window(self, slot: int, blob) -> None:
        # the head's KV rows up to the snapshot position are still in its slot when nothing started the slot over since
        # (same slot, same generation): only the length rolls back. Otherwise (another conversation used the slot, or the
        # snapshot comes back into another slot) the head starts over
        if (blob is None or blob["base"] != self.base[slot] or blob.get("slot") != slot or blob.get("gen") != self.gen[slot]
                or blob["len"] > self.eng.slot_len[slot]):
            self.reset(slot)
            return
        self.eng.slot_len[slot] = min(self.eng.slot_len[slot], blob["len"])
        self.kept[slot] = blob["kept"]
