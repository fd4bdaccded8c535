"""Tokenizers and the incremental UTF-8-safe detokenizer.

`HFTokenizer` wraps a Hugging Face `tokenizer.json` (byte-level BPE, as the served models use); `ByteTokenizer` is
a self-contained 256-byte + specials vocabulary for tests, the mock engine and random-init benchmarks.
`IncrementalDecoder` never emits a split multi-byte character: bytes of an incomplete UTF-8 sequence are held back
until the rest arrives (reference `Tok` / `IncrementalDecoder`, `crates/fe-server/src/tokenizer.rs`)."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence


class ByteTokenizer:
    """ids 0..255 = bytes; then the special tokens in `SPECIALS` order."""

    SPECIALS = ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>", "<tool_call>", "</tool_call>"]

    def __init__(self, vocab_size: int = 4096):
        self.vocab_size = max(vocab_size, 256 + len(self.SPECIALS))
        self.special_ids: Dict[str, int] = {s: 256 + i for i, s in enumerate(self.SPECIALS)}
        self.id_to_special = {v: k for k, v in self.special_ids.items()}
        self.eos_ids = [self.special_ids["<|endoftext|>"], self.special_ids["<|im_end|>"]]

    def encode(self, text: str) -> List[int]:
        out: List[int] = []
        i = 0
        while i < len(text):
            for s, sid in self.special_ids.items():
                if text.startswith(s, i):
                    out.append(sid)
                    i += len(s)
                    break
            else:
                j = i + 1
                while j < len(text) and not any(text.startswith(s, j) for s in self.special_ids):
                    j += 1
                out.extend(text[i:j].encode("utf-8"))
                i = j
        return out

    def token_bytes(self, tid: int) -> bytes:
        if tid < 256:
            return bytes([tid])
        s = self.id_to_special.get(tid)
        return s.encode("utf-8") if s is not None else b""

    def decode(self, ids: Sequence[int]) -> str:
        return b"".join(self.token_bytes(int(t)) for t in ids).decode("utf-8", errors="replace")

    def is_special(self, tid: int) -> bool:
        return tid in self.id_to_special


class HFTokenizer:
    def __init__(self, model_dir: str):
        from tokenizers import Tokenizer as _T
        self.tk = _T.from_file(os.path.join(model_dir, "tokenizer.json"))
        self.vocab_size = self.tk.get_vocab_size(with_added_tokens=True)
        cfg = {}
        p = os.path.join(model_dir, "tokenizer_config.json")
        if os.path.exists(p):
            cfg = json.load(open(p))
        self.special_ids = {}
        for tok in (cfg.get("added_tokens_decoder") or {}).values():
            tid = self.tk.token_to_id(tok["content"])
            if tid is not None:
                self.special_ids[tok["content"]] = tid
        eos = cfg.get("eos_token")
        eos = eos["content"] if isinstance(eos, dict) else eos
        self.eos_ids = [self.tk.token_to_id(t) for t in {eos, "<|im_end|>", "<|endoftext|>"} if t and self.tk.token_to_id(t) is not None]
        self._special_set = set(self.special_ids.values())

    def encode(self, text: str) -> List[int]:
        return self.tk.encode(text, add_special_tokens=False).ids

    def decode(self, ids: Sequence[int]) -> str:
        return self.tk.decode(list(ids), skip_special_tokens=False)

    def token_bytes(self, tid: int) -> bytes:
        return self.tk.decode([tid], skip_special_tokens=False).encode("utf-8")

    def is_special(self, tid: int) -> bool:
        return tid in self._special_set


def load_tokenizer(model_dir: Optional[str], vocab_size: int = 4096):
    if model_dir and os.path.exists(os.path.join(model_dir, "tokenizer.json")):
        return HFTokenizer(model_dir)
    return ByteTokenizer(vocab_size)


class IncrementalDecoder:
    """Feed token ids, get text that is always valid UTF-8 and never ends inside a character."""

    def __init__(self, tok):
        self.tok = tok
        self.pending = b""
        self.ids: List[int] = []
        self.emitted = ""

    def push(self, ids: Sequence[int]) -> str:
        if isinstance(self.tok, ByteTokenizer):
            self.pending += b"".join(self.tok.token_bytes(int(t)) for t in ids)
            cut = len(self.pending)
            # hold back an incomplete trailing sequence (at most 3 bytes)
            for back in range(1, min(4, len(self.pending)) + 1):
                b = self.pending[-back]
                if b & 0xC0 == 0x80:
                    continue
                need = 1 if b < 0x80 else 2 if b >> 5 == 0b110 else 3 if b >> 4 == 0b1110 else 4 if b >> 3 == 0b11110 else 1
                if need > back:
                    cut = len(self.pending) - back
                break
            out, self.pending = self.pending[:cut], self.pending[cut:]
            return out.decode("utf-8", errors="replace")
        # BPE tokenizers: re-decode the tail and emit what is stable (no replacement char at the end)
        self.ids.extend(int(t) for t in ids)
        text = self.tok.decode(self.ids)
        if text.endswith("�"):
            return ""
        out = text[len(self.emitted):]
        self.emitted = text
        if len(self.ids) > 64:
            self.ids, self.emitted = [], ""
        return out

    def flush(self) -> str:
        out = self.pending.decode("utf-8", errors="replace") if self.pending else ""
        self.pending = b""
        return out
