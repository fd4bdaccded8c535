"""Context-copy speculation: propose the continuation of an earlier occurrence of the current suffix.

Code edits and tool outputs repeat long spans of their own context; a suffix match against the sequence so far
gives draft tokens for free. Counterpart of the reference's `Copier` (`crates/fe-model/src/copy.rs:1-221`:
KEY 3, MIN_MATCH 5, MAX_MATCH 64, SCAN 512, MISSES 4, SILENCE 16; `sync / propose / observe`).
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

KEY = 3            # n-gram length of the index
MIN_MATCH = 5      # shortest suffix match worth proposing from
MAX_MATCH = 64     # longest proposal
SCAN = 512         # most candidate positions examined per proposal
MISSES = 4         # consecutive failed proposals before going quiet
SILENCE = 16       # steps to stay quiet


class Copier:
    def __init__(self):
        self.tokens: List[int] = []
        self.index: Dict[Tuple[int, ...], List[int]] = {}
        self.misses = 0
        self.quiet = 0

    def sync(self, tokens: Sequence[int]) -> None:
        """Bring the index up to date with the sequence (prompt + generated so far); handles rollbacks."""
        n = len(self.tokens)
        if len(tokens) < n or list(tokens[:n]) != self.tokens:
            self.tokens, self.index = [], {}
            n = 0
        for i in range(n, len(tokens)):
            self.tokens.append(int(tokens[i]))
            if i + 1 >= KEY:
                key = tuple(self.tokens[i + 1 - KEY:i + 1])
                self.index.setdefault(key, []).append(i + 1)      # position right after the n-gram

    def propose(self, max_len: int = MAX_MATCH) -> List[int]:
        if self.quiet > 0:
            self.quiet -= 1
            return []
        t = self.tokens
        n = len(t)
        if n < MIN_MATCH + 1:
            return []
        cands = self.index.get(tuple(t[n - KEY:n]), [])
        best_len, best_pos = 0, -1
        for pos in reversed(cands[-SCAN:]):
            if pos >= n:
                continue
            m = 0
            while m < MAX_MATCH and pos - 1 - m >= 0 and t[pos - 1 - m] == t[n - 1 - m]:
                m += 1
            if m > best_len:
                best_len, best_pos = m, pos
        if best_len < MIN_MATCH:
            return []
        return t[best_pos:best_pos + min(max_len, MAX_MATCH)]

    def observe(self, proposed: int, accepted: int) -> None:
        """Feedback after verification: a proposal that got nothing accepted counts as a miss."""
        if proposed == 0:
            return
        if accepted == 0:
            self.misses += 1
            if self.misses >= MISSES:
                self.quiet, self.misses = SILENCE, 0
        else:
            self.misses = 0
