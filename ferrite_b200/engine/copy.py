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
    """`lo` / `hi`: bounds of the adaptive proposal length. A proposal that lands whole doubles the next one (up to `hi`),
    one of which less than half lands halves it (down to `lo`); going quiet resets it (reference `Copier::observe`,
    `crates/fe-model/src/copy.rs:105-125`)."""

    def __init__(self, lo: int = 4, hi: int = MAX_MATCH):
        self.tokens: List[int] = []
        self.index: Dict[Tuple[int, ...], List[int]] = {}
        # the index and the suffix match run in C++ when the extension is built (`csrc/host_runtime.cpp`); the Python
        # statement below is the same algorithm and serves otherwise
        from .._ext import host
        h = host()
        self.native = h.CopyIndex(KEY, MIN_MATCH, MAX_MATCH, SCAN) if h is not None else None
        self.misses = 0
        self.quiet = 0
        self.lo, self.hi = max(1, lo), max(lo, hi)
        self.extra = self.lo                 # copy rows to propose next time

    def sync(self, tokens: Sequence[int]) -> None:
        """Bring the index up to date with the sequence (prompt + generated so far); handles rollbacks."""
        if self.native is not None:
            # per step the sequence only grows: when its length did not shrink and the indexed sequence's last tokens are
            # still in place, only the new tokens cross into C++; anything else is a full (exact) resync
            n = self.native.size()
            k = min(n, 8)
            if len(tokens) >= n and [int(t) for t in tokens[n - k:n]] == list(self.native.tail(k)):
                if len(tokens) > n:
                    self.native.extend([int(t) for t in tokens[n:]])
            else:
                self.native.sync([int(t) for t in tokens])
            return
        n = len(self.tokens)
        if len(tokens) < n or list(tokens[:n]) != self.tokens:
            self.tokens, self.index = [], {}
            n = 0
        for i in range(n, len(tokens)):
            self.tokens.append(int(tokens[i]))
            if i + 1 >= KEY:
                key = tuple(self.tokens[i + 1 - KEY:i + 1])
                self.index.setdefault(key, []).append(i + 1)      # position right after the n-gram

    def propose(self, max_len: int = MAX_MATCH, adaptive: bool = False) -> List[int]:
        """Up to `max_len` tokens (with `adaptive`: up to the current adaptive length) that followed the latest longest
        earlier occurrence of the sequence's end. A continuation that reaches the end of the sequence goes on with the
        copy itself, so a loop with a period shorter than the proposal continues."""
        if self.quiet > 0:
            self.quiet -= 1
            return []
        if self.native is not None:
            return list(self.native.propose(min(max_len, MAX_MATCH, self.extra if adaptive else MAX_MATCH)))
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
                if m == MAX_MATCH:
                    break
        if best_len < MIN_MATCH:
            return []
        want = min(max_len, MAX_MATCH, self.extra if adaptive else MAX_MATCH)
        out: List[int] = []
        for j in range(want):
            i = best_pos + j
            out.append(t[i] if i < n else out[i - n])
        return out

    def observe(self, proposed: int, accepted: int) -> None:
        """Feedback after verification: how many of the proposed copy rows were kept."""
        if proposed == 0:
            return
        if accepted == proposed:
            self.extra = min(self.hi, self.extra * 2)
        elif 2 * accepted < proposed:
            self.extra = max(self.lo, self.extra // 2)
        if accepted == 0:
            self.misses += 1
            if self.misses >= MISSES:
                self.quiet, self.misses, self.extra = SILENCE, 0, self.lo
        else:
            self.misses = 0


def graft(toks: List[int], parents: List[int], copy: Sequence[int], room: int) -> Tuple[int, int]:
    """Put a copy proposal onto a verify tree. `toks[0]` is the segment's root (the token being fed), `parents[r]` the row
    a row hangs from (-1 for the root), `copy` the tokens proposed after the root. The copy is followed down the rows that
    already hold it; up to `room` of what is left is appended as a chain below the deepest of them. Returns (tokens of
    the copy found in the tree, rows added). Reference `graft`, `crates/fe-model/src/copy.rs:128-147`."""
    from .._ext import host
    h = host()
    if h is not None:
        t2, p2, found, added = h.host_graft([int(t) for t in toks], [int(x) for x in parents], [int(t) for t in copy], int(room))
        toks[:], parents[:] = list(t2), list(p2)
        return int(found), int(added)
    r, i = 0, 0
    while i < len(copy):
        nxt = next((c for c in range(r + 1, len(toks)) if parents[c] == r and toks[c] == copy[i]), None)
        if nxt is None:
            break
        r, i = nxt, i + 1
    add = min(len(copy) - i, max(0, room))
    for t in copy[i:i + add]:
        parents.append(r)
        toks.append(int(t))
        r = len(toks) - 1
    return i, add
