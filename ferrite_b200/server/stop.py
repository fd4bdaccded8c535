"""Stop-string matching on a text stream: text that could still become a stop string is held back.
Counterpart of `StopMatcher::push/flush` (`crates/fe-server/src/stop.rs:4-59`)."""
from __future__ import annotations

from typing import List, Optional, Tuple


class StopMatcher:
    def __init__(self, stops: List[str], include: bool = False):
        self.stops = [s for s in stops if s]
        self.include = include
        self.buf = ""
        self.hit: Optional[str] = None
        # the scan runs in C++ on UTF-8 bytes when the extension is built (`csrc/host_runtime.cpp`)
        from .._ext import host
        h = host()
        self.native = h.StopScanner([s.encode("utf-8") for s in self.stops], include) if (h is not None and self.stops) else None

    def push(self, text: str) -> Tuple[str, bool]:
        """Returns (text safe to emit, stopped)."""
        if self.hit is not None:
            return "", True
        if not self.stops:
            return text, False
        if self.native is not None:
            out, stopped = self.native.push(text.encode("utf-8"))
            if stopped:
                self.hit = self.native.hit().decode("utf-8")
            return out.decode("utf-8"), stopped
        self.buf += text
        best = None
        for s in self.stops:
            i = self.buf.find(s)
            if i >= 0 and (best is None or i < best[0]):
                best = (i, s)
        if best is not None:
            i, s = best
            out = self.buf[:i + (len(s) if self.include else 0)]
            self.hit, self.buf = s, ""
            return out, True
        # keep the longest suffix that is a proper prefix of some stop string
        hold = 0
        for s in self.stops:
            for k in range(min(len(s) - 1, len(self.buf)), 0, -1):
                if self.buf.endswith(s[:k]):
                    hold = max(hold, k)
                    break
        out = self.buf[:len(self.buf) - hold]
        self.buf = self.buf[len(self.buf) - hold:]
        return out, False

    def flush(self) -> str:
        if self.native is not None:
            return self.native.flush().decode("utf-8")
        out, self.buf = self.buf, ""
        return out
