"""Minimal HTTP/SSE client on `http.client` shared by the conformance suite and the bench clients."""
from __future__ import annotations

import http.client
import json
import time
from typing import Any, Dict, Iterator, Optional, Tuple
from urllib.parse import urlparse


class Client:
    def __init__(self, base_url: str, timeout: float = 120.0):
        u = urlparse(base_url)
        self.host, self.port = u.hostname or "127.0.0.1", u.port or 80
        self.prefix = u.path.rstrip("/")
        self.timeout = timeout

    def _conn(self) -> http.client.HTTPConnection:
        return http.client.HTTPConnection(self.host, self.port, timeout=self.timeout)

    def get(self, path: str) -> Tuple[int, Any]:
        c = self._conn()
        c.request("GET", self.prefix + path)
        r = c.getresponse()
        body = r.read()
        c.close()
        try:
            return r.status, json.loads(body)
        except ValueError:
            return r.status, body.decode("utf-8", "replace")

    def post(self, path: str, payload: Dict[str, Any]) -> Tuple[int, Any, Dict[str, str]]:
        c = self._conn()
        c.request("POST", self.prefix + path, json.dumps(payload), {"Content-Type": "application/json"})
        r = c.getresponse()
        body = r.read()
        headers = {k.lower(): v for k, v in r.getheaders()}
        c.close()
        try:
            return r.status, json.loads(body), headers
        except ValueError:
            return r.status, body.decode("utf-8", "replace"), headers

    def stream(self, path: str, payload: Dict[str, Any]) -> Iterator[Tuple[float, Optional[Dict[str, Any]]]]:
        """Yields (seconds since the request was sent, event) per SSE data line; the `[DONE]` line yields None."""
        c = self._conn()
        t0 = time.perf_counter()
        c.request("POST", self.prefix + path, json.dumps(dict(payload, stream=True)), {"Content-Type": "application/json"})
        r = c.getresponse()
        if r.status != 200:
            body = r.read().decode("utf-8", "replace")
            c.close()
            raise RuntimeError(f"HTTP {r.status}: {body[:300]}")
        for raw in r:
            line = raw.decode("utf-8", "replace").strip()
            if not line.startswith("data:"):
                continue
            data = line[5:].strip()
            if data == "[DONE]":
                yield time.perf_counter() - t0, None
                break
            yield time.perf_counter() - t0, json.loads(data)
        c.close()
