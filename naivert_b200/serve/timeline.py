"""Host-side request timeline: named spans on the server's monotonic clock, relative to HTTP
handler entry.  No CUDA calls and no device clock inference happen here.

Parity: naivert/serve/timeline.py (schema ``naivert.request_timeline.v1``).
"""
from __future__ import annotations

import time
from contextlib import contextmanager
from typing import Any, Dict, List, Optional

SCHEMA = "naivert.request_timeline.v1"


class RequestTimeline:
    def __init__(self, origin: Optional[float] = None):
        self.origin = time.monotonic() if origin is None else origin
        self.spans: List[Dict[str, Any]] = []

    def now_ms(self) -> float:
        return (time.monotonic() - self.origin) * 1e3

    def record(self, lane: str, name: str, start_ms: float, duration_ms: float, **args) -> None:
        self.spans.append({"lane": lane, "name": name, "start_ms": round(start_ms, 3),
                           "duration_ms": round(max(0.0, duration_ms), 3), "args": args})

    @contextmanager
    def span(self, lane: str, name: str, **args):
        t0 = self.now_ms()
        try:
            yield args
        finally:
            self.record(lane, name, t0, self.now_ms() - t0, **args)

    def snapshot(self) -> Dict[str, Any]:
        return {"schema": SCHEMA, "clock": "monotonic", "origin": "http_handler_entry", "end_ms": round(self.now_ms(), 3),
                "spans": list(self.spans)}
