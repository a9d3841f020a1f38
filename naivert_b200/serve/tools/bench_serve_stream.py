"""Host-path ceiling of the serving layer: streams from a fake engine that produces tokens
instantly, so the measured rate is what FastAPI + SSE + detokenisation can sustain on this host.

    python -m naivert_b200.serve.tools.bench_serve_stream --tokens 20000

Parity: tools/serve/bench_serve_stream.py of the reference (HTTP ceiling with a fake engine).
"""
from __future__ import annotations

import argparse
import json
import socket
import threading
import time

from ..chat import ByteTokenizer, ChatFormatter
from ..context import ServerContext
from ..http import build_app
from ..messages_api import ServerDefaults


class _Cfg:
    capacity, max_output_tokens = 1 << 20, 1 << 19
    eos_token_ids = (ByteTokenizer().eos_token_id,)


class _Session:
    def __init__(self, n, per_step):
        self.left, self.per, self.done, self.stop_reason, self.cached_tokens = n, per_step, False, None, 0

    def step(self, timeout):
        k = min(self.per, self.left)
        self.left -= k
        if self.left == 0:
            self.done, self.stop_reason = True, "output_limit"
        return [97 + (i % 26) for i in range(k)]

    def cancel(self):
        self.left, self.done, self.stop_reason = 0, True, "cancelled"

    def finish(self):
        return {}


class _Engine:
    config = _Cfg()

    def __init__(self, per_step):
        self.per = per_step

    def align_prompt(self, t, s):
        return t

    def open_session(self, tokens, max_decode, session_id, sampling):
        return _Session(max_decode, self.per)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=20000)
    ap.add_argument("--per-step", type=int, default=4)
    a = ap.parse_args(argv)
    import httpx
    import uvicorn
    eng = _Engine(a.per_step)
    app = build_app(lambda: ServerContext(eng, ChatFormatter(ByteTokenizer())), ServerDefaults(max_output_tokens=1 << 19))
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    srv = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning"))
    threading.Thread(target=srv.run, daemon=True).start()
    base = f"http://127.0.0.1:{port}"
    for _ in range(200):
        try:
            if httpx.get(base + "/health", timeout=1).status_code == 200:
                break
        except Exception:       # noqa: BLE001
            time.sleep(0.05)
    t0 = time.perf_counter()
    n_events = 0
    with httpx.stream("POST", base + "/v1/messages", timeout=None,
                      json={"model": "naive-n0.5", "max_tokens": a.tokens, "stream": True, "messages": [{"role": "user", "content": "go"}]}) as r:
        for line in r.iter_lines():
            n_events += line.startswith("event: content_block_delta")
    dt = time.perf_counter() - t0
    print(json.dumps({"tokens": a.tokens, "seconds": round(dt, 3), "tokens_per_s": round(a.tokens / dt, 1), "delta_events": n_events}))
    srv.should_exit = True
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
