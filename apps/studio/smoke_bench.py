#!/usr/bin/env python3
"""One fixed request through every way the Studio reaches the server, timed and compared.

    python apps/studio/smoke_bench.py --api http://127.0.0.1:8080 [--proxy http://127.0.0.1:8000] [--seed 42]

The same prompt and seed go out as a JSON request, as a server-sent-event stream, and (with ``--proxy``) as a stream
through ``local_server.py``.  Per mode: HTTP status, time to response headers, time to first content, total time,
output tokens, the device rate the server reports (``naivert.timings.decode_tok_s_device``) and a hash of the text.
Same seed, same prompt: the texts must be identical in every mode; the exit code is 1 when they are not or a request
fails.  The server's sampler is seeded per request, so this is also the determinism check of the HTTP path.

Reference counterpart: apps/studio/tests/pelican_bench.py (direct against proxied requests of one prompt).
"""
from __future__ import annotations

import argparse
import hashlib
import http.client
import json
import sys
import time
from urllib.parse import urlsplit

PROMPT = "Draw a pelican riding a bicycle as an SVG image. Answer with the SVG markup only."


def one_request(endpoint: str, model: str, seed: int, stream: bool, max_tokens: int, prompt: str = PROMPT, timeout: float = 1200.0) -> dict:
    u = urlsplit(endpoint)
    cls = http.client.HTTPSConnection if u.scheme == "https" else http.client.HTTPConnection
    conn = cls(u.hostname, u.port, timeout=timeout)
    body = {"model": model, "max_tokens": max_tokens, "seed": seed, "stream": stream, "thinking": {"type": "disabled"},
            "messages": [{"role": "user", "content": prompt}]}
    t0 = time.perf_counter()
    conn.request("POST", "/v1/messages", json.dumps(body), {"content-type": "application/json", "x-session-id": f"smoke-{seed}-{int(stream)}"})
    resp = conn.getresponse()
    out = {"status": resp.status, "headers_ms": round((time.perf_counter() - t0) * 1e3, 2), "first_content_ms": None}
    if resp.status != 200:
        out["error"] = resp.read(2048).decode("utf-8", "replace")
        conn.close()
        return out
    text, usage, timings, stop, complete = [], {}, {}, None, False
    if stream:
        event, data = None, []
        for raw in resp:
            line = raw.decode("utf-8").rstrip("\r\n")
            if line.startswith("event: "):
                event = line[7:]
            elif line.startswith("data: "):
                data.append(line[6:])
            elif not line and data:
                d = json.loads("\n".join(data))
                if event == "content_block_delta":
                    piece = d["delta"].get("text")
                    if piece:
                        if out["first_content_ms"] is None:
                            out["first_content_ms"] = round((time.perf_counter() - t0) * 1e3, 2)
                        text.append(piece)
                elif event == "message_delta":
                    usage, stop = d.get("usage", {}), d.get("delta", {}).get("stop_reason")
                    timings = (d.get("naivert") or {}).get("timings", {})
                elif event == "message_stop":
                    complete = True
                elif event == "error":
                    out["error"] = json.dumps(d)
                event, data = None, []
    else:
        m = json.loads(resp.read())
        out["first_content_ms"] = round((time.perf_counter() - t0) * 1e3, 2)
        text = [b.get("text", "") for b in m.get("content", []) if b.get("type") == "text"]
        usage, stop, timings = m.get("usage", {}), m.get("stop_reason"), (m.get("naivert") or {}).get("timings", {})
        complete = m.get("type") == "message"
    conn.close()
    full = "".join(text)
    out.update(total_s=round(time.perf_counter() - t0, 4), complete=complete, stop_reason=stop,
               output_tokens=usage.get("output_tokens"), device_tok_s=timings.get("decode_tok_s_device"),
               chars=len(full), sha256=hashlib.sha256(full.encode()).hexdigest())
    return out


def run(api: str, proxy: str = None, model: str = "naive-n0.5", seed: int = 42, max_tokens: int = 8192, prompt: str = PROMPT) -> dict:
    modes = {"json": (api, False), "sse": (api, True)}
    if proxy:
        modes["sse_via_proxy"] = (proxy, True)
    results = {name: one_request(ep, model, seed, stream, max_tokens, prompt) for name, (ep, stream) in modes.items()}
    ok = all(r["status"] == 200 and r.get("complete") and "error" not in r for r in results.values())
    same = len({r.get("sha256") for r in results.values()}) == 1
    return {"prompt_sha256": hashlib.sha256(prompt.encode()).hexdigest(), "seed": seed, "modes": results,
            "all_completed": ok, "texts_identical": same, "ok": ok and same}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--api", required=True, help="origin of the API server")
    ap.add_argument("--proxy", default=None, help="origin of apps/studio/local_server.py in front of it")
    ap.add_argument("--model", default="naive-n0.5")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--max-tokens", type=int, default=8192)
    a = ap.parse_args(argv)
    rep = run(a.api, a.proxy, a.model, a.seed, a.max_tokens)
    print(json.dumps(rep, indent=1))
    return 0 if rep["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
