#!/usr/bin/env python3
"""Minimal chat client for the Messages endpoint (uses the anthropic SDK when present, else httpx)."""
import argparse
import json
import sys


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--base-url", default="http://127.0.0.1:8080")
    ap.add_argument("--model", default="naive-n0.5")
    ap.add_argument("--max-tokens", type=int, default=512)
    ap.add_argument("--session", default="chat-http")
    ap.add_argument("prompt", nargs="*", default=["Explain KV caching in three sentences."])
    a = ap.parse_args()
    import httpx
    body = {"model": a.model, "max_tokens": a.max_tokens, "stream": True,
            "messages": [{"role": "user", "content": " ".join(a.prompt)}]}
    with httpx.stream("POST", a.base_url + "/v1/messages", json=body, headers={"x-session-id": a.session}, timeout=None) as r:
        for line in r.iter_lines():
            if line.startswith("data: "):
                ev = json.loads(line[6:])
                if ev.get("type") == "content_block_delta":
                    d = ev["delta"]
                    sys.stdout.write(d.get("text") or d.get("thinking") or "")
                    sys.stdout.flush()
                elif ev.get("type") == "message_delta":
                    print("\n---", json.dumps(ev.get("usage")), json.dumps(ev.get("naivert", {}).get("timings", {})))


if __name__ == "__main__":
    main()
