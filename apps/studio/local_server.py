"""Local server for the Studio client: serves the static files of this folder and forwards ``/v1/*`` and ``/health``
to the API server, so the browser talks to one origin (no CORS set-up) - streaming responses are passed through chunk
by chunk.

    python apps/studio/local_server.py --api http://127.0.0.1:8080 --port 8000

Reference counterpart: apps/studio/local_server.mjs (a node script; this image has no node, and the server side of
this repository is Python).
"""
from __future__ import annotations

import argparse
import http.client
import os
import sys
from http.server import SimpleHTTPRequestHandler, ThreadingHTTPServer
from urllib.parse import urlsplit

HERE = os.path.dirname(os.path.abspath(__file__))
HOP = {"connection", "keep-alive", "proxy-authenticate", "proxy-authorization", "te", "trailers", "transfer-encoding", "upgrade"}


def make_handler(api: str):
    target = urlsplit(api)

    class Handler(SimpleHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def __init__(self, *a, **kw):
            super().__init__(*a, directory=HERE, **kw)

        def log_message(self, fmt, *args):                  # quiet by default
            if os.environ.get("STUDIO_VERBOSE"):
                super().log_message(fmt, *args)

        def _proxied(self) -> bool:
            return self.path.startswith("/v1/") or self.path == "/health"

        def _forward(self):
            n = int(self.headers.get("content-length") or 0)
            body = self.rfile.read(n) if n else None
            conn_cls = http.client.HTTPSConnection if target.scheme == "https" else http.client.HTTPConnection
            conn = conn_cls(target.hostname, target.port, timeout=600)
            try:
                headers = {k: v for k, v in self.headers.items() if k.lower() not in HOP and k.lower() != "host"}
                conn.request(self.command, self.path, body=body, headers=headers)
                resp = conn.getresponse()
                self.send_response(resp.status)
                for k, v in resp.getheaders():
                    if k.lower() not in HOP and k.lower() != "content-length":
                        self.send_header(k, v)
                self.send_header("Transfer-Encoding", "chunked")
                self.end_headers()
                while True:                                  # pass server-sent events through as they arrive
                    chunk = resp.read1(65536)
                    if not chunk:
                        break
                    self.wfile.write(f"{len(chunk):x}\r\n".encode() + chunk + b"\r\n")
                    self.wfile.flush()
                self.wfile.write(b"0\r\n\r\n")
            except (ConnectionError, OSError) as e:
                try:
                    self.send_error(502, f"API server unreachable: {e}")
                except OSError:
                    pass
            finally:
                conn.close()

        def do_GET(self):
            if self._proxied():
                return self._forward()
            return super().do_GET()

        def do_POST(self):
            if self._proxied():
                return self._forward()
            self.send_error(405)

    return Handler


def serve(api: str, host: str = "127.0.0.1", port: int = 8000) -> ThreadingHTTPServer:
    return ThreadingHTTPServer((host, port), make_handler(api))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--api", default="http://127.0.0.1:8080")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    a = ap.parse_args(argv)
    srv = serve(a.api, a.host, a.port)
    print(f"studio on http://{a.host}:{a.port}/ -> {a.api}", flush=True)
    try:
        srv.serve_forever()
    except KeyboardInterrupt:
        pass
    return 0


if __name__ == "__main__":
    sys.exit(main())
