"""The real server process on a GPU (random-init small model): JSON + SSE, same seed twice gives the
same text, a follow-up request reuses the parked prefix.  With 2+ GPUs the same through torchrun (rank 0
serves, rank 1 follows)."""
import json
import os
import socket
import subprocess
import sys
import time

import httpx
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _serve(nproc):
    port = _free_port()
    args = [os.path.join(ROOT, "examples", "serve_sessions.py"), "--model", "small", "--random-init", "--capacity", "4096",
            "--port", str(port), "--max-decode-tokens", "2048", "--log-level", "warning"]
    if nproc == 1:
        cmd = [sys.executable] + args
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
               "127.0.0.1", "--master-port", str(_free_port())] + args
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    base = f"http://127.0.0.1:{port}"
    t0 = time.time()
    while time.time() - t0 < 300:
        if proc.poll() is not None:
            raise RuntimeError("server exited: " + proc.stdout.read()[-3000:])
        try:
            if httpx.get(base + "/health", timeout=2).status_code == 200:
                return proc, base
        except Exception:
            pass
        time.sleep(0.5)
    proc.kill()
    raise RuntimeError("server did not become ready")


def _check(base):
    body = {"model": "small", "max_tokens": 48, "temperature": 0.8, "seed": 7,
            "messages": [{"role": "user", "content": "Tell me about caches. " * 4}]}
    a = httpx.post(base + "/v1/messages", json=body, headers={"x-session-id": "s"}, timeout=120)
    assert a.status_code == 200, a.text
    ma = a.json()
    assert ma["usage"]["output_tokens"] > 0 and ma["stop_reason"] in ("max_tokens", "end_turn")
    assert ma["naivert"]["timings"]["decode_tok_s_device"] > 0
    b = httpx.post(base + "/v1/messages", json=body, headers={"x-session-id": "other"}, timeout=120).json()
    assert [x.get("text") for x in b["content"]] == [x.get("text") for x in ma["content"]]       # same seed, same text
    c = httpx.post(base + "/v1/messages", json=dict(body, seed=8), timeout=120).json()
    assert c["usage"]["output_tokens"] > 0
    follow = dict(body)
    follow["messages"] = body["messages"] + [{"role": "assistant", "content": ma["content"]},
                                             {"role": "user", "content": "And what about the draft model?"}]
    d = httpx.post(base + "/v1/messages", json=follow, headers={"x-session-id": "s"}, timeout=120).json()
    assert d["usage"]["cache_read_input_tokens"] > 0, d["usage"]
    with httpx.stream("POST", base + "/v1/messages", json=dict(body, stream=True), timeout=120) as r:
        text = "".join(r.iter_text())
    assert "event: message_start" in text and "event: message_stop" in text
    assert httpx.get(base + "/health").json()["slot"] == "IDLE"


@pytest.mark.parametrize("nproc", [1, 2])
def test_server_process(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    proc, base = _serve(nproc)
    try:
        _check(base)
    finally:
        proc.terminate()
        try:
            proc.wait(20)
        except subprocess.TimeoutExpired:
            proc.kill()
