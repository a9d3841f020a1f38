"""Deployment scripts without a GPU: env -> flags mapping of the entrypoint, environment check."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_entrypoint_env_to_flags():
    env = dict(os.environ, NAIVERT_DRY_RUN="1", NAIVERT_GPUS="4", NAIVERT_PORT="9000", NAIVERT_RANDOM_INIT="1",
               NAIVERT_STORE_GB="12", NAIVERT_TARGET_CHECKPOINT="/ckpt/t", NAIVERT_CORS_ORIGIN="https://ui.example")
    out = subprocess.run(["bash", os.path.join(ROOT, "devops", "entrypoint.sh")], env=env, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    line = out.stdout.strip()
    assert line.startswith("gpus=4") and "--port 9000" in line and "--random-init" in line
    assert "--store-gb 12" in line and "--target /ckpt/t" in line and "--cors-origin https://ui.example" in line
    assert "--draft" not in line


def test_check_env_reports():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "devops", "warm_kernels.py"), "--check-env"], capture_output=True, text=True)
    rep = json.loads(out.stdout)
    assert "packages" in rep and rep["packages"]["fastapi"] != "" and "nvcc" in rep


def _fake_docker(tmp_path, nogpu_exit=1):
    """A stand-in for the docker CLI that logs its arguments and plays the container's part for every step."""
    log = tmp_path / "docker_calls.log"
    fake = tmp_path / "docker"
    fake.write_text(f"""#!/usr/bin/env bash
echo "$@" >> {log}
case "$1" in
  build|rm) exit 0 ;;
  image) echo 123456789; exit 0 ;;
  compose) exit 0 ;;
  run)
    if [[ "$*" == *"--name naivert-b200-tier1-"* ]]; then echo "no CUDA device"; exit {nogpu_exit}; fi
    exit 0 ;;
esac
exit 64
""")
    fake.chmod(0o755)
    return fake, log


def test_tier1_passes_with_expected_exit_codes(tmp_path):
    fake, log = _fake_docker(tmp_path)
    out_dir = tmp_path / "out"
    env = dict(os.environ, NAIVERT_DOCKER=str(fake), NAIVERT_VALIDATION_DIR=str(out_dir))
    p = subprocess.run(["bash", os.path.join(ROOT, "devops", "tier1.sh"), "img:test"], env=env, capture_output=True, text=True)
    assert p.returncode == 0 and "TIER1_OK" in p.stdout, p.stdout + p.stderr
    calls = log.read_text()
    assert "build -f devops/Dockerfile -t img:test ." in calls and "compose -f devops/docker-compose.yml config -q" in calls
    assert "-m pytest tests -x -q -m not gpu" in calls
    assert (out_dir / "nogpu.exit").read_text().strip() == "1" and (out_dir / "size_bytes").read_text().strip() == "123456789"


def test_tier1_fails_when_gpuless_start_succeeds(tmp_path):
    """A server that comes up without GPUs (exit 0) or hangs is a failed check, not a pass."""
    fake, _ = _fake_docker(tmp_path, nogpu_exit=0)
    env = dict(os.environ, NAIVERT_DOCKER=str(fake), NAIVERT_VALIDATION_DIR=str(tmp_path / "out"))
    p = subprocess.run(["bash", os.path.join(ROOT, "devops", "tier1.sh")], env=env, capture_output=True, text=True)
    assert p.returncode == 1 and "nogpu exited 0, expected 1" in p.stderr and "TIER1_FAILED" in p.stderr


def test_compose_file_is_consistent_with_the_entrypoint():
    import re
    import yaml
    doc = yaml.safe_load(open(os.path.join(ROOT, "devops", "docker-compose.yml")))
    svc = doc["services"]["server"]
    assert svc["container_name"] == "naivert-b200" and "python -c" in svc["healthcheck"]["test"]
    assert svc["ipc"] == "host" and svc["build"]["dockerfile"] == "devops/Dockerfile"
    assert svc["deploy"]["resources"]["reservations"]["devices"][0]["capabilities"] == ["gpu"]
    entry = open(os.path.join(ROOT, "devops", "entrypoint.sh")).read()
    known = set(re.findall(r"NAIVERT_[A-Z_]+", entry))
    for key in svc["environment"]:
        if key.startswith("NAIVERT_"):
            assert key in known, f"{key} is set by compose but not read by the entrypoint"


def test_studio_local_server_serves_files_and_proxies_streams():
    """Static files from apps/studio and a pass-through of /health and a chunked /v1/messages stream."""
    import http.client
    import importlib.util
    import threading
    from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

    class Api(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, *a):
            pass

        def do_GET(self):
            body = b'{"status": "ok"}'
            self.send_response(200); self.send_header("content-type", "application/json")
            self.send_header("content-length", str(len(body))); self.end_headers(); self.wfile.write(body)

        def do_POST(self):
            n = int(self.headers.get("content-length") or 0)
            sent = self.rfile.read(n)
            self.send_response(200); self.send_header("content-type", "text/event-stream")
            self.send_header("x-echo-session", self.headers.get("x-session-id", "")); self.send_header("Transfer-Encoding", "chunked"); self.end_headers()
            for piece in (b"event: message_start\ndata: {}\n\n", b"event: echo\ndata: " + sent + b"\n\n"):
                self.wfile.write(f"{len(piece):x}\r\n".encode() + piece + b"\r\n"); self.wfile.flush()
            self.wfile.write(b"0\r\n\r\n")

    api = ThreadingHTTPServer(("127.0.0.1", 0), Api)
    threading.Thread(target=api.serve_forever, daemon=True).start()
    spec = importlib.util.spec_from_file_location("studio_local_server", os.path.join(ROOT, "apps", "studio", "local_server.py"))
    mod = importlib.util.module_from_spec(spec); spec.loader.exec_module(mod)
    srv = mod.serve(f"http://127.0.0.1:{api.server_address[1]}", port=0)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        c = http.client.HTTPConnection("127.0.0.1", srv.server_address[1], timeout=10)
        c.request("GET", "/index.html"); r = c.getresponse(); page = r.read()
        assert r.status == 200 and b"<html" in page.lower()
        c.request("GET", "/health"); r = c.getresponse()
        assert r.status == 200 and json.loads(r.read())["status"] == "ok"
        c.request("POST", "/v1/messages", body=b'{"x": 1}', headers={"content-type": "application/json", "x-session-id": "S"})
        r = c.getresponse(); text = r.read().decode()
        assert r.status == 200 and r.getheader("x-echo-session") == "S"
        assert "event: message_start" in text and 'data: {"x": 1}' in text
        c.request("POST", "/other", body=b""); r = c.getresponse(); r.read()
        assert r.status == 405
    finally:
        srv.shutdown(); api.shutdown()


def test_reference_retarget_edits_only_the_architecture_strings(tmp_path, monkeypatch):
    """The comparison arm runs a copy of the reference in which only the architecture strings differ: every edited
    line is reported, other files are byte-identical, the prefill-only vendored trees are left out."""
    import importlib.util
    sp = importlib.util.spec_from_file_location("retarget_reference", os.path.join(ROOT, "baseline", "retarget_reference.py"))
    mod = importlib.util.module_from_spec(sp)
    sp.loader.exec_module(mod)
    src = tmp_path / "src"
    (src / "naivert" / "kernels").mkdir(parents=True)
    (src / "naivert" / "prefill" / "kernels" / "fa4").mkdir(parents=True)
    (src / "devops").mkdir()
    builder = "FLAGS = ['-gencode', 'arch=compute_103a,code=sm_103a']\nKEEP = 1\nARCH_LIST = '10.3a'\n"
    (src / "naivert" / "kernels" / "build.py").write_text(builder)
    (src / "naivert" / "kernels" / "body.cuh").write_text("// compute_103a stays in non-script sources\n")
    (src / "naivert" / "prefill" / "kernels" / "fa4" / "x.py").write_text("compute_103a\n")
    (src / "devops" / "Dockerfile").write_text("ENV TORCH_CUDA_ARCH_LIST='10.3a'\n")
    (src / "README.md").write_text("untouched compute_103a\n")
    monkeypatch.setattr(mod, "DEST", str(tmp_path / "copy"))
    edits = mod.retarget(str(src))
    dest = tmp_path / "copy"
    assert sorted((e[0], e[1]) for e in edits) == [("devops/Dockerfile", 1), ("naivert/kernels/build.py", 1), ("naivert/kernels/build.py", 3)]
    assert (dest / "naivert" / "kernels" / "build.py").read_text() == builder.replace("compute_103a", "compute_100a").replace(
        "sm_103a", "sm_100a").replace("'10.3a'", "'10.0a'")
    assert (dest / "naivert" / "kernels" / "body.cuh").read_text() == (src / "naivert" / "kernels" / "body.cuh").read_text()
    assert (dest / "README.md").read_text() == "untouched compute_103a\n"
    assert not (dest / "naivert" / "prefill" / "kernels").exists()
    assert all("103a" not in e[3] and "10.3a" not in e[3] for e in edits)
    # running it again replaces the copy instead of layering edits
    assert len(mod.retarget(str(src))) == 3
