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
