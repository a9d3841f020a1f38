#!/usr/bin/env python3
"""Deployment checks.

    --check-env     toolchain + python packages + (if present) GPU architecture
    --compile       build the sm_100a kernel library and verify the binding struct sizes
    --serve-smoke   start the server with a small random-init model, send one request, stop it

Parity: devops/warm_kernels.py of the reference (``--check-env/--compile/--serve-smoke``).
"""
import argparse
import importlib
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def check_env() -> dict:
    from naivert_b200.ops import build
    out = {"nvcc": build.find_nvcc(), "packages": {}, "gpu": None}
    for m in ("torch", "safetensors", "fastapi", "uvicorn", "pydantic", "httpx"):
        try:
            out["packages"][m] = getattr(importlib.import_module(m), "__version__", "ok")
        except Exception as e:          # noqa: BLE001
            out["packages"][m] = f"MISSING ({type(e).__name__})"
    try:
        import torch
        if torch.cuda.is_available():
            cc = torch.cuda.get_device_capability(0)
            out["gpu"] = {"name": torch.cuda.get_device_name(0), "cc": f"{cc[0]}.{cc[1]}", "count": torch.cuda.device_count(),
                          "supported": cc == (10, 0)}
    except Exception as e:              # noqa: BLE001
        out["gpu"] = f"error: {e}"
    out["ok"] = out["nvcc"] is not None and not any("MISSING" in str(v) for v in out["packages"].values())
    return out


def compile_all() -> dict:
    from naivert_b200.ops import build
    t0 = time.time()
    path = build.compile_library()
    from naivert_b200.ops import kernels
    res = {"library": path, "seconds": round(time.time() - t0, 1), "units": [u for u in build.source_inventory() if u.endswith(".cu")]}
    try:
        kernels.aux_lib()
        res["bindings"] = "ok"
    except OSError as e:
        res["bindings"] = f"not loadable here ({e})"
        return res
    # argument structs against the sources, and every kernel variant the runtimes ask for against the built library
    from naivert_b200.ops import abi, variants
    res["abi_mismatches"] = abi.check_all()
    res["variant_problems"] = variants.check_library(kernels.lib())
    res["variants"] = sorted(variants.variants())
    res["ok"] = not res["abi_mismatches"] and not res["variant_problems"]
    return res


def serve_smoke(port: int = 18080) -> dict:
    import httpx
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "examples", "serve_sessions.py"), "--model", "small", "--random-init",
                             "--capacity", "2048", "--port", str(port), "--log-level", "warning"])
    base = f"http://127.0.0.1:{port}"
    try:
        for _ in range(600):
            try:
                if httpx.get(base + "/health", timeout=2).status_code == 200:
                    break
            except Exception:           # noqa: BLE001
                pass
            if proc.poll() is not None:
                return {"ok": False, "error": "server exited"}
            time.sleep(0.5)
        r = httpx.post(base + "/v1/messages", json={"model": "small", "max_tokens": 16, "messages": [{"role": "user", "content": "ping"}]}, timeout=120)
        return {"ok": r.status_code == 200, "status": r.status_code, "usage": r.json().get("usage")}
    finally:
        proc.terminate()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--check-env", action="store_true")
    ap.add_argument("--compile", action="store_true")
    ap.add_argument("--serve-smoke", action="store_true")
    a = ap.parse_args()
    rc = 0
    if a.check_env:
        r = check_env()
        print(json.dumps(r, indent=1))
        rc |= 0 if r["ok"] else 1
    if a.compile:
        r = compile_all()
        print(json.dumps(r, indent=1))
        rc |= 0 if r.get("ok", True) else 1
    if a.serve_smoke:
        r = serve_smoke()
        print(json.dumps(r, indent=1))
        rc |= 0 if r["ok"] else 1
    return rc


if __name__ == "__main__":
    sys.exit(main())
