"""Native build: every CUDA translation unit is compiled for sm_100a with nvcc into one
in-tree shared library and loaded through ctypes.

A manifest (source digest + flags) is written beside the library; ``load_library`` rebuilds
when the digest changes and nvcc is present, and otherwise loads the library that travelled
with the tree.  On a machine with a GPU a missing or stale library that cannot be rebuilt
is a hard error - there is no Python fallback for the kernels.

Parity: naivert/kernels/build.py (``KernelBuildManifest``, digest-named modules, arch flags
:148-175) and naivert/kernels/toolchain.py (``SM_COUNT``).
"""
from __future__ import annotations

import ctypes
import hashlib
import json
import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor
from dataclasses import asdict, dataclass
from typing import List, Optional

SM_COUNT = 148
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--ftz=false", "--prec-div=true", "--prec-sqrt=true",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(_ROOT, "csrc")
LIB_DIR = os.path.join(_ROOT, "_lib")
LIB_NAME = "libnaivert_b200.so"
# The checking flavour: the same sources with -DNRT_BOUNDS_CHECK (every data-derived index is tested before use and the
# first violation is recorded, csrc/ptx.cuh).  Built on request (``python -m naivert_b200.ops.build --bounds``) beside the
# regular library and loaded instead of it when NAIVERT_BOUNDS_CHECK=1.
BOUNDS_LIB_NAME = "libnaivert_b200_bounds.so"
BOUNDS_UNITS = ("attn_decode", "moe_fused", "target_kernels", "draft")      # translation units that export nrt_bounds_<unit>


def bounds_flavour() -> bool:
    return os.environ.get("NAIVERT_BOUNDS_CHECK", "0") == "1"


@dataclass(frozen=True)
class KernelBuildManifest:
    digest: str
    sources: List[str]
    flags: List[str]
    nvcc: str

    def path(self) -> str:
        return os.path.join(LIB_DIR, "manifest.json")


def source_inventory() -> List[str]:
    out = []
    for root, _, files in os.walk(CSRC):
        for f in sorted(files):
            if f.endswith((".cu", ".cuh", ".hpp", ".h", ".cpp")):
                out.append(os.path.relpath(os.path.join(root, f), CSRC))
    return sorted(out)


def source_digest() -> str:
    h = hashlib.sha256()
    for rel in source_inventory():
        h.update(rel.encode())
        with open(os.path.join(CSRC, rel), "rb") as f:
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def find_nvcc() -> Optional[str]:
    cand = os.environ.get("NAIVERT_CUDA_HOME")
    if cand and os.path.isfile(os.path.join(cand, "bin", "nvcc")):
        return os.path.join(cand, "bin", "nvcc")
    return shutil.which("nvcc") or ("/usr/local/cuda/bin/nvcc" if os.path.isfile("/usr/local/cuda/bin/nvcc") else None)


def _read_manifest() -> Optional[dict]:
    p = os.path.join(LIB_DIR, "manifest.json")
    if os.path.isfile(p):
        try:
            return json.load(open(p))
        except Exception:
            return None
    return None


def is_current() -> bool:
    m = _read_manifest()
    return bool(m) and m.get("digest") == source_digest() and os.path.isfile(os.path.join(LIB_DIR, LIB_NAME))


def compile_library(verbose: bool = False, ptxas_info: bool = False, bounds: bool = False) -> str:
    """Compile every .cu under csrc/ (objects in parallel) and link the shared library (``bounds``: the checking flavour)."""
    nvcc = find_nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build the sm_100a kernels")
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(LIB_DIR, "obj_bounds" if bounds else "obj")
    os.makedirs(obj_dir, exist_ok=True)
    units = [s for s in source_inventory() if s.endswith(".cu")]
    rdc_units = [u for u in units if os.path.basename(u).startswith("rdc_")]
    flags = ARCH_FLAGS + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + (["-DNRT_BOUNDS_CHECK"] if bounds else [])

    def one(rel):
        obj = os.path.join(obj_dir, rel.replace("/", "_") + ".o")
        cmd = [nvcc] + flags + ["-I", CSRC, "-c", os.path.join(CSRC, rel), "-o", obj]
        if rel in rdc_units:
            cmd.insert(1, "-rdc=true")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {rel}:\n{r.stderr[-4000:]}")
        if verbose or ptxas_info:
            print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(units))) as ex:
        objs = list(ex.map(one, units))
    out = os.path.join(LIB_DIR, BOUNDS_LIB_NAME if bounds else LIB_NAME)
    link = [nvcc] + ARCH_FLAGS + ["-shared", "-o", out] + objs + ["-lcudart"]
    if rdc_units:
        link.insert(1, "-rdc=true")
        link += ["-lcudadevrt"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stderr[-4000:]}")
    man = KernelBuildManifest(source_digest(), source_inventory(), flags, nvcc)
    with open(os.path.join(LIB_DIR, "manifest_bounds.json") if bounds else man.path(), "w") as f:
        json.dump(asdict(man), f, indent=1)
    return out


_LIB: Optional[ctypes.CDLL] = None


def load_library(rebuild: Optional[bool] = None) -> ctypes.CDLL:
    """Load (building if stale and possible) the kernel library."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if bounds_flavour():
        path = os.path.join(LIB_DIR, BOUNDS_LIB_NAME)
        man = os.path.join(LIB_DIR, "manifest_bounds.json")
        cur = os.path.isfile(path) and os.path.isfile(man) and json.load(open(man)).get("digest") == source_digest()
        if not cur:
            if find_nvcc() is None:
                raise RuntimeError(f"{path} is missing or stale and cannot be built here")
            compile_library(bounds=True)
        _LIB = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
        return _LIB
    path = os.path.join(LIB_DIR, LIB_NAME)
    stale = not is_current()
    if rebuild or (rebuild is None and stale and find_nvcc() is not None):
        compile_library()
    if not os.path.isfile(path):
        raise RuntimeError(f"{path} is missing and cannot be built here; the CUDA kernels have no fallback")
    _LIB = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    return _LIB


def main(argv: Optional[List[str]] = None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description="Build the sm_100a kernel library in-tree.")
    ap.add_argument("--bounds", action="store_true", help="build the index-checking flavour (libnaivert_b200_bounds.so) as well")
    ap.add_argument("--only-bounds", action="store_true", help="build only the index-checking flavour")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers / spills / shared memory per kernel")
    a = ap.parse_args(argv)
    if not a.only_bounds:
        print(compile_library(ptxas_info=a.ptxas_info))
    if a.bounds or a.only_bounds:
        print(compile_library(ptxas_info=a.ptxas_info, bounds=True))
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(main())
