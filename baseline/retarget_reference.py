"""Prepare the reference tree for the same-box comparison arm of ``bench.py``.

The reference is not pip-installable (no ``setup.py`` / ``pyproject.toml``), so it is copied as a
source tree into ``baseline/_ref``.  Its kernel builders hard-code the B300 architecture
(``compute_103a``), for which this CUDA toolkit cannot generate code that runs on a B200; the only
edit made to the copy is that architecture string (``compute_103a`` -> ``compute_100a``,
``sm_103a`` -> ``sm_100a``, arch list ``10.3a`` -> ``10.0a``).  Every edited line is listed in
``baseline/RETARGET.txt``; nothing else of the copy differs from the source.

    python baseline/retarget_reference.py [--source /path/to/reference]
"""
from __future__ import annotations

import argparse
import os
import shutil

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
SUBS = (("compute_103a", "compute_100a"), ("sm_103a", "sm_100a"), ("'10.3a'", "'10.0a'"))
SUFFIXES = (".py", ".sh")
# Vendored third-party sources that only the reference's prefill path uses (FlashAttention-4, FlashInfer, DeepEP) and
# its build outputs are left out of the copy: the comparison arm drives the decode / verify kernels, and the GPU
# runner refuses multi-GPU calls while the tree carries those sources (their TMA loads broadcast across a cluster).
PRUNE = ("naivert/kernels/naive_n0p5/prefill_ext", "naivert/prefill/kernels", "tests/gpu/prefill_native", "tests/build")


def retarget(source: str) -> list:
    if os.path.isdir(DEST):
        shutil.rmtree(DEST)
    shutil.copytree(source, DEST, symlinks=True)
    for rel in PRUNE:
        shutil.rmtree(os.path.join(DEST, rel), ignore_errors=True)
    edits = []
    for root, _, files in os.walk(DEST):
        for name in sorted(files):
            if not name.endswith(SUFFIXES) and name != "Dockerfile":
                continue
            path = os.path.join(root, name)
            try:
                text = open(path, encoding="utf-8").read()
            except UnicodeDecodeError:
                continue
            if not any(a in text for a, _ in SUBS):
                continue
            lines = text.split("\n")
            for i, line in enumerate(lines):
                new = line
                for a, b in SUBS:
                    new = new.replace(a, b)
                if new != line:
                    edits.append((os.path.relpath(path, DEST), i + 1, line.strip(), new.strip()))
                    lines[i] = new
            with open(path, "w", encoding="utf-8") as f:
                f.write("\n".join(lines))
    return edits


def make_overlay() -> str:
    """Directory of symbolic links to the newest CCCL / CUTLASS header trees installed with the Python packages
    (flashinfer vendors CCCL 3.x and CUTLASS 4.5), for the reference's own include-path knob."""
    import importlib.util
    spec = importlib.util.find_spec("flashinfer")
    if spec is None or not spec.submodule_search_locations:
        raise SystemExit("flashinfer (the package that vendors the headers) is not installed")
    data = os.path.join(list(spec.submodule_search_locations)[0], "data")
    links = {"cub": "cccl/cub/cub", "cuda": "cccl/libcudacxx/include/cuda", "nv": "cccl/libcudacxx/include/nv",
             "thrust": "cccl/thrust/thrust", "cute": "cutlass/include/cute", "cutlass": "cutlass/include/cutlass"}
    out = os.path.join(HERE, "include_overlay")
    os.makedirs(out, exist_ok=True)
    for name, rel in links.items():
        dst = os.path.join(out, name)
        if os.path.islink(dst):
            os.unlink(dst)
        os.symlink(os.path.join(data, rel), dst)
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--source", default=os.environ.get("NAIVERT_REFERENCE_SRC"), required="NAIVERT_REFERENCE_SRC" not in os.environ,
                    help="checkout of the reference repository (or set NAIVERT_REFERENCE_SRC)")
    ap.add_argument("--overlay", action="store_true", help="also (re)create baseline/include_overlay")
    a = ap.parse_args()
    if a.overlay:
        print("include overlay:", make_overlay())
    edits = retarget(a.source)
    with open(os.path.join(HERE, "RETARGET.txt"), "w") as f:
        f.write("# lines of the reference copy that differ from the source (architecture string only)\n")
        for rel, ln, old, new in edits:
            f.write(f"{rel}:{ln}\n  - {old}\n  + {new}\n")
    print(f"{len(edits)} lines edited in {DEST}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
