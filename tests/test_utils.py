"""Guarded tensors, layering (import direction), build manifest."""
import ast
import os

import pytest
import torch

from naivert_b200.utils.guarded import CanaryError, GuardedPool

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_guarded_pool_detects_overrun_and_underrun():
    pool = GuardedPool()
    a = pool.alloc("a", (4, 8), torch.float32)
    b = pool.alloc("b", (3,), torch.int32)
    a.fill_(1.0)
    b.fill_(7)
    pool.verify()
    raw = pool._items[0][1]
    raw[4096 + 4 * 8 * 4 + 1] = 0                      # one byte past the end of "a"
    with pytest.raises(CanaryError, match="a .*overrun"):
        pool.verify()
    raw[4096 + 4 * 8 * 4 + 1] = 0x5A
    pool._items[1][1][10] = 0
    with pytest.raises(CanaryError, match="b .*underrun"):
        pool.verify()


# lower layers never import higher ones: models/ops < parallel < runtime < serve
ORDER = {"models": 0, "ops": 0, "utils": 0, "parallel": 1, "runtime": 2, "prefill": 2, "serve": 3}


def test_layering_import_direction():
    pkg = os.path.join(ROOT, "naivert_b200")
    bad = []
    for layer, level in ORDER.items():
        d = os.path.join(pkg, layer)
        for fn in os.listdir(d) if os.path.isdir(d) else []:
            if not fn.endswith(".py"):
                continue
            tree = ast.parse(open(os.path.join(d, fn)).read())
            for node in ast.walk(tree):
                if isinstance(node, ast.ImportFrom) and node.level == 2 and node.module:
                    dep = node.module.split(".")[0]
                    if dep in ORDER and ORDER[dep] > level:
                        bad.append(f"{layer}/{fn} imports {dep}")
    assert not bad, bad


def test_build_manifest_digest_tracks_sources(tmp_path, monkeypatch):
    from naivert_b200.ops import build
    d1 = build.source_digest()
    assert d1 == build.source_digest() and len(d1) == 64
    inv = build.source_inventory()
    assert "gemm.cu" in inv and "ptx.cuh" in inv and all(not p.startswith("/") for p in inv)
    monkeypatch.setattr(build, "NVCC_FLAGS", build.NVCC_FLAGS + ["-DX"])
    assert build.source_digest() != d1


def test_prefill_chunk_plan():
    from naivert_b200.prefill.native import plan_chunks
    cs = plan_chunks(0, 699, 256, 16)
    assert [(c.pos0, c.rows) for c in cs] == [(0, 256), (256, 256), (512, 176)]
    assert plan_chunks(100, 110, 256, 16) == []
    cs = plan_chunks(64, 64 + 4096 * 2 + 40, 4096, 128)
    assert sum(c.rows for c in cs) == 4096 * 2 and all(c.rows % 128 == 0 for c in cs)
    import pytest
    with pytest.raises(ValueError):
        plan_chunks(0, 100, 250, 16)
