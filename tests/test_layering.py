"""Import direction between the sub-packages: a lower layer never imports an upper one.

utils < ops < models, parallel < runtime, prefill < serve.  Sub-packages of one tier may import each other
(runtime and prefill share the decode caches).  Parity: the reference keeps the same direction between its
ops/bindings, models, runtime and serve packages (tests/reference/test_layer_boundaries.py).
"""
import ast
import os

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "naivert_b200")
TIER = {"utils": 0, "ops": 1, "models": 2, "parallel": 2, "runtime": 3, "prefill": 3, "serve": 4}


def _imports(path, pkg_parts):
    tree = ast.parse(open(path).read())
    for node in ast.walk(tree):
        if isinstance(node, ast.ImportFrom):
            if node.level > 0:
                base = pkg_parts[:len(pkg_parts) - (node.level - 1)] if node.level > 1 else list(pkg_parts)
                full = base + (node.module.split(".") if node.module else [])
                if not node.module:                       # "from .. import x, y"
                    for alias in node.names:
                        yield (base + [alias.name])[0]
                    continue
                yield full[0] if full else None
            elif node.module and node.module.split(".")[0] == "naivert_b200":
                parts = node.module.split(".")
                yield parts[1] if len(parts) > 1 else None
        elif isinstance(node, ast.Import):
            for alias in node.names:
                parts = alias.name.split(".")
                if parts[0] == "naivert_b200" and len(parts) > 1:
                    yield parts[1]


def test_lower_layers_do_not_import_upper_layers():
    bad = []
    seen = set()
    for dp, _, files in os.walk(ROOT):
        rel = os.path.relpath(dp, ROOT)
        parts = [] if rel == "." else rel.split(os.sep)
        if not parts or parts[0] not in TIER:
            continue
        for f in files:
            if not f.endswith(".py"):
                continue
            for tgt in _imports(os.path.join(dp, f), parts):
                if tgt in TIER and tgt != parts[0]:
                    seen.add((parts[0], tgt))
                    if TIER[tgt] > TIER[parts[0]]:
                        bad.append(f"{os.path.join(rel, f)} imports {tgt}")
    assert not bad, bad
    assert ("runtime", "ops") in seen and ("models", "ops") in seen          # the walk really saw the imports


def test_no_committed_module_reaches_into_working_files():
    for base in (ROOT, os.path.join(os.path.dirname(ROOT), "tests"), os.path.join(os.path.dirname(ROOT), "examples")):
        for dp, _, files in os.walk(base):
            for f in files:
                if f.endswith(".py") and f != "test_layering.py":
                    text = open(os.path.join(dp, f)).read()
                    assert "_work/" not in text and "_work." not in text and '"_work"' not in text, os.path.join(dp, f)


FORBIDDEN_TOP_LEVEL = {"triton", "tilelang", "tvm", "jax", "flash_attn", "flashinfer", "vllm", "cutlass", "deep_gemm", "sgl_kernel"}


def test_no_compatibility_layer_or_kernel_library_is_imported():
    """The compute path is this repository's own sm_100a kernels: no module of the package, the benchmark or the
    examples imports a kernel DSL, a multi-backend layer or a third-party kernel library (the reference guards its
    tree the same way with an import hook: tests/support/external_dependency_guard.py)."""
    top = os.path.dirname(ROOT)
    files = [os.path.join(top, "bench.py"), os.path.join(top, "__graft_entry__.py")]
    for base in (ROOT, os.path.join(top, "examples"), os.path.join(top, "devops")):
        for dp, _, fs in os.walk(base):
            files += [os.path.join(dp, f) for f in fs if f.endswith(".py")]
    bad = []
    for path in files:
        tree = ast.parse(open(path).read())
        for node in ast.walk(tree):
            names = []
            if isinstance(node, ast.Import):
                names = [a.name for a in node.names]
            elif isinstance(node, ast.ImportFrom) and node.level == 0 and node.module:
                names = [node.module]
            elif isinstance(node, ast.Call) and getattr(node.func, "id", getattr(node.func, "attr", "")) in ("import_module", "__import__"):
                names = [a.value for a in node.args[:1] if isinstance(a, ast.Constant) and isinstance(a.value, str)]
            for n in names:
                if n.split(".")[0] in FORBIDDEN_TOP_LEVEL:
                    bad.append(f"{os.path.relpath(path, top)} imports {n}")
    assert not bad, bad
    assert len(files) > 40


def test_no_torch_compile_on_any_path():
    top = os.path.dirname(ROOT)
    for dp, _, fs in os.walk(ROOT):
        for f in fs:
            if f.endswith(".py"):
                src = open(os.path.join(dp, f)).read()
                assert "torch.compile(" not in src and "@torch.compile" not in src, os.path.join(dp, f)
    assert "torch.compile(" not in open(os.path.join(top, "bench.py")).read()
