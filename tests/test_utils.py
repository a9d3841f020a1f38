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


def test_contract_header_matches_python():
    from naivert_b200.runtime import contract as C
    h = C.parse_header()
    for name, value in h.items():
        if name.startswith("NRT_CTRL_") and name != "NRT_CTRL_RESERVED3":
            assert getattr(C, name[4:]) == value, name
    stops = {v: k for k, v in h.items() if k.startswith("NRT_STOP_")}
    assert set(stops) == set(C.STOP_REASONS), (stops, C.STOP_REASONS)
    assert h["NRT_CTRL_WORDS"] == 16


def test_power_of_two_scale_variants():
    import torch
    from naivert_b200.ops import quant as Q
    g = torch.Generator().manual_seed(0)
    s = torch.tensor([0.0, 0.25, 0.3, 1.0, 1.5, 3.9e-5])
    assert Q.ue8m0_round_up(s).tolist() == [1.0, 0.25, 0.5, 1.0, 2.0, 2.0 ** -14]
    w = torch.randn(256, 384, generator=g) * 0.02
    w8, si = Q.quantize_fp8_block(w)
    q2, s2 = Q.requant_block_ue8m0(w8, si)
    assert torch.all(torch.log2(s2) == torch.log2(s2).round())
    back = Q.dequant_block(q2, s2)
    assert (back - w).abs().max() <= 0.13 * w.abs().max()      # two e4m3 roundings
    x = torch.randn(4, 128, generator=g)
    q, sc = Q.quantize_mxfp8(x)
    assert sc.shape == (4, 4) and torch.all(torch.log2(sc) == torch.log2(sc).round())
    assert (Q.dequant_mxfp8(q, sc) - x).abs().max() <= 0.07 * x.abs().max()


def test_moe_math_pieces():
    import torch
    from naivert_b200.models import moe_math as M
    from naivert_b200.models.spec import MoeRoutingSpec
    g = torch.Generator().manual_seed(1)
    rt = MoeRoutingSpec(score_func="sigmoid", expert_count=8, top_k=2, intermediate=128, shared_expert_count=0,
                        route_scale=1.0, normalize_top_k=True)
    x = torch.randn(5, 64, generator=g).bfloat16()
    xn = M.rmsnorm(x, torch.ones(64), 1e-5)
    assert abs(xn.pow(2).mean().item() - 1.0) < 0.05
    w, b = torch.randn(8, 64, generator=g) * 0.1, torch.zeros(8)
    b[3] = 10.0                                           # the bias forces expert 3 into every selection ...
    ids, p = M.route(xn, w, b, rt)
    assert (ids == 3).any(-1).all() and torch.allclose(p.sum(-1), torch.ones(5), atol=1e-6)
    score = torch.sigmoid(xn @ w.t())
    sel3 = (ids == 3).float()
    # ... but its weight is the unbiased score
    assert torch.allclose((p * sel3).sum(-1), score[:, 3] / torch.gather(score, 1, ids.long()).sum(-1), atol=1e-5)
    outs = [torch.randn(5, 64, generator=g).bfloat16() for _ in range(8)]
    y = M.combine(x, outs, ids, p)
    r0 = x[0].float() + sum(pp * outs[e][0].float() for e, pp in sorted(zip(ids[0].tolist(), p[0].tolist())))
    assert torch.equal(y[0], r0.to(torch.bfloat16))
    parts = [torch.randn(5, 64, generator=g) for _ in range(4)]
    z = M.combine_tp_partials(x, parts)
    assert torch.equal(z, (x.float() + sum(pp.to(torch.bfloat16).float() for pp in parts)).to(torch.bfloat16)) or \
        (z.float() - (x.float() + sum(parts))).abs().max() < 0.1
    q = M.quantize_down_activation(torch.randn(3, 256, generator=g))
    assert q.shape == (3, 256)


def test_audit_prefix_capture(tmp_path):
    import json
    from naivert_b200.serve.tools.audit_prefix_capture import audit
    sys_p = [{"type": "text", "text": "be brief", "cache_control": {"type": "ephemeral"}}]
    r1 = {"system": sys_p, "messages": [{"role": "user", "content": "zqxj-secret"}]}
    r2 = {"system": "be brief" and [{"type": "text", "text": "be brief"}],
          "messages": [{"role": "user", "content": [{"type": "text", "text": "zqxj-secret"}]},
                       {"role": "assistant", "content": [{"type": "thinking", "thinking": "x"}, {"type": "text", "text": "yo"}]},
                       {"role": "user", "content": "more"}]}
    r3 = {"system": sys_p, "messages": [{"role": "user", "content": "changed"}, {"role": "user", "content": "more"}]}
    cap = tmp_path / "cap.jsonl"
    rows = [{"rid": "a", "body": json.dumps(r1)}, {"rid": "b", "body": json.dumps(r2)}, {"rid": "c", "body": json.dumps(r3)},
            {"rid": "b", "response": True, "usage": {"input_tokens": 7, "cache_read_input_tokens": 5}}]
    cap.write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    rep = audit(cap, [["a", "b"], ["a", "c"], ["a", "zzz"]])
    ab, ac, az = rep["pairs"]
    assert ab["messages_prefix_equal"] and ab["system_equal"] and ab["added_roles"] == ["assistant", "user"]
    assert ab["added_assistant_block_types"] == [["thinking", "text"]] and ab["later_usage"]["cache_read_input_tokens"] == 5
    assert not ac["messages_prefix_equal"] and ac["first_changed_message"] == 0
    assert "error" in az and len(rep["capture_sha256"]) == 64
    assert "zqxj-secret" not in json.dumps(rep)


def test_acceptance_histogram():
    from naivert_b200.runtime.session_engine import acceptance_histogram
    assert acceptance_histogram([0, 7, 7, 3, 9, -1]) == [2, 0, 0, 1, 0, 0, 0, 3]
    assert acceptance_histogram([]) == [0] * 8


def test_ep_layout_reference_invariants():
    import torch
    from naivert_b200.prefill.ep_moe import ep_layout_reference
    g = torch.Generator().manual_seed(2)
    tp, E, T, k = 2, 16, 40, 4
    ids = [torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]) for _ in range(tp)]
    for item_rows in (16, 64):
        lay = ep_layout_reference(ids, E, item_rows)
        for d in range(tp):
            taken = {}
            for s in range(tp):
                for e, row in zip(ids[s].flatten().tolist(), lay["slot"][s].flatten().tolist()):
                    if e // (E // tp) == d:
                        assert row not in taken                     # every pair has its own row
                        taken[row] = e
            for el, (base, rows) in enumerate(zip(lay["seg_base"][d], lay["seg_rows"][d])):
                assert base % item_rows == 0
                got = sorted(r for r, e in taken.items() if e == d * (E // tp) + el)
                assert got == list(range(base, base + rows))        # a segment is dense and starts at its base
            covered = sum(min(item_rows, lay["seg_rows"][d][el] - (r0 - lay["seg_base"][d][el])) for el, r0 in lay["items"][d])
            assert covered == sum(lay["seg_rows"][d])               # the work list covers every received row once
        assert sum(sum(r) for r in lay["seg_rows"]) == tp * T * k


def test_xid_delta_check(tmp_path):
    from naivert_b200.utils import xid_check as X
    old = "[ 10.0] NVRM: Xid (PCI:0000:1b:00): 31, pid=1, name=python, Ch 00000008\n[ 11.0] usb 1-1: new device\n"
    new = old + "[ 99.5] NVRM: Xid (PCI:0000:1b:00): 109, pid=7, name=python, errorString CTX SWITCH TIMEOUT\n"
    assert X.new_xid_lines(old, old) == [] and X.xid_codes(X.new_xid_lines(old, new)) == [109]
    # the same text appearing a second time is a new event
    assert len(X.new_xid_lines(old, old + old)) == 1
    a, b, c = tmp_path / "a.txt", tmp_path / "b.txt", tmp_path / "c.txt"
    src_old, src_new = tmp_path / "old.log", tmp_path / "new.log"
    src_old.write_text(old); src_new.write_text(new)
    assert X.main(["snapshot", str(a), "--source", str(src_old)]) == 0
    assert X.main(["snapshot", str(b), "--source", str(src_new)]) == 0
    assert X.main(["compare", str(a), str(a)]) == 0 and X.main(["compare", str(a), str(b)]) == 1
    assert X.main(["snapshot", str(c), "--source", str(tmp_path / "missing.log")]) == 0
    assert X.main(["compare", str(a), str(c)]) == 0 and X.main(["compare", str(a), str(c), "--strict"]) == 1


def test_ctypes_mirrors_match_the_c_argument_structs():
    """Field names, offsets and sizes of every kernel argument struct, parsed from the CUDA sources, equal the ctypes
    classes of ops/kernels.py; structs declared in several translation units are identical there."""
    from naivert_b200.ops import abi
    problems = abi.check_all()
    assert not problems, problems
    assert len(abi.check_all.report) == len(abi.STRUCTS) >= 18
    # the parser itself: layout of a struct with padding, arrays and a nested struct
    inner = abi.parse_fields("int a; const float* p; unsigned char pad[3];", {})
    lay, size, align = abi.layout(inner)
    assert lay == [("a", 0, 4), ("p", 8, 8), ("pad", 16, 3)] and size == 24 and align == 8
    outer = abi.parse_fields("Inner x[2]; unsigned long long t; uint16_t h;", {"Inner": (24, 8)})
    assert abi.layout(outer)[0] == [("x", 0, 48), ("t", 48, 8), ("h", 56, 2)] and abi.layout(outer)[1] == 64


def test_bindings_generated_from_the_cuda_sources_equal_the_kept_mirrors(tmp_path):
    """``abi.generate`` / ``abi --emit`` build ctypes classes from the C declarations; every class used by the launch
    wrappers has the same field names, offsets, sizes and total size as its generated counterpart."""
    import ctypes as C
    import importlib.util
    from naivert_b200.ops import abi, kernels as K
    out = tmp_path / "generated_abi.py"
    out.write_text(abi.emit_module())
    sp = importlib.util.spec_from_file_location("generated_abi", out)
    gen = importlib.util.module_from_spec(sp)
    sp.loader.exec_module(gen)

    def lay(cls):
        return [(n, getattr(cls, n).offset, getattr(cls, n).size) for n, _ in cls._fields_]

    parsed, cache = abi.parse_all(), {}
    for name, (_, cls_name) in abi.STRUCTS.items():
        kept, emitted, built = getattr(K, cls_name), getattr(gen, name), abi.generate(name, parsed, cache)
        assert lay(kept) == lay(emitted) == lay(built), name
        assert C.sizeof(kept) == C.sizeof(emitted) == C.sizeof(built), name
    # nested argument structs are the generated classes themselves, pointers are void pointers
    g = abi.generate("GemmArgs", parsed, cache)
    kinds = dict(g._fields_)
    assert any(t is cache["FabricArgs"] for t in kinds.values()) and C.c_void_p in kinds.values()


def test_kernel_variants_fail_closed():
    from dataclasses import replace
    from naivert_b200.ops import variants as V
    table = V.variants()
    assert len(table) >= 25 and all(v.variant_id.endswith(f".sm100a.abi{v.abi_version}") for v in table.values())
    assert len({v.entry for v in table.values()}) == len(table)
    for e in V.STEP_VARIANTS + V.PREFILL_VARIANTS:
        assert V.by_entry(e).entry == e
    g = V.by_entry("nrt_gemm_launch")
    assert g.args_bytes and g.max_rows == 16
    assert V.require_variant(g, replace(g)) == g
    with pytest.raises(ValueError, match="differs from the library"):
        V.require_variant(g, replace(g, args_bytes=g.args_bytes + 8))
    with pytest.raises(ValueError, match="differs"):
        V.require_variant(g, replace(g, abi_version=g.abi_version + 1, variant_id=f"x.sm100a.abi{g.abi_version + 1}"))
    with pytest.raises(ValueError):
        V.KernelVariant("gemm.sm90a.abi1", "f")
    with pytest.raises(ValueError):
        V.KernelVariant("gemm.sm100a.abi1", "f", args_struct="GemmArgs")

    class FakeLib:                                   # a library built before nrt_moe_layer existed, with an older GemmArgs
        def nrt_gemm_launch(self): ...
        def nrt_gemm_args_size(self): return g.args_bytes - 16
    with pytest.raises(ValueError, match="exports no nrt_moe_layer"):
        V.library_variant(FakeLib(), V.by_entry("nrt_moe_layer"))
    with pytest.raises(ValueError, match="argument bytes"):
        V.require_entries(FakeLib(), ["nrt_gemm_launch"])
    # the built library, when present, provides every variant with the expected ABI
    from naivert_b200.ops import kernels as K
    try:
        lib = K.lib()
    except Exception:
        return
    assert V.check_library(lib) == []
    assert len(V.require_entries(lib, V.STEP_VARIANTS + V.PREFILL_VARIANTS)) == len(V.STEP_VARIANTS + V.PREFILL_VARIANTS)


def test_decode_modes_and_call_plans():
    import re
    from naivert_b200.models.registry import resolve_model
    from naivert_b200.ops import variants as V
    from naivert_b200.runtime import modes as M
    spec = resolve_model("naive-n0.5")
    # every launcher a mode names is a known kernel variant
    for m in M.MODES.values():
        assert m.pointer_fields == M.POINTER_FIELDS
        for e in m.entries:
            assert V.by_entry(e).entry == e
    greedy, rnd = M.MODES["greedy_step"], M.MODES["speculative_round"]
    null = {b.name for b in greedy.buffers if b.storage == "null"}
    assert null == M.DRAFT_ONLY | {"host_ring"} and all(b.storage != "null" for b in rnd.buffers)
    assert [b.storage for b in rnd.buffers if b.name == "block_ids"] == ["borrowed"]
    # call-index plans: unique, inside one epoch, consecutive calls in different slabs
    plan = M.allreduce_call_plan(spec)
    assert len(plan) == 2 * spec.layer_count + 1 + 2 * spec.draft.layer_count
    assert M.layer_call_tags(20) == (40, 41) and dict(plan)["draft.input"] == M.DRAFT_CALL_BASE
    xp = dict(M.exchange_call_plan())
    assert xp["sampler.nucleus3.digit"] == 9 and xp["tail.pause_consensus"] == 13 and xp["markov.6"] == 22
    with pytest.raises(ValueError, match="same slab"):
        M._check_plan([("a", 2), ("b", 6)], 64, 4, "exchange")
    with pytest.raises(ValueError, match="used by"):
        M._check_plan([("a", 2), ("b", 3), ("c", 2)], 64, 4, "exchange")
    with pytest.raises(ValueError, match="outside"):
        M._check_plan([("a", 64)], 64, 4, "exchange")
    # the plan is what the sources use
    csrc = os.path.join(ROOT, "naivert_b200", "csrc")
    samp = open(os.path.join(csrc, "sampler.cu")).read()
    used = set(re.findall(r"a\.x, (\d+)\)", samp)) | set(re.findall(r"a\.x, (\d \+ 2 \* pass)\)", samp))
    assert used == {"0", "1", "2 + 2 * pass", "3 + 2 * pass", "10", "11", "12", "13"}
    assert "16 + step" in open(os.path.join(csrc, "draft.cu")).read()
    src = open(os.path.join(ROOT, "naivert_b200", "runtime", "draft.py")).read()
    assert f"DRAFT_CALL_BASE = {M.DRAFT_CALL_BASE}" in src
    assert "epoch) * 1024u" in open(os.path.join(csrc, "gemm.cuh")).read()
    assert f"kXchgSlabs = {M.XCHG_SLABS}" in open(os.path.join(csrc, "fabric.cuh")).read()
    # capacity rule
    assert M.request_fits(8192, 1024, 8192 + 1024 + 32) and not M.request_fits(8192, 1024, 8192 + 1024 + 31)
    assert not M.request_fits(0, 10, 1000)


def test_status_words_are_explained():
    from naivert_b200.parallel.fabric import explain_status
    assert explain_status(0) == "ok"
    assert "nucleus pass 2: bins to the owning rank" in explain_status(0x700 | 6)
    assert "threshold digit" in explain_status(0x700 | 3) and "Markov step 3" in explain_status(0x700 | 19)
    assert "tail pause consensus" in explain_status(0x700 | 13) and "arg-max" in explain_status(0x700 | 60)
    assert "sampler phase 2" in explain_status(0x800 | 0x42) and "Markov step 3" in explain_status(0x800 | 0x23)
    assert "fused MoE arrival" in explain_status(0x801) and "mailbox" in explain_status(0x501)
    assert "return slot 3" in explain_status(0x583) and "all-gather flag of source rank 2" in explain_status(0x562)
    assert "unknown" in explain_status(0x999)
    # the classes are the enumerators of the device header
    src = open(os.path.join(ROOT, "naivert_b200", "csrc", "ptx.cuh")).read()
    for name, value in (("kSiteTmaFull", 0x100), ("kSiteStageEmpty", 0x200), ("kSiteAccFull", 0x300), ("kSiteAccEmpty", 0x400),
                        ("kSiteMailbox", 0x500), ("kSiteCluster", 0x600), ("kSiteRendezvous", 0x700), ("kSiteGrid", 0x800)):
        assert f"{name} = 0x{value:x}" in src


def test_fabric_byte_formulas_match_the_device_layout():
    """The host sizes the peer-mapped regions; the kernels address them.  Both sides are derived here from the same
    constants, read out of the CUDA sources: the last word any kernel can address lies inside the allocation."""
    import re
    from naivert_b200.ops import kernels as K
    from naivert_b200.parallel import fabric as F
    gem = open(os.path.join(ROOT, "naivert_b200", "csrc", "gemm.cuh")).read()
    fab = open(os.path.join(ROOT, "naivert_b200", "csrc", "fabric.cuh")).read()

    def const(src, name):
        return int(re.search(rf"constexpr int {name} = (\d+);", src).group(1))
    assert const(gem, "kMaxPeers") == K.K_MAX_PEERS and const(gem, "kMailboxSlabs") == K.K_MAILBOX_SLABS
    assert "constexpr int kRowPairs = kTok / 2;" in gem and const(gem, "kTok") // 2 == K.K_ROW_PAIRS
    assert const(gem, "kArRows") // 2 <= K.K_ROW_PAIRS
    words, slabs, peers = const(fab, "kXchgMaxWords"), const(fab, "kXchgSlabs"), const(fab, "kXchgPeers")
    for tp in (2, 4, 8):
        for feats in (4096, 8192):
            # all-reduce mailbox: word index (slab * tp + source) * kRowPairs * features + pair * features + feature
            last = ((K.K_MAILBOX_SLABS - 1) * tp + tp - 1) * K.K_ROW_PAIRS * feats + (K.K_ROW_PAIRS - 1) * feats + feats - 1
            assert (last + 1) * 8 == F.mailbox_bytes(tp, feats)
        # small exchange: word index ((slab * tp + source) * kXchgMaxWords + i) * 2 + half
        last = (((slabs - 1) * tp + tp - 1) * words + words - 1) * 2 + 1
        assert (last + 1) * 8 == F.xchg_bytes(tp)
    assert peers == K.K_MAX_PEERS
    # the largest exchange of a round (15 distributions x 256 bins) fits the value range of one call
    samp = open(os.path.join(ROOT, "naivert_b200", "csrc", "sampler.cu")).read()
    assert "kRowsP = 8, kRowsQ = 7" in samp and 15 * 256 <= words


def test_stamp_reports_from_synthetic_buffers():
    """The phase reports of the step profiler read plain buffers of %globaltimer stamps: median / last CTA per phase,
    relative to the layer's first stamp; stamps older than that (a CTA that was not last in this replay) are ignored."""
    import torch
    from naivert_b200.runtime.step_profile import report_sampler_stamps, report_stamps
    t0 = 1_000_000
    gemm = torch.zeros(300 * 16, dtype=torch.int64)
    g = gemm.view(300, 16)
    for cta in range(4):
        g[cta, 0] = t0 + 100 * cta                    # entry
        g[cta, 2] = t0 + 2000 + 100 * cta             # upstream done
        g[cta, 11] = t0 + 9000 + 1000 * cta           # epilogue done
    g[0, 9] = t0 - 500                                # a stale stamp of an earlier replay
    g[1, 10] = 7                                      # mailbox sweeps
    g[1, 3] = t0 + 3000
    lines = report_stamps({"args_o": gemm}, 20)
    text = "\n".join(lines)
    assert "layer 20 o: 4 CTAs" in lines[0]
    assert any("upstream done" in l and "2.15 /     2.30" in l for l in lines), text
    assert any("epilogue done" in l and "12.00" in l for l in lines), text
    assert any("mailbox sweeps (max)" in l and l.strip().endswith("7") for l in lines), text
    assert not any("peer words arrived" in l for l in lines), text          # the stale stamp lies before the layer's first
    samp = torch.zeros(32, dtype=torch.int64)
    assert report_sampler_stamps(samp) == []
    samp[30] = t0
    for ph in range(7):
        samp[2 * ph], samp[2 * ph + 1] = t0 + 10_000 * ph + 3000, t0 + 10_000 * ph + 8000
    out = report_sampler_stamps(samp)
    assert len(out) == 8 and "maxima" in out[1] and "3.00 /     8.00" in out[1] and "63.00 /    68.00" in out[7]
