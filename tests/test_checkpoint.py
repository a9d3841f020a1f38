"""Checkpoint writer/reader round trip, header validation, identity, TP slicing."""
import json
import os

import pytest
import torch

from naivert_b200.models import checkpoint as ck
from naivert_b200.models.naive_n0p5 import NAIVE_N0P5, tiny_spec
from naivert_b200.models.reference import ReferenceModel
from naivert_b200.models.weights import (init_state_dict, interleave_rope, prepare_weights, shard_weights)


def test_roundtrip_and_identity(tmp_path):
    spec = tiny_spec("fp8")
    root = str(tmp_path / "tgt")
    ident = ck.write_target_checkpoint(root, spec, seed=3, shard_bytes=1 << 20)
    c = ck.LocalCheckpoint(root)
    assert c.identity() == ident
    assert len(set(c.weight_map.values())) > 1          # really sharded
    ck.validate_target_layout(spec, c)
    sd = c.load_tensors()
    ref = init_state_dict(spec, seed=3)
    assert set(sd) == set(ref)
    for k in ref:
        assert sd[k].dtype == ref[k].dtype
        assert torch.equal(sd[k].view(torch.uint8) if sd[k].dtype == torch.float8_e4m3fn else sd[k],
                           ref[k].view(torch.uint8) if ref[k].dtype == torch.float8_e4m3fn else ref[k])
    assert ident.dtype_counts["F8_E4M3"] == 2 * (8 + 1) * 3
    w, ident2 = ck.load_rank_weights(spec, root, rank=0, tp=1)
    assert ident2 == ident
    assert w["layers"][0]["wq"].shape[0] == 4 * 64
    with pytest.raises(ValueError):          # 64-wide expert slices straddle the 128-wide scale blocks
        ck.load_rank_weights(spec, root, rank=1, tp=2)
    spec32 = tiny_spec("fp32")
    ck.write_target_checkpoint(str(tmp_path / "t32"), spec32, seed=3)
    w2, _ = ck.load_rank_weights(spec32, str(tmp_path / "t32"), rank=1, tp=2)
    assert w2["layers"][0]["wq"].shape[0] == 2 * 64 and w2["layers"][0]["gate"]["w"].shape == (9, 64, 256)


def test_pinned_identity_mismatch(tmp_path):
    spec = tiny_spec("fp32")
    a = ck.write_target_checkpoint(str(tmp_path / "a"), spec, seed=0)
    b = ck.write_target_checkpoint(str(tmp_path / "b"), tiny_spec("fp8"), seed=0)
    with pytest.raises(ck.CheckpointError):
        ck.load_rank_weights(spec, str(tmp_path / "a"), 0, 1, expect=b)
    ck.load_rank_weights(spec, str(tmp_path / "a"), 0, 1, expect=a)


def test_bad_header_rejected(tmp_path):
    p = tmp_path / "x.safetensors"
    hdr = json.dumps({"t": {"dtype": "F16", "shape": [2], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 4)
    with pytest.raises(ck.CheckpointError):
        ck.read_header(str(p))
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 4)
    with pytest.raises(ck.CheckpointError):
        ck.read_header(str(p))


def test_missing_tensor_detected(tmp_path):
    spec = tiny_spec("fp32")
    sd = init_state_dict(spec, 0)
    sd.pop("model.layers.1.self_attn.attention_sink_bias")
    ck.write_target_checkpoint(str(tmp_path / "t"), spec, state_dict=sd)
    with pytest.raises(ck.CheckpointError):
        ck.validate_target_layout(spec, ck.LocalCheckpoint(str(tmp_path / "t")))


def test_full_geometry_tensor_census():
    names = ck.expected_target_names(NAIVE_N0P5)
    counts = {}
    for dt in names.values():
        counts[dt] = counts.get(dt, 0) + 1
    # 47 MoE layers x 256 experts x 3 projections in e4m3, each with an fp32 block-scale tensor,
    # plus 47 routers and 47 correction biases in fp32 (the reference pins the same census).
    assert counts["F8_E4M3"] == 36096
    assert counts["F32"] == 36096 + 94
    assert sum(counts.values()) == 72664


def test_interleave_rope_matches_rotate_half():
    torch.manual_seed(0)
    heads, hd, rd, H = 2, 8, 4, 5
    w = torch.randn(heads * hd, H)
    x = torch.randn(H)
    y = (w @ x).reshape(heads, hd)
    ang = torch.tensor([0.3, 1.1])
    # rotate-half convention on the checkpoint order
    re, im = y[:, :2], y[:, 2:4]
    want_re, want_im = re * ang.cos() - im * ang.sin(), re * ang.sin() + im * ang.cos()
    yi = (interleave_rope(w, heads, hd, rd) @ x).reshape(heads, hd)
    got_re = yi[:, 0:4:2] * ang.cos() - yi[:, 1:4:2] * ang.sin()
    got_im = yi[:, 0:4:2] * ang.sin() + yi[:, 1:4:2] * ang.cos()
    assert torch.allclose(got_re, want_re, atol=1e-6) and torch.allclose(got_im, want_im, atol=1e-6)
    assert torch.equal(yi[:, rd:], y[:, rd:])


def test_tp_sharded_partials_recombine():
    spec = tiny_spec("fp32")
    w = prepare_weights(spec, init_state_dict(spec, 0))
    full = ReferenceModel(spec, w, tp=1, capacity=32)
    toks = torch.arange(8)
    want = full.step(toks, 0)
    # o_proj columns of both ranks tile the full matrix; lm_head rows tile the vocabulary
    s0, s1 = shard_weights(spec, w, 0, 2), shard_weights(spec, w, 1, 2)
    assert torch.equal(torch.cat((s0["lm_head"], s1["lm_head"])), w["lm_head"])
    assert torch.equal(torch.cat((s0["layers"][0]["wo"]["w"], s1["layers"][0]["wo"]["w"]), 1), w["layers"][0]["wo"]["w"])
    got = ReferenceModel(spec, w, tp=2, capacity=32).step(toks, 0)
    assert torch.allclose(got, want, atol=1e-4)


def test_draft_checkpoint(tmp_path):
    spec = tiny_spec("fp32")
    ck.write_draft_checkpoint(str(tmp_path / "d"), spec)
    w, _ = ck.load_draft_rank_weights(spec, str(tmp_path / "d"), rank=0, tp=2)
    assert w["fc"].shape == (256, 256)
    bad = tiny_spec("fp32")
    import dataclasses
    bad = dataclasses.replace(bad, draft=dataclasses.replace(bad.draft, markov_rank=16))
    with pytest.raises(ck.CheckpointError):
        ck.load_draft_rank_weights(bad, str(tmp_path / "d"), 0, 1)


def test_resolve_newest_step(tmp_path, monkeypatch):
    for s in ("step_5", "step_40"):
        os.makedirs(tmp_path / "run" / s)
    monkeypatch.setenv("NAIVERT_MODEL_ROOTS", str(tmp_path))
    assert ck.resolve_checkpoint("run").endswith("step_40")


def _same(a, b, path=""):
    if isinstance(a, dict):
        assert set(a) == set(b), path
        for k in a:
            _same(a[k], b[k], f"{path}.{k}")
    elif isinstance(a, (list, tuple)):
        assert len(a) == len(b), path
        for i, (x, y) in enumerate(zip(a, b)):
            _same(x, y, f"{path}[{i}]")
    elif isinstance(a, torch.Tensor):
        assert a.dtype == b.dtype and a.shape == b.shape, path
        x = a.view(torch.uint8) if a.dtype == torch.float8_e4m3fn else a
        y = b.view(torch.uint8) if b.dtype == torch.float8_e4m3fn else b
        assert torch.equal(x, y), path
    else:
        assert a == b, path


@pytest.mark.parametrize("tp", [1, 2, 4])
def test_sliced_rank_load_equals_shard_of_full(tmp_path, tp):
    """Reading only a rank's rows / columns from the shards gives exactly shard_weights(prepare_weights(full)),
    and touches a fraction of the checkpoint's bytes."""
    from naivert_b200.models.naive_n0p5 import small_w8a8_spec
    spec = small_w8a8_spec(2)
    root = str(tmp_path / "tgt")
    ck.write_target_checkpoint(root, spec, seed=5, shard_bytes=8 << 20)
    c = ck.LocalCheckpoint(root)
    full = prepare_weights(spec, c.load_tensors())
    total = sum(os.path.getsize(os.path.join(root, f)) for f in set(c.weight_map.values()))
    for rank in range(tp):
        rd = ck.SliceReader(c)
        got = ck.load_rank_weights_sliced(spec, c, rank, tp, reader=rd)
        _same(got, shard_weights(spec, full, rank, tp))
        if tp > 1:
            assert rd.bytes_read < 0.75 * total
        rd.close()


def test_header_rejects_overlapping_payload(tmp_path):
    p = tmp_path / "y.safetensors"
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                      "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 12)
    with pytest.raises(ck.CheckpointError):
        ck.read_header(str(p))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                      "b": {"dtype": "F32", "shape": [2], "data_offsets": [12, 20]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 20)
    with pytest.raises(ck.CheckpointError):
        ck.read_header(str(p))


def test_rank_tensor_abi_describes_the_sharded_weights():
    """The slot table computed from the specification alone matches what sharding real tensors produces, at every
    tensor-parallel degree, and a wrong slice is named by its slot."""
    import pytest
    import torch
    from naivert_b200.models import weights as W
    from naivert_b200.models.naive_n0p5 import small_w8a8_spec
    from naivert_b200.models.registry import resolve_model
    from naivert_b200.models.tensor_abi import RankTensorAbi, TensorSlot, check_rank_weights, rank_tensor_abi
    spec = small_w8a8_spec(4)
    full = W.prepare_weights(spec, W.init_state_dict(spec))
    for tp in (1, 2, 4, 8):
        for rank in {0, tp - 1}:
            w = W.shard_weights(spec, full, rank, tp)
            abi = check_rank_weights(spec, w, rank, tp)
            tensors = 0

            def count(d):
                nonlocal tensors
                for v in d.values() if isinstance(d, dict) else d:
                    if isinstance(v, (dict, list)):
                        count(v)
                    elif isinstance(v, torch.Tensor):
                        tensors += 1
            count(w)
            assert tensors == len(abi.domain("parameter"))             # nothing in the dictionary is undescribed
            assert abi.parameter_bytes == sum(s.nbytes for s in abi.slots if s.domain == "parameter") > 0
    w = W.shard_weights(spec, full, 1, 2)
    w["layers"][1]["gate"]["w"] = w["layers"][1]["gate"]["w"][:, :-128]
    with pytest.raises(ValueError, match=r"layers\.1\.gate\.w has shape"):
        check_rank_weights(spec, w, 1, 2)
    w = W.shard_weights(spec, full, 0, 2)
    del w["layers"][0]["iwq"]
    with pytest.raises(ValueError, match=r"layers\.0\.iwq is missing"):
        check_rank_weights(spec, w, 0, 2)
    w = W.shard_weights(spec, full, 0, 2)
    w["layers"][2]["wq"] = w["layers"][2]["wq"].float()
    with pytest.raises(ValueError, match="element type"):
        check_rank_weights(spec, w, 0, 2)
    # planning without tensors: the full model at 8 ranks, with a one-million-token context
    big = resolve_model("naive-n0.5")
    abi = rank_tensor_abi(big, 3, 8, capacity=1 << 20)
    assert 38e9 < abi.parameter_bytes < 45e9                           # ~40 GB of weights per rank
    assert 7e9 < abi.cache_bytes < 7.6e9                               # target KV + indexer keys (the draft adds ~2.7 GB)
    assert abi.slot("layers.1.gate.w").shape == (256, 256, 4096) and abi.slot("layers.0.ik").domain == "cache"
    assert [s.index for s in abi.domain("cache")] == list(range(len(abi.domain("cache"))))
    with pytest.raises(ValueError, match="unique"):
        RankTensorAbi("x", (TensorSlot("a", "parameter", 0, (1,), "bf16", 16, "row_major"),
                            TensorSlot("a", "parameter", 1, (1,), "bf16", 16, "row_major")))
    with pytest.raises(ValueError, match="cover"):
        RankTensorAbi("x", (TensorSlot("a", "cache", 1, (1,), "bf16", 16, "row_major"),))
    with pytest.raises(ValueError):
        rank_tensor_abi(big, 8, 8)


def test_list_weights_and_server_flags(tmp_path, monkeypatch, capsys):
    """``--list-weights`` prints the short names the resolver accepts; ``--checkpoint`` is the draft's second name and
    ``--output-capacity`` caps the per-request output."""
    import importlib.util
    import os
    from naivert_b200.models import checkpoint as ck
    models, drafts = tmp_path / "models", tmp_path / "drafts"
    (models / "flash" / "step_7").mkdir(parents=True)
    (models / "flash" / "step_12").mkdir()
    for d in (models / "flash" / "step_7", models / "flash" / "step_12"):
        (d / "config.json").write_text("{}")
        (d / ck.INDEX_NAME).write_text("{}")
    (models / "notes").mkdir()                                   # not a checkpoint
    (drafts / "markov-a").mkdir(parents=True)
    (drafts / "markov-a" / "config.json").write_text("{}")
    (drafts / "markov-a" / "model.safetensors").write_bytes(b"")
    monkeypatch.setenv("NAIVERT_MODEL_ROOTS", str(models))
    monkeypatch.setenv("NAIVERT_DRAFT_ROOTS", str(drafts) + ":" + str(tmp_path / "absent"))
    text = ck.list_weights()
    assert "flash" in text and text.count("step_12") == 1 and "step_7" not in text and "notes" not in text
    assert "markov-a" in text.split("drafts (--draft):")[1]
    assert ck.resolve_checkpoint("flash").endswith("step_12")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sp = importlib.util.spec_from_file_location("serve_sessions_cli", os.path.join(root, "examples", "serve_sessions.py"))
    cli = importlib.util.module_from_spec(sp)
    sp.loader.exec_module(cli)
    a = cli.parse_args(["--checkpoint", "markov-a", "--output-capacity", "4096", "--draft-ingest", "loop"])
    assert a.draft == "markov-a" and a.output_capacity == 4096 and a.draft_ingest == "loop"
    assert cli.main(["--list-weights"]) == 0
    assert "targets (--target):" in capsys.readouterr().out


def test_device_init_has_the_sharded_layout_and_replicates_what_must_be_equal():
    """The benchmark's weights are drawn per rank in the sharded layout: they fill the slot table of every TP degree,
    replicated tensors are identical on all ranks, sharded ones differ, and the draw is reproducible."""
    import torch
    from naivert_b200.models.device_init import init_draft_rank_weights_device, init_rank_weights_device
    from naivert_b200.models.naive_n0p5 import small_w8a8_spec
    from naivert_b200.models.tensor_abi import check_rank_weights
    from naivert_b200.models import weights as W
    spec = small_w8a8_spec(4)
    for tp in (1, 2, 4, 8):
        ws = [init_rank_weights_device(spec, r, tp, seed=0, device="cpu") for r in sorted({0, tp - 1})]
        for r, w in zip(sorted({0, tp - 1}), ws):
            check_rank_weights(spec, w, r, tp)
        if tp > 1:
            a, b = ws
            assert torch.equal(a["embed"], b["embed"]) and torch.equal(a["norm"], b["norm"])
            assert torch.equal(a["layers"][1]["router_w"], b["layers"][1]["router_w"])          # replicated
            assert torch.equal(a["layers"][0]["iwq"], b["layers"][0]["iwq"])
            assert not torch.equal(a["layers"][1]["wq"], b["layers"][1]["wq"])                   # sharded
            assert not torch.equal(a["lm_head"], b["lm_head"])
    again = init_rank_weights_device(spec, 1, 2, seed=0, device="cpu")
    first = init_rank_weights_device(spec, 1, 2, seed=0, device="cpu")
    assert torch.equal(again["layers"][2]["gate"]["w"].view(torch.uint8), first["layers"][2]["gate"]["w"].view(torch.uint8))
    other = init_rank_weights_device(spec, 1, 2, seed=5, device="cpu")
    assert not torch.equal(other["lm_head"], first["lm_head"])
    # the draft's device init has the structure of the sharded prepared draft weights
    dref = W.shard_draft_weights(spec, W.prepare_draft_weights(spec, W.init_draft_state_dict(spec)), 1, 2)
    ddev = init_draft_rank_weights_device(spec, 1, 2, device="cpu")

    def shapes(d, pre=""):
        out = {}
        for k, v in (d.items() if isinstance(d, dict) else enumerate(d)):
            if isinstance(v, (dict, list)):
                out.update(shapes(v, f"{pre}{k}."))
            elif isinstance(v, torch.Tensor):
                out[f"{pre}{k}"] = (tuple(v.shape), str(v.dtype))
        return out
    assert shapes(dref) == shapes(ddev)
