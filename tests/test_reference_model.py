"""CPU reference configuration: tiny random-init decoder, bitwise repeatability, verify == seq-1."""
import torch

from naivert_b200.models.naive_n0p5 import tiny_spec
from naivert_b200.models.reference import ReferenceDraft, ReferenceModel, topk_stable
from naivert_b200.models.weights import (init_draft_state_dict, init_state_dict, prepare_draft_weights,
                                         prepare_weights)


def _model(mode="fp32", tp=1):
    spec = tiny_spec(mode)
    w = prepare_weights(spec, init_state_dict(spec, seed=0))
    return spec, w, ReferenceModel(spec, w, tp=tp, capacity=640)


def test_tiny_decode_bitwise_repeatable():
    spec, w, m = _model()
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, spec.vocab, (512,), generator=g)
    t1, l1 = m.greedy_decode(prompt, 32)
    k1 = [k.clone() for k in m.k]
    t2, l2 = m.greedy_decode(prompt, 32)
    assert torch.equal(t1, t2)
    assert torch.equal(l1, l2)
    for a, b in zip(k1, m.k):
        assert torch.equal(a, b)
    # the sparse path was exercised (more keys visible than top_k)
    assert any(s is not None for s in m.last_selection[0])


def test_rows_equal_single_steps():
    spec, w, m = _model()
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, spec.vocab, (96,), generator=g)
    for i in range(0, 88, 8):
        m.step(toks[i:i + 8], i)
    block = m.step(toks[88:96], 88)
    m2 = ReferenceModel(spec, w, capacity=640)
    for i in range(0, 88, 8):
        m2.step(toks[i:i + 8], i)
    singles = torch.cat([m2.step(toks[88 + j:89 + j], 88 + j) for j in range(8)])
    assert torch.allclose(block, singles, atol=1e-5, rtol=1e-5)


def test_fp8_recipe_runs_and_tp_partials_close():
    spec = tiny_spec("fp8")
    # tiny dims are not multiples of 128 in K for experts (128 ok) / hidden 256 ok
    w = prepare_weights(spec, init_state_dict(spec, seed=0))
    g = torch.Generator().manual_seed(2)
    toks = torch.randint(0, spec.vocab, (16,), generator=g)
    a = ReferenceModel(spec, w, tp=1, capacity=64).step(toks, 0)
    b = ReferenceModel(spec, w, tp=1, capacity=64).step(toks, 0)
    assert torch.equal(a, b)
    assert torch.isfinite(a).all()


def test_topk_stable_ties_lowest_index():
    v = torch.tensor([1.0, 3.0, 3.0, 2.0, 3.0])
    assert topk_stable(v, 2).tolist() == [1, 2]
    assert topk_stable(v, 4).tolist() == [1, 2, 3, 4]


def test_draft_block_runs():
    spec = tiny_spec("fp32")
    w = prepare_weights(spec, init_state_dict(spec, seed=0))
    dw = prepare_draft_weights(spec, init_draft_state_dict(spec, seed=1))
    m = ReferenceModel(spec, w, capacity=64)
    toks = torch.arange(16) % spec.vocab
    _, feats = m.step(toks, 0, return_features=True)
    f = torch.cat([feats[i] for i in spec.draft.target_layer_ids], dim=-1)
    d = ReferenceDraft(spec, dw, w, capacity=64)
    d.ingest(f, 0)
    x = d.block(anchor=5, pos0=16)
    lg = d.head_logits(x)
    assert lg.shape == (8, spec.vocab) and torch.isfinite(lg).all()
    assert d.markov_bias(3).shape == (spec.vocab,)


def test_flagship_geometry_matches_the_golden_contract():
    """The geometry of the flagship model, written down once from the published description (layer pattern, head
    shapes, expert counts, draft block) and compared field by field: a change of any of them is a change of contract."""
    import json
    import os
    from naivert_b200.models.registry import resolve_model
    from naivert_b200.models.spec import FULL_DSA, SLIDING_WINDOW
    g = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "naive_n0p5_geometry.json")))
    s = resolve_model(g["name"])
    assert s.layer_count == g["layers"] and [i for i, k in enumerate(s.layer_kinds) if k == FULL_DSA] == g["full_dsa_layers"]
    assert all(k in (FULL_DSA, SLIDING_WINDOW) for k in s.layer_kinds)
    assert (s.hidden, s.vocab, s.vocab_shard(8), s.norm_eps) == (g["hidden"], g["vocab"], g["vocab_per_rank_tp8"], g["norm_eps"])
    assert list(s.stop_token_ids) == g["stop_token_ids"] and s.think_end_token_id == g["think_end_token_id"]
    assert s.precision_id == g["precision_id"] and s.weight_dtype == "fp8"
    for key, kind in (("dsa", FULL_DSA), ("swa", SLIDING_WINDOW)):
        a, w = s.attention[kind], g[key]
        assert (a.head_count, a.kv_head_count, a.head_dim, a.v_head_dim, a.rope_dim, a.rope_theta, a.sink_bias) == \
            (w["heads"], w["kv_heads"], w["head_dim"], w["v_head_dim"], w["rope_dim"], w["rope_theta"], w["sink_bias"])
    assert s.attention[FULL_DSA].value_scale == g["dsa"]["value_scale"] and s.attention[SLIDING_WINDOW].sliding_window == g["swa"]["window"]
    ix, w = s.indexer, g["indexer"]
    assert (ix.head_count, ix.head_dim, ix.rope_dim, ix.top_k) == (w["heads"], w["head_dim"], w["rope_dim"], w["top_k"])
    rt, w = s.routing, g["moe"]
    assert (rt.expert_count, rt.top_k, rt.score_func, rt.intermediate, rt.shared_expert_count, rt.route_scale, rt.normalize_top_k,
            rt.group_count) == (w["experts"], w["top_k"], w["score"], w["intermediate"], w["shared_experts"], w["route_scale"],
                                w["normalize_top_k"], w["groups"])
    assert (s.dense_layer_count, s.dense_intermediate, s.dense_inter_local(8)) == \
        (g["dense"]["layers"], g["dense"]["intermediate"], g["dense"]["intermediate_per_rank_tp8"])
    d, w = s.draft, g["draft"]
    assert (d.layer_count, d.hidden, d.head_count, d.kv_head_count, d.head_dim, d.intermediate, d.markov_rank, d.block_size,
            d.window, d.mask_token_id, list(d.target_layer_ids)) == \
        (w["layers"], w["hidden"], w["heads"], w["kv_heads"], w["head_dim"], w["intermediate"], w["markov_rank"], w["block_size"],
         w["window"], w["mask_token_id"], w["target_layer_ids"])
    t = g["tp8"]
    assert s.attention[FULL_DSA].local_heads(8) == t["q_heads_per_rank"] and s.expert_inter_local(8) == t["expert_intermediate_per_rank"]
    assert len(s.attention[FULL_DSA].kv_head_for_rank(3, 8)) == t["dsa_kv_heads_per_rank"]
    assert len(s.attention[SLIDING_WINDOW].kv_head_for_rank(3, 8)) == t["swa_kv_heads_per_rank"]
