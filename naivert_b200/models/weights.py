"""Logical (un-sharded) model weights, random initialisation and TP sharding.

The *state dict* uses the reference checkpoint's tensor names and dtypes
(naivert/models/naive_n0p5/checkpoint_fp8.py:125-147 and
naivert/models/naive_n0p5/dspark.py:64-113): attention / indexer / dense MLP / embeddings /
norms in BF16, routed experts in F8_E4M3 with an FP32 ``weight_scale_inv`` per 128x128 block,
router weight and ``e_score_correction_bias`` in FP32.

``prepare_weights`` applies the load-time transforms the reference applies
(checkpoint_fp8.py:39-47 ``interleave_rope``; :166-171,200-212 fp8 quantisation of o_proj
and the dense MLP) and returns plain nested dicts; ``shard_weights`` slices them for one
tensor-parallel rank (checkpoint_fp8.py:129-138,180-198).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops.quant import quantize_fp8_block
from .spec import FULL_DSA, DraftSpec, ModelSpec

StateDict = Dict[str, torch.Tensor]


# --------------------------------------------------------------------------- random init
def init_state_dict(spec: ModelSpec, seed: int = 0, std: float = 0.02, device="cpu") -> StateDict:
    """Random-init target checkpoint (weights N(0, std)), reference tensor names."""
    g = torch.Generator(device=device).manual_seed(seed)
    fp8 = spec.weight_dtype == "fp8"
    wdt = torch.bfloat16 if fp8 else torch.float32

    def rnd(*shape, s=std):
        return torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * s

    sd: StateDict = {}
    H = spec.hidden
    sd["model.embed_tokens.weight"] = rnd(spec.vocab, H).to(wdt)
    sd["model.norm.weight"] = (1.0 + rnd(H, s=0.05)).to(wdt)
    sd["lm_head.weight"] = rnd(spec.vocab, H).to(wdt)
    ix = spec.indexer
    rt = spec.routing

    def put_expert(prefix, n_out, n_in):
        w = rnd(n_out, n_in)
        if fp8:
            q, s = quantize_fp8_block(w)
            sd[prefix + ".weight"] = q
            sd[prefix + ".weight_scale_inv"] = s
        else:
            sd[prefix + ".weight"] = w

    for L, kind in enumerate(spec.layer_kinds):
        a = spec.attention[kind]
        p = f"model.layers.{L}."
        sd[p + "input_layernorm.weight"] = (1.0 + rnd(H, s=0.05)).to(wdt)
        sd[p + "post_attention_layernorm.weight"] = (1.0 + rnd(H, s=0.05)).to(wdt)
        sd[p + "self_attn.q_proj.weight"] = rnd(a.head_count * a.head_dim, H).to(wdt)
        sd[p + "self_attn.k_proj.weight"] = rnd(a.kv_head_count * a.head_dim, H).to(wdt)
        sd[p + "self_attn.v_proj.weight"] = rnd(a.kv_head_count * a.v_head_dim, H).to(wdt)
        sd[p + "self_attn.o_proj.weight"] = rnd(H, a.head_count * a.v_head_dim).to(wdt)
        if a.sink_bias:
            sd[p + "self_attn.attention_sink_bias"] = rnd(a.head_count, s=1.0).to(wdt)
        if kind == FULL_DSA:
            sd[p + "self_attn.indexer.wq.weight"] = rnd(ix.head_count * ix.head_dim, H).to(wdt)
            sd[p + "self_attn.indexer.wk.weight"] = rnd(ix.head_dim, H).to(wdt)
            sd[p + "self_attn.indexer.weights_proj.weight"] = rnd(ix.head_count, H).to(wdt)
            sd[p + "self_attn.indexer.k_norm.weight"] = (1.0 + rnd(ix.head_dim, s=0.05)).to(wdt)
            sd[p + "self_attn.indexer.k_norm.bias"] = rnd(ix.head_dim, s=0.05).to(wdt)
        if spec.is_dense(L):
            I = spec.dense_intermediate
            sd[p + "mlp.gate_proj.weight"] = rnd(I, H).to(wdt)
            sd[p + "mlp.up_proj.weight"] = rnd(I, H).to(wdt)
            sd[p + "mlp.down_proj.weight"] = rnd(H, I).to(wdt)
        else:
            sd[p + "mlp.gate.weight"] = rnd(rt.expert_count, H, s=0.03).float()
            if rt.score_func == "sigmoid":
                sd[p + "mlp.gate.e_score_correction_bias"] = rnd(rt.expert_count, s=0.05).float()
            for e in range(rt.expert_count):
                put_expert(p + f"mlp.experts.{e}.gate_proj", rt.intermediate, H)
                put_expert(p + f"mlp.experts.{e}.up_proj", rt.intermediate, H)
                put_expert(p + f"mlp.experts.{e}.down_proj", H, rt.intermediate)
            for s_ in range(rt.shared_expert_count):
                put_expert(p + f"mlp.shared_experts.{s_}.gate_proj", rt.intermediate, H)
                put_expert(p + f"mlp.shared_experts.{s_}.up_proj", rt.intermediate, H)
                put_expert(p + f"mlp.shared_experts.{s_}.down_proj", H, rt.intermediate)
    return sd


def init_draft_state_dict(spec: ModelSpec, seed: int = 1, std: float = 0.02, device="cpu") -> StateDict:
    """Random-init draft checkpoint in the reference's single-file layout."""
    d: DraftSpec = spec.draft
    g = torch.Generator(device=device).manual_seed(seed)
    wdt = torch.bfloat16 if spec.weight_dtype == "fp8" else torch.float32

    def rnd(*shape, s=std):
        return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * s).to(wdt)

    Hd = d.hidden
    sd: StateDict = {
        "fc.weight": rnd(Hd, len(d.target_layer_ids) * spec.hidden),
        "hidden_norm.weight": 1.0 + rnd(Hd, s=0.05),
        "norm.weight": 1.0 + rnd(Hd, s=0.05),
        "mask_embedding": rnd(Hd),
        "markov_head.markov_w1.weight": rnd(spec.vocab, d.markov_rank, s=0.1),
        "markov_head.markov_w2.weight": rnd(spec.vocab, d.markov_rank, s=0.1),
    }
    for i in range(d.layer_count):
        p = f"layers.{i}."
        sd[p + "input_layernorm.weight"] = 1.0 + rnd(Hd, s=0.05)
        sd[p + "post_attention_layernorm.weight"] = 1.0 + rnd(Hd, s=0.05)
        sd[p + "self_attn.q_proj.weight"] = rnd(d.head_count * d.head_dim, Hd)
        sd[p + "self_attn.k_proj.weight"] = rnd(d.kv_head_count * d.head_dim, Hd)
        sd[p + "self_attn.v_proj.weight"] = rnd(d.kv_head_count * d.head_dim, Hd)
        sd[p + "self_attn.o_proj.weight"] = rnd(Hd, d.head_count * d.head_dim)
        sd[p + "self_attn.q_norm.weight"] = 1.0 + rnd(d.head_dim, s=0.05)
        sd[p + "self_attn.k_norm.weight"] = 1.0 + rnd(d.head_dim, s=0.05)
        sd[p + "mlp.gate_proj.weight"] = rnd(d.intermediate, Hd)
        sd[p + "mlp.up_proj.weight"] = rnd(d.intermediate, Hd)
        sd[p + "mlp.down_proj.weight"] = rnd(Hd, d.intermediate)
    return sd


# --------------------------------------------------------------------------- load-time transforms
def interleave_rope(w: torch.Tensor, heads: int, head_dim: int, rope_dim: int) -> torch.Tensor:
    """Checkpoint rows store the rotary part of each head in rotate-half order
    (first half = real parts, second half = imaginary parts).  The kernels rotate
    *adjacent* pairs, so rows are re-ordered to (re0, im0, re1, im1, ...)."""
    rows = w.reshape(heads, head_dim, *w.shape[1:])
    half = rope_dim // 2
    rot = rows[:, :rope_dim]
    inter = torch.stack((rot[:, :half], rot[:, half:rope_dim]), dim=2).reshape(heads, rope_dim, *w.shape[1:])
    return torch.cat((inter, rows[:, rope_dim:]), dim=1).reshape(w.shape).contiguous()


def _q8(w: torch.Tensor, fp8: bool):
    if not fp8:
        return {"w": w.float(), "s": None}
    q, s = quantize_fp8_block(w.float())
    return {"w": q, "s": s}


def _expert(sd: StateDict, prefix: str, fp8: bool):
    w = sd[prefix + ".weight"]
    return {"w": w, "s": sd.get(prefix + ".weight_scale_inv") if fp8 else None}


def prepare_weights(spec: ModelSpec, sd: StateDict) -> dict:
    """State dict -> logical weights.  Linear weights become ``{"w": tensor, "s": scale|None}``;
    ``s`` is the 128x128 block scale for e4m3 weights."""
    fp8 = spec.weight_dtype == "fp8"
    ix, rt = spec.indexer, spec.routing
    out = {"embed": sd["model.embed_tokens.weight"], "norm": sd["model.norm.weight"],
           "lm_head": sd["lm_head.weight"], "layers": []}
    for L, kind in enumerate(spec.layer_kinds):
        a = spec.attention[kind]
        p = f"model.layers.{L}."
        lw = {
            "kind": kind,
            "g_in": sd[p + "input_layernorm.weight"],
            "g_post": sd[p + "post_attention_layernorm.weight"],
            "wq": interleave_rope(sd[p + "self_attn.q_proj.weight"], a.head_count, a.head_dim, a.rope_dim),
            "wk": interleave_rope(sd[p + "self_attn.k_proj.weight"], a.kv_head_count, a.head_dim, a.rope_dim),
            "wv": sd[p + "self_attn.v_proj.weight"],
            "wo": _q8(sd[p + "self_attn.o_proj.weight"], fp8),
            "sink": sd.get(p + "self_attn.attention_sink_bias"),
        }
        if kind == FULL_DSA:
            lw["iwq"] = interleave_rope(sd[p + "self_attn.indexer.wq.weight"], ix.head_count, ix.head_dim, ix.rope_dim)
            lw["iwk"] = interleave_rope(sd[p + "self_attn.indexer.wk.weight"], 1, ix.head_dim, ix.rope_dim)
            lw["iww"] = sd[p + "self_attn.indexer.weights_proj.weight"]
            # LayerNorm acts on the key *before* the rotation, in checkpoint channel order:
            # permute its affine parameters the same way as the rows of wk.
            lw["ik_w"] = interleave_rope(sd[p + "self_attn.indexer.k_norm.weight"], 1, ix.head_dim, ix.rope_dim)
            lw["ik_b"] = interleave_rope(sd[p + "self_attn.indexer.k_norm.bias"], 1, ix.head_dim, ix.rope_dim)
        if spec.is_dense(L):
            lw["dense"] = {n: _q8(sd[p + f"mlp.{n}_proj.weight"], fp8) for n in ("gate", "up", "down")}
        else:
            lw["router_w"] = sd[p + "mlp.gate.weight"].float()
            b = sd.get(p + "mlp.gate.e_score_correction_bias")
            lw["router_b"] = b.float() if b is not None else torch.zeros(rt.expert_count)
            for name in ("gate", "up", "down"):
                ws = [_expert(sd, p + f"mlp.experts.{e}.{name}_proj", fp8) for e in range(rt.expert_count)]
                ws += [_expert(sd, p + f"mlp.shared_experts.{s_}.{name}_proj", fp8)
                       for s_ in range(rt.shared_expert_count)]
                lw[name] = {"w": torch.stack([x["w"] for x in ws]),
                            "s": torch.stack([x["s"] for x in ws]) if fp8 else None}
        out["layers"].append(lw)
    return out


def prepare_draft_weights(spec: ModelSpec, sd: StateDict) -> dict:
    d = spec.draft
    sd = {(k[6:] if k.startswith("model.") else k): v for k, v in sd.items()}
    out = {"fc": sd["fc.weight"], "hidden_norm": sd["hidden_norm.weight"], "norm": sd["norm.weight"],
           "mask_embedding": sd["mask_embedding"],
           "markov_w1": sd["markov_head.markov_w1.weight"], "markov_w2": sd["markov_head.markov_w2.weight"],
           "layers": []}
    for i in range(d.layer_count):
        p = f"layers.{i}."
        out["layers"].append({
            "g_in": sd[p + "input_layernorm.weight"], "g_post": sd[p + "post_attention_layernorm.weight"],
            "wq": interleave_rope(sd[p + "self_attn.q_proj.weight"], d.head_count, d.head_dim, d.head_dim),
            "wk": interleave_rope(sd[p + "self_attn.k_proj.weight"], d.kv_head_count, d.head_dim, d.head_dim),
            "wv": sd[p + "self_attn.v_proj.weight"], "wo": sd[p + "self_attn.o_proj.weight"],
            "q_norm": interleave_rope(sd[p + "self_attn.q_norm.weight"], 1, d.head_dim, d.head_dim),
            "k_norm": interleave_rope(sd[p + "self_attn.k_norm.weight"], 1, d.head_dim, d.head_dim),
            "gate": sd[p + "mlp.gate_proj.weight"], "up": sd[p + "mlp.up_proj.weight"],
            "down": sd[p + "mlp.down_proj.weight"],
        })
    return out


# --------------------------------------------------------------------------- TP sharding
def _rows(w, rank, tp):
    n = w.shape[0] // tp
    return w[rank * n:(rank + 1) * n].contiguous()


def _slice_q8(q, dim, lo, hi, block=128):
    """Slice a (weight, block-scale) pair along ``dim`` (0 = out rows, 1 = in columns)."""
    w, s = q["w"], q["s"]
    idx = [slice(None)] * w.dim()
    idx[w.dim() - 2 + dim] = slice(lo, hi)
    ws = w[tuple(idx)].contiguous()
    if s is None:
        return {"w": ws, "s": None}
    if lo % block or (hi % block and hi != w.shape[w.dim() - 2 + dim]):
        raise ValueError(f"fp8 slice [{lo},{hi}) is not aligned to the {block}-wide scale blocks")
    sidx = [slice(None)] * s.dim()
    sidx[s.dim() - 2 + dim] = slice(lo // block, -(-hi // block))
    return {"w": ws, "s": s[tuple(sidx)].contiguous()}


def shard_weights(spec: ModelSpec, w: dict, rank: int, tp: int) -> dict:
    """Logical weights -> the slices rank ``rank`` of ``tp`` owns.

    q heads, o_proj columns, dense/expert intermediate channels and the vocabulary are split;
    KV heads are split while tp <= kv heads and shared beyond; the indexer, router, norms,
    sinks (by head) and the embedding table are replicated."""
    out = {"embed": w["embed"], "norm": w["norm"], "lm_head": _rows(w["lm_head"], rank, tp), "layers": []}
    for L, lw in enumerate(w["layers"]):
        a = spec.attention[lw["kind"]]
        nh = a.local_heads(tp)
        kvs = a.kv_head_for_rank(rank, tp)
        r = {"kind": lw["kind"], "g_in": lw["g_in"], "g_post": lw["g_post"]}
        r["wq"] = lw["wq"][rank * nh * a.head_dim:(rank + 1) * nh * a.head_dim].contiguous()
        r["wk"] = torch.cat([lw["wk"][h * a.head_dim:(h + 1) * a.head_dim] for h in kvs]).contiguous()
        r["wv"] = torch.cat([lw["wv"][h * a.v_head_dim:(h + 1) * a.v_head_dim] for h in kvs]).contiguous()
        r["wo"] = _slice_q8(lw["wo"], 1, rank * nh * a.v_head_dim, (rank + 1) * nh * a.v_head_dim)
        r["sink"] = None if lw["sink"] is None else lw["sink"][rank * nh:(rank + 1) * nh].contiguous()
        for k in ("iwq", "iwk", "iww", "ik_w", "ik_b"):
            if k in lw:
                r[k] = lw[k]
        if "dense" in lw:
            I = spec.dense_inter_local(tp)
            r["dense"] = {"gate": _slice_q8(lw["dense"]["gate"], 0, rank * I, (rank + 1) * I),
                          "up": _slice_q8(lw["dense"]["up"], 0, rank * I, (rank + 1) * I),
                          "down": _slice_q8(lw["dense"]["down"], 1, rank * I, (rank + 1) * I)}
        else:
            I = spec.expert_inter_local(tp)
            r["router_w"], r["router_b"] = lw["router_w"], lw["router_b"]
            r["gate"] = _slice_q8(lw["gate"], 0, rank * I, (rank + 1) * I)
            r["up"] = _slice_q8(lw["up"], 0, rank * I, (rank + 1) * I)
            r["down"] = _slice_q8(lw["down"], 1, rank * I, (rank + 1) * I)
        out["layers"].append(r)
    return out


def shard_expert_weights(spec: ModelSpec, w: dict, rank: int, tp: int) -> list:
    """Expert-parallel layout for prefill: rank ``rank`` holds ``expert_count / tp`` *whole* experts of every MoE
    layer (``None`` for dense layers).  Block scales ride along unchanged, so the values are those of the
    tensor-parallel slices.  Parity: naivert/prefill/operands.py ``load_expert_rank``."""
    E = spec.routing.expert_count
    if E % tp:
        raise ValueError(f"{E} experts do not divide over {tp} ranks")
    n = E // tp
    out = []
    for lw in w["layers"]:
        if "dense" in lw:
            out.append(None)
            continue
        out.append({name: {"w": lw[name]["w"][rank * n:(rank + 1) * n].contiguous(),
                           "s": lw[name]["s"][rank * n:(rank + 1) * n].contiguous()} for name in ("gate", "up", "down")})
    return out


def shard_draft_weights(spec: ModelSpec, w: dict, rank: int, tp: int) -> dict:
    d = spec.draft
    taps = len(d.target_layer_ids)
    if taps % tp:
        raise ValueError(f"{taps} feature taps do not split over tp={tp}")
    kf = taps // tp * spec.hidden
    nh = d.head_count // tp
    nkv = max(1, d.kv_head_count // tp)
    kv0 = rank * nkv if tp <= d.kv_head_count else rank // (tp // d.kv_head_count)
    I = d.intermediate // tp
    V = spec.vocab_shard(tp)
    out = {"fc": w["fc"][:, rank * kf:(rank + 1) * kf].contiguous(), "hidden_norm": w["hidden_norm"],
           "norm": w["norm"], "mask_embedding": w["mask_embedding"], "markov_w1": w["markov_w1"],
           "markov_w2": w["markov_w2"][rank * V:(rank + 1) * V].contiguous(), "layers": []}
    hd = d.head_dim
    for lw in w["layers"]:
        out["layers"].append({
            "g_in": lw["g_in"], "g_post": lw["g_post"], "q_norm": lw["q_norm"], "k_norm": lw["k_norm"],
            "wq": lw["wq"][rank * nh * hd:(rank + 1) * nh * hd].contiguous(),
            "wk": lw["wk"][kv0 * hd:(kv0 + nkv) * hd].contiguous(),
            "wv": lw["wv"][kv0 * hd:(kv0 + nkv) * hd].contiguous(),
            "wo": lw["wo"][:, rank * nh * hd:(rank + 1) * nh * hd].contiguous(),
            "gate": lw["gate"][rank * I:(rank + 1) * I].contiguous(),
            "up": lw["up"][rank * I:(rank + 1) * I].contiguous(),
            "down": lw["down"][:, rank * I:(rank + 1) * I].contiguous(),
        })
    return out
