"""Random-init weights generated directly on the device in the rank-sharded layout.

Full-size benchmark weights (hundreds of GB across the node) cannot pass through a CPU
checkpoint in reasonable time, so each rank draws its own shard on its GPU: replicated tensors
(embedding, norms, router, indexer, sinks) use a rank-independent seed and are identical on
every rank; sharded tensors use a rank-dependent seed.  e4m3 expert weights are drawn as
N(0, 96) codes with block scales around std/96, i.e. the distribution a block-quantised
N(0, std) matrix has.  The result has exactly the structure ``shard_weights`` produces.
"""
from __future__ import annotations

import torch

from .spec import FULL_DSA, ModelSpec


def _gen(seed: int, device) -> torch.Generator:
    return torch.Generator(device=device).manual_seed(seed)


def _randn(g, *shape, std=0.02, dtype=torch.bfloat16):
    return (torch.randn(*shape, generator=g, device=g.device, dtype=torch.float32) * std).to(dtype)


def _rand_q8(g, *shape, std=0.02, chunk_elems=1 << 28):
    """e4m3 tensor + 128x128 block scales [.., n/128, k/128] of an N(0, std) matrix."""
    dev = g.device
    out = torch.empty(*shape, dtype=torch.float8_e4m3fn, device=dev)
    flat = out.view(-1)
    n = flat.numel()
    for lo in range(0, n, chunk_elems):
        hi = min(n, lo + chunk_elems)
        flat[lo:hi] = (torch.randn(hi - lo, generator=g, device=dev, dtype=torch.float32) * 96.0).clamp_(-448, 448).to(
            torch.float8_e4m3fn)
    sshape = list(shape)
    sshape[-2], sshape[-1] = -(-shape[-2] // 128), -(-shape[-1] // 128)
    scale = (std / 96.0) * (1.0 + 0.1 * torch.rand(*sshape, generator=g, device=dev, dtype=torch.float32))
    return {"w": out, "s": scale}


def init_rank_weights_device(spec: ModelSpec, rank: int, tp: int, seed: int = 0, device="cuda", std: float = 0.02) -> dict:
    if spec.weight_dtype != "fp8":
        raise ValueError("device init implements the fp8 layout")
    H, ix, rt = spec.hidden, spec.indexer, spec.routing
    rep = _gen(seed * 1000003 + 17, device)                 # replicated tensors
    shd = _gen(seed * 1000003 + 101 + rank, device)         # this rank's shards
    V = spec.vocab_shard(tp)
    out = {"embed": _randn(rep, spec.vocab, H, std=std), "norm": 1.0 + _randn(rep, H, std=0.05),
           "lm_head": _randn(shd, V, H, std=std), "layers": []}
    for L, kind in enumerate(spec.layer_kinds):
        a = spec.attention[kind]
        nh, nkv = a.local_heads(tp), a.local_kv_heads(tp)
        # ranks that share a KV head must hold identical k/v rows
        kvg = _gen(seed * 1000003 + 5000 + L * 64 + a.kv_head_for_rank(rank, tp)[0], device)
        lw = {"kind": kind, "g_in": 1.0 + _randn(rep, H, std=0.05), "g_post": 1.0 + _randn(rep, H, std=0.05),
              "wq": _randn(shd, nh * a.head_dim, H, std=std), "wk": _randn(kvg, nkv * a.head_dim, H, std=std),
              "wv": _randn(kvg, nkv * a.v_head_dim, H, std=std),
              "wo": _rand_q8(shd, H, nh * a.v_head_dim, std=std),
              "sink": _randn(shd, nh, std=1.0) if a.sink_bias else None}
        if kind == FULL_DSA:
            lw["iwq"] = _randn(rep, ix.head_count * ix.head_dim, H, std=std)
            lw["iwk"] = _randn(rep, ix.head_dim, H, std=std)
            lw["iww"] = _randn(rep, ix.head_count, H, std=std)
            lw["ik_w"] = 1.0 + _randn(rep, ix.head_dim, std=0.05)
            lw["ik_b"] = _randn(rep, ix.head_dim, std=0.05)
        if spec.is_dense(L):
            I = spec.dense_inter_local(tp)
            lw["dense"] = {"gate": _rand_q8(shd, I, H, std=std), "up": _rand_q8(shd, I, H, std=std),
                           "down": _rand_q8(shd, H, I, std=std)}
        else:
            I = spec.expert_inter_local(tp)
            lw["router_w"] = _randn(rep, rt.expert_count, H, std=0.03, dtype=torch.float32)
            lw["router_b"] = _randn(rep, rt.expert_count, std=0.05, dtype=torch.float32)
            lw["gate"] = _rand_q8(shd, rt.expert_count, I, H, std=std)
            lw["up"] = _rand_q8(shd, rt.expert_count, I, H, std=std)
            lw["down"] = _rand_q8(shd, rt.expert_count, H, I, std=std)
        out["layers"].append(lw)
    return out


def init_expert_rank_weights_device(spec: ModelSpec, rank: int, tp: int, seed: int = 0, device="cuda", std: float = 0.02) -> list:
    """Whole experts of rank ``rank`` (expert-parallel prefill layout), one entry per layer (``None`` for dense
    layers).  Drawn independently of the tensor-parallel slices: a benchmark model, not a consistent one."""
    H, rt = spec.hidden, spec.routing
    g = _gen(seed * 1000003 + 9001 + rank, device)
    n, I = rt.expert_count // tp, rt.intermediate
    out = []
    for L in range(spec.layer_count):
        if spec.is_dense(L):
            out.append(None)
            continue
        out.append({"gate": _rand_q8(g, n, I, H, std=std), "up": _rand_q8(g, n, I, H, std=std),
                    "down": _rand_q8(g, n, H, I, std=std)})
    return out


def init_draft_rank_weights_device(spec: ModelSpec, rank: int, tp: int, seed: int = 1, device="cuda", std: float = 0.02) -> dict:
    d = spec.draft
    rep = _gen(seed * 1000003 + 23, device)
    shd = _gen(seed * 1000003 + 211 + rank, device)
    taps = len(d.target_layer_ids)
    kf = taps // tp * spec.hidden
    nh, nkv, I, V = d.head_count // tp, max(1, d.kv_head_count // tp), d.intermediate // tp, spec.vocab_shard(tp)
    kv0 = rank * nkv if tp <= d.kv_head_count else rank // (tp // d.kv_head_count)
    hd, Hd = d.head_dim, d.hidden
    out = {"fc": _randn(shd, Hd, kf, std=std), "hidden_norm": 1.0 + _randn(rep, Hd, std=0.05),
           "norm": 1.0 + _randn(rep, Hd, std=0.05), "mask_embedding": _randn(rep, Hd, std=std),
           "markov_w1": _randn(rep, spec.vocab, d.markov_rank, std=0.1),
           "markov_w2": _randn(shd, V, d.markov_rank, std=0.1), "layers": []}
    for l in range(d.layer_count):
        kvg = _gen(seed * 1000003 + 7000 + l * 64 + kv0, device)
        out["layers"].append({
            "g_in": 1.0 + _randn(rep, Hd, std=0.05), "g_post": 1.0 + _randn(rep, Hd, std=0.05),
            "q_norm": 1.0 + _randn(rep, hd, std=0.05), "k_norm": 1.0 + _randn(rep, hd, std=0.05),
            "wq": _randn(shd, nh * hd, Hd, std=std), "wk": _randn(kvg, nkv * hd, Hd, std=std),
            "wv": _randn(kvg, nkv * hd, Hd, std=std), "wo": _randn(shd, Hd, nh * hd, std=std),
            "gate": _randn(shd, I, Hd, std=std), "up": _randn(shd, I, Hd, std=std), "down": _randn(shd, Hd, I, std=std)})
    return out
