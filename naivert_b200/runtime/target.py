"""Per-rank target runtime: packed weights, KV caches, scratch and the verify/decode step.

``TargetRuntime.step()`` enqueues one forward pass of ``rows`` consecutive token rows
(1 = seq-1 decode, 8 = verify, up to 16) on the current stream.  Nothing on that path
allocates or synchronises, positions and token ids live in device memory, so the same
call is captured into the CUDA graph of a speculative round.

Kernel sequence per layer: RMSNorm(+e4m3 packet) -> fused q/k/v(/indexer) projection
(tcgen05, bf16) -> RoPE / KV append / indexer quantisation -> [indexer logits -> exact top-k]
-> row attention (+ e4m3 packet of o) -> o_proj (tcgen05 fp8) fused with the tensor-parallel
all-reduce and residual -> RMSNorm -> router -> grouped gate/up (SiLU, e4m3 packet) -> grouped
down fused with probability weighting, all-reduce and residual.

Parity: ``RankRuntime.phases`` (tests/gpu/naive_n0p5_e2e/run_naive_n0p5_decode.py:327-440) and
``VerifyRuntime.phases`` (tests/gpu/naive_n0p5_e2e/run_naive_n0p5_verify.py:148-272); cache
layout naivert/models/naive_n0p5/checkpoint_fp8.py:254-260.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..models.spec import FULL_DSA, ModelSpec
from ..ops import kernels as K

PAD_ROWS = K.K_TOK


def _pad128(n: int) -> int:
    return -(-n // 128) * 128


def LocalFabric(device="cuda"):
    """Fabric of a single rank (tp = 1): status and epoch words, no peers."""
    from ..parallel.fabric import Fabric
    return Fabric(0, 1, 0, device=torch.device(device) if not isinstance(device, torch.device) else device)


class _Linear8:
    """Packed e4m3 weight (+ block scales) with its tensor map."""

    def __init__(self, q: dict, device):
        self.w = q["w"].to(device).contiguous()
        self.s = q["s"].to(device).float().contiguous()
        self.map = K.weight_tmap(self.w.view(torch.uint8))
        self.n, self.k = self.w.shape[-2], self.w.shape[-1]


class TargetRuntime:
    def __init__(self, spec: ModelSpec, rank_weights: dict, fabric, rows: int = 8, capacity: int = 16384,
                 device="cuda", pdl: bool = True, shape_tp: int = 0, prefill_chunk: int = 0):
        if spec.weight_dtype != "fp8":
            raise ValueError("the CUDA runtime implements the W8A8 recipe only")
        if spec.routing.shared_expert_count:
            raise ValueError("shared experts are only supported by the torch oracle")
        self.spec, self.fab, self.rows, self.capacity, self.dev, self.pdl = spec, fabric, rows, capacity, device, pdl
        # a chunked prefill appends `prefill_chunk` rows to a sliding-window ring in one launch: the ring must hold
        # the window of the chunk's first row and the whole chunk at once
        self.prefill_chunk = prefill_chunk
        # shape_tp > 1 with a single-rank fabric runs one rank's share of a tp-way model without peers
        # (kernel profiling of the per-rank shapes; the results are not a model output)
        self.tp, self.rank = (shape_tp, 0) if shape_tp else (fabric.tp, fabric.rank)
        # the router can normalise its own input (one launch fewer per MoE layer); measured slower on B200
        # (every CTA re-normalises all rows), so the separate RMSNorm kernel stays the default
        self.fuse_router_norm = False
        # fused step (default): RMSNorm inside the projections' operand build, q/k/v post-processing inside the
        # projection epilogue, one prologue launch.  NAIVERT_LEGACY_STEP=1 keeps the separate kernels (A/B timing).
        import os
        self.fused = os.environ.get("NAIVERT_LEGACY_STEP", "0") != "1"
        s = spec
        H = s.hidden
        dev = device
        bf, f32, i32, u8 = torch.bfloat16, torch.float32, torch.int32, torch.uint8

        # ---- control + step inputs
        self.ctrl = torch.zeros(16, dtype=i32, device=dev)          # [0] = position of row 0
        self.tokens = torch.zeros(PAD_ROWS, dtype=i32, device=dev)
        # ---- activations (16 padded rows)
        self.x = torch.zeros(PAD_ROWS, H, dtype=bf, device=dev)
        self.xn = torch.zeros(PAD_ROWS, H, dtype=bf, device=dev)
        self.x8 = torch.zeros(PAD_ROWS, H, dtype=u8, device=dev)
        self.xs = torch.ones(PAD_ROWS, H // 128, dtype=f32, device=dev)
        self.map_xn, self.map_x8 = K.act_tmap(self.xn), K.act_tmap(self.x8)
        rt = s.routing
        self.max_slots = min(rt.expert_count, PAD_ROWS * rt.top_k)
        self.step_slots = min(rt.expert_count, rows * rt.top_k)
        I = s.expert_inter_local(self.tp)
        Id = s.dense_inter_local(self.tp)
        self.y8 = torch.zeros(self.max_slots * PAD_ROWS, I, dtype=u8, device=dev)
        self.ys = torch.ones(self.max_slots * PAD_ROWS, max(1, I // 128), dtype=f32, device=dev)
        self.map_y8 = K.act_tmap(self.y8)
        if s.dense_layer_count:
            self.yd8 = torch.zeros(PAD_ROWS, Id, dtype=u8, device=dev)
            self.yds = torch.ones(PAD_ROWS, Id // 128, dtype=f32, device=dev)
            self.map_yd8 = K.act_tmap(self.yd8)
        self.scores = torch.zeros(PAD_ROWS, rt.expert_count, dtype=f32, device=dev)
        self.ticket = torch.zeros(1, dtype=i32, device=dev)
        self.n_active = torch.zeros(1, dtype=i32, device=dev)
        self.active_ids = torch.zeros(self.max_slots, dtype=i32, device=dev)
        self.probs = torch.zeros(self.max_slots, PAD_ROWS, dtype=f32, device=dev)
        self.topk_ids = torch.zeros(PAD_ROWS, rt.top_k, dtype=i32, device=dev)
        self.topk_p = torch.zeros(PAD_ROWS, rt.top_k, dtype=f32, device=dev)
        V = s.vocab_shard(self.tp)
        self.logits = torch.zeros(PAD_ROWS, V, dtype=f32, device=dev)
        taps = s.draft.target_layer_ids if s.draft is not None else ()
        if len(set(taps)) != len(taps):
            raise ValueError("draft feature taps must be distinct layers")
        # feature rows of all taps side by side: [16][taps * hidden] (the draft fc operand)
        self.feats = torch.zeros(PAD_ROWS, max(1, len(taps)) * H, dtype=bf, device=dev)
        self.tap_of_layer = {L: j for j, L in enumerate(taps)}

        # ---- weights
        w = rank_weights
        self.embed = w["embed"].to(dev).to(bf).contiguous()
        self.g_final = w["norm"].to(dev).to(bf).contiguous()
        self.lm_head = w["lm_head"].to(dev).to(bf).contiguous()
        self.map_lm = K.weight_tmap(self.lm_head)
        ix = s.indexer
        self.layers: List[dict] = []
        max_qkv = 0
        for L, lw in enumerate(w["layers"]):
            a = s.attention[lw["kind"]]
            nh, nkv = a.local_heads(self.tp), a.local_kv_heads(self.tp)
            parts = [lw["wq"], lw["wk"], lw["wv"]]
            cols = {"q": 0, "k": nh * a.head_dim, "v": nh * a.head_dim + nkv * a.head_dim}
            n = cols["v"] + nkv * a.v_head_dim
            if lw["kind"] == FULL_DSA:
                # indexer heads and the indexer key start on 128-feature tiles: the projection epilogue reduces
                # over one tile (quantisation scale, LayerNorm)
                pad = _pad128(n) - n
                if pad:
                    parts.append(torch.zeros(pad, H, dtype=bf, device=dev))
                n += pad
                cols["iq"], cols["ik"] = n, n + ix.head_count * ix.head_dim
                cols["iw"] = cols["ik"] + ix.head_dim
                parts += [lw["iwq"], lw["iwk"], lw["iww"]]
                n = cols["iw"] + ix.head_count
            wqkv = torch.zeros(_pad128(n), H, dtype=bf, device=dev)
            wqkv[:n] = torch.cat([p.to(dev).to(bf) for p in parts])
            max_qkv = max(max_qkv, wqkv.shape[0])
            d = {"kind": lw["kind"], "a": a, "nh": nh, "nkv": nkv, "cols": cols, "wqkv": wqkv,
                 "map_qkv": K.weight_tmap(wqkv), "g_in": lw["g_in"].to(dev).to(bf).contiguous(),
                 "g_post": lw["g_post"].to(dev).to(bf).contiguous(), "wo": _Linear8(lw["wo"], dev),
                 "sink": None if lw["sink"] is None else lw["sink"].to(dev).to(bf).contiguous()}
            if lw["kind"] == FULL_DSA:
                d["ik_w"] = lw["ik_w"].to(dev).to(bf).contiguous()
                d["ik_b"] = lw["ik_b"].to(dev).to(bf).contiguous()
                d["k"] = torch.zeros(capacity, nkv, a.head_dim, dtype=bf, device=dev)
                d["v"] = torch.zeros(capacity, nkv, a.v_head_dim, dtype=bf, device=dev)
                d["ik"] = torch.zeros(capacity, ix.head_dim, dtype=u8, device=dev)
                d["iks"] = torch.ones(capacity, dtype=f32, device=dev)
                d["ring"] = 0
            else:
                ring = a.sliding_window + max(PAD_ROWS, prefill_chunk)
                d["k"] = torch.zeros(ring, nkv, a.head_dim, dtype=bf, device=dev)
                d["v"] = torch.zeros(ring, nkv, a.v_head_dim, dtype=bf, device=dev)
                d["ring"] = ring
            if "dense" in lw:
                d["dense"] = {n_: _Linear8(lw["dense"][n_], dev) for n_ in ("gate", "up", "down")}
            else:
                d["router_w"] = lw["router_w"].to(dev).float().contiguous()
                d["router_b"] = lw["router_b"].to(dev).float().contiguous()
                d["gate"], d["up"], d["down"] = (_Linear8(lw[n_], dev) for n_ in ("gate", "up", "down"))
            self.layers.append(d)
        self.qkv = torch.zeros(PAD_ROWS, max_qkv, dtype=f32, device=dev)
        # sums of squares of the residual rows per 128-feature tile, left behind by whoever wrote the rows
        # (prologue, o_proj / down epilogues) for the RMSNorm fused into the next projection
        self.ssq = torch.zeros(H // 128, PAD_ROWS, dtype=f32, device=dev)
        # fused MoE block (router + gate/up + down + all-reduce in one launch): hand-off buffers shared by all layers
        import os as _os
        self.moe_fused = self.fused and _os.environ.get("NAIVERT_MOE_FUSED", "1") == "1" and rows <= 8
        # Routing runs inside the fused kernel (scores, grid-wide arrival, selection repeated per CTA): one launch per
        # MoE block, 4.43 ms per round at 8-way shapes against 4.52 ms with the router as its own launch in front
        # (NAIVERT_MOE_ROUTER_INSIDE=0), which stays available for A/B timing.
        self.moe_split_router = _os.environ.get("NAIVERT_MOE_ROUTER_INSIDE", "1") != "1"
        flag_words, part_floats = K.moe_scratch_sizes(H)
        self.moe_sync = torch.zeros(2, dtype=torch.int64, device=dev)
        self.moe_slot_flags = torch.zeros(flag_words, dtype=i32, device=dev)
        self.moe_part = torch.zeros(part_floats, dtype=f32, device=dev)
        self.moe_part_flags = torch.zeros(H // 128 * 4, dtype=i32, device=dev)
        a0 = s.attention[s.layer_kinds[0]]
        nh_max = max(s.attention[k].local_heads(self.tp) for k in set(s.layer_kinds))
        self.q = torch.zeros(PAD_ROWS, nh_max, a0.head_dim, dtype=bf, device=dev)
        self.o8 = torch.zeros(PAD_ROWS, nh_max * a0.v_head_dim, dtype=u8, device=dev)
        self.os = torch.ones(PAD_ROWS, nh_max * a0.v_head_dim // 128, dtype=f32, device=dev)
        self.map_o8 = K.act_tmap(self.o8)
        self.rope = {kind: torch.zeros(PAD_ROWS, s.attention[kind].rope_dim // 2, 2, dtype=f32, device=dev)
                     for kind in set(s.layer_kinds)}
        self.idx_rope = torch.zeros(PAD_ROWS, ix.rope_dim // 2, 2, dtype=f32, device=dev)
        if FULL_DSA in s.layer_kinds:
            self.iq8 = torch.zeros(PAD_ROWS * ix.head_count, ix.head_dim, dtype=u8, device=dev)
            self.ihw = torch.zeros(PAD_ROWS, ix.head_count, dtype=f32, device=dev)
            self.iq_scale = torch.ones(PAD_ROWS, ix.head_count, dtype=f32, device=dev)
            self.idx_logits = torch.zeros(PAD_ROWS, capacity, dtype=f32, device=dev)
            self.sel = torch.zeros(PAD_ROWS, ix.top_k, dtype=i32, device=dev)
            # long contexts select with many CTAs per row (six launches); short ones with one CTA per row
            self.topk_grid = capacity > 65536
            self.topk_state = torch.zeros(PAD_ROWS * K.topk_grid_state_bytes() // 4, dtype=i32, device=dev)
            self.use_sweep = ix.head_dim == 128 and ix.head_count % 16 == 0 and PAD_ROWS * ix.head_count == 256
        self.attn_splits = 4
        # tensor-core attention: 16 key splits for the 2048 selected keys of a full-attention row, one CTA per
        # (KV head, row) for a sliding window
        self.dsa_splits = 16
        kv_max = max(s.attention[k].local_kv_heads(self.tp) for k in set(s.layer_kinds))
        self.attn_part = torch.zeros(max(PAD_ROWS * nh_max * self.attn_splits * (a0.v_head_dim + 2),
                                         K.attn_decode_part_floats(PAD_ROWS, kv_max, self.dsa_splits)), dtype=f32, device=dev)
        self.attn_tickets = torch.zeros(PAD_ROWS * nh_max, dtype=i32, device=dev)
        # greedy arg-max over all ranks' vocabulary shards (seq-1 greedy decoding, sampler cross-check)
        self.greedy = torch.zeros(PAD_ROWS, dtype=i32, device=dev)
        self._argmax_keys = torch.zeros(PAD_ROWS, dtype=torch.int64, device=dev)
        self._argmax_ticket = torch.zeros(1, dtype=i32, device=dev)
        self._build_args()

    # ------------------------------------------------------------------ argument blocks (built once)
    def _gemm_args(self, n, k, rows) -> K.GemmArgs:
        g = K.GemmArgs()
        g.n_total, g.k_total, g.rows, g.a_group = n, k, rows, 0
        g.out_scale = 1.0
        g.status = self.fab.status.data_ptr()
        return g

    def _build_args(self):
        s, R = self.spec, self.rows
        H = s.hidden
        ix = s.indexer
        pos0 = self.ctrl.data_ptr()
        for L, d in enumerate(self.layers):
            a, nh, nkv, cols = d["a"], d["nh"], d["nkv"], d["cols"]
            g = self._gemm_args(d["wqkv"].shape[0], H, R)
            g.out_f32, g.ld_out = self.qkv.data_ptr(), self.qkv.shape[1]
            d["args_qkv"] = g
            p = g.post if self.fused else K.AttnPostArgs()
            if self.fused:
                g.nx, g.ngamma, g.nssq, g.neps = self.x.data_ptr(), d["g_in"].data_ptr(), self.ssq.data_ptr(), s.norm_eps
            p.qkv, p.ld, p.rows, p.pos0 = self.qkv.data_ptr(), self.qkv.shape[1], R, pos0
            p.heads, p.kv_heads, p.head_dim, p.v_dim, p.rope_dim = nh, nkv, a.head_dim, a.v_head_dim, a.rope_dim
            p.value_scale = a.value_scale
            p.rope = self.rope[d["kind"]].data_ptr()
            p.q_out, p.k_cache, p.v_cache, p.ring = self.q.data_ptr(), d["k"].data_ptr(), d["v"].data_ptr(), d["ring"]
            p.norm_eps = s.norm_eps
            p.col_q, p.col_k, p.col_v = cols["q"], cols["k"], cols["v"]
            if d["kind"] == FULL_DSA:
                p.idx_heads, p.idx_dim, p.idx_rope = ix.head_count, ix.head_dim, ix.rope_dim
                p.idx_rope_tab = self.idx_rope.data_ptr()
                p.ik_w, p.ik_b = d["ik_w"].data_ptr(), d["ik_b"].data_ptr()
                p.ln_eps, p.idx_weight_scale = s.norm_eps, ix.weight_scale
                p.iq8, p.ihw = self.iq8.data_ptr(), self.ihw.data_ptr()
                p.ik_cache, p.ik_scale = d["ik"].data_ptr(), d["iks"].data_ptr()
                p.col_iq, p.col_ik, p.col_iw = cols["iq"], cols["ik"], cols["iw"]
                p.iq_scale = self.iq_scale.data_ptr() if self.fused else None
                ia = K.IndexArgs()
                ia.iq_scale = p.iq_scale
                ia.iq8, ia.ihw, ia.ik, ia.iks, ia.pos0 = (self.iq8.data_ptr(), self.ihw.data_ptr(), d["ik"].data_ptr(),
                                                          d["iks"].data_ptr(), pos0)
                ia.rows, ia.heads, ia.dim, ia.top_k = R, ix.head_count, ix.head_dim, ix.top_k
                ia.logits, ia.ld = self.idx_logits.data_ptr(), self.idx_logits.shape[1]
                d["args_index"] = ia
                if self.use_sweep:
                    d["sweep_maps"] = K.sweep_maps(d["ik"], self.iq8)
                    sw = K.SweepArgs()
                    sw.ihw, sw.iks, sw.pos0 = self.ihw.data_ptr(), d["iks"].data_ptr(), pos0
                    sw.rows, sw.heads, sw.top_k = R, ix.head_count, ix.top_k
                    sw.logits, sw.ld, sw.status = self.idx_logits.data_ptr(), self.idx_logits.shape[1], self.fab.status.data_ptr()
                    sw.iq_scale = p.iq_scale
                    d["args_sweep"] = sw
            d["args_post"] = p
            t = K.AttnArgs()
            t.q, t.k_cache, t.v_cache, t.pos0 = self.q.data_ptr(), d["k"].data_ptr(), d["v"].data_ptr(), pos0
            t.rows, t.heads, t.kv_heads, t.head_dim, t.v_dim = R, nh, nkv, a.head_dim, a.v_head_dim
            t.scale = a.softmax_scale
            if a.sliding_window is not None:
                t.mode, t.window, t.ring = 0, a.sliding_window, d["ring"]
            else:
                t.mode, t.top_k, t.sel = 1, ix.top_k, self.sel.data_ptr()
            t.sink = None if d["sink"] is None else d["sink"].data_ptr()
            t.o8, t.o_scale = self.o8.data_ptr(), self.os.data_ptr()
            t.part, t.tickets = self.attn_part.data_ptr(), self.attn_tickets.data_ptr()
            d["args_attn"] = t
            d["attn_tc"] = self.fused and K.attn_decode_ok(t)
            # o_proj + all-reduce + residual
            g = self._gemm_args(H, d["wo"].k, R)
            g.w_scale0, g.a_scale = d["wo"].s.data_ptr(), self.os.data_ptr()
            g.out_bf16, g.ld_out, g.resid = self.x.data_ptr(), H, self.x.data_ptr()
            g.fab = self.fab.fabric_args(2 * L, H)
            g.ssq_out = self.ssq.data_ptr() if self.fused else None
            d["args_o"] = g
            tap = self.tap_of_layer.get(L)
            copy_ptr = None if tap is None else self.feats.data_ptr() + tap * H * 2
            if "dense" in d:
                dn = d["dense"]
                g = self._gemm_args(dn["gate"].n, H, R)
                g.w_scale0, g.w_scale1, g.a_scale = dn["gate"].s.data_ptr(), dn["up"].s.data_ptr(), self.xs.data_ptr()
                g.out_q, g.out_qscale = self.yd8.data_ptr(), self.yds.data_ptr()
                if self.fused:
                    g.nx, g.ngamma, g.nssq, g.neps = self.x.data_ptr(), d["g_post"].data_ptr(), self.ssq.data_ptr(), s.norm_eps
                d["args_gu"] = g
                g = self._gemm_args(H, dn["down"].k, R)
                g.w_scale0, g.a_scale = dn["down"].s.data_ptr(), self.yds.data_ptr()
                g.out_bf16, g.ld_out, g.resid = self.x.data_ptr(), H, self.x.data_ptr()
                g.out_copy, g.ld_copy = copy_ptr, self.feats.shape[1]
                g.fab = self.fab.fabric_args(2 * L + 1, H)
                g.ssq_out = self.ssq.data_ptr() if self.fused else None
                d["args_down"] = g
            else:
                rt = s.routing
                r = K.RouterArgs()
                r.w, r.bias = d["router_w"].data_ptr(), d["router_b"].data_ptr()
                if self.fused:                       # RMSNorm applied while the router reads the rows
                    r.xn, r.x, r.gamma, r.eps = None, self.x.data_ptr(), d["g_post"].data_ptr(), s.norm_eps
                    r.ssq = self.ssq.data_ptr()
                    r.x8, r.xs = self.x8.data_ptr(), self.xs.data_ptr()      # the packet the expert GEMMs read
                    d["router_fused"] = True
                else:
                    r.xn = self.xn.data_ptr()
                    d["router_fused"] = False
                r.hidden, r.experts, r.rows, r.top_k = H, rt.expert_count, R, rt.top_k
                r.sigmoid, r.normalize, r.route_scale = int(rt.score_func == "sigmoid"), int(rt.normalize_top_k), rt.route_scale
                r.scores, r.ticket = self.scores.data_ptr(), self.ticket.data_ptr()
                r.n_active, r.active_ids, r.probs = self.n_active.data_ptr(), self.active_ids.data_ptr(), self.probs.data_ptr()
                r.topk_ids, r.topk_p, r.max_slots = self.topk_ids.data_ptr(), self.topk_p.data_ptr(), self.max_slots
                d["args_router"] = r
                g = self._gemm_args(d["gate"].n, H, R)
                g.n_active, g.active_ids, g.max_slots = self.n_active.data_ptr(), self.active_ids.data_ptr(), self.max_slots
                g.w_scale0, g.w_scale1, g.a_scale = d["gate"].s.data_ptr(), d["up"].s.data_ptr(), self.xs.data_ptr()
                g.out_q, g.out_qscale = self.y8.data_ptr(), self.ys.data_ptr()
                d["args_gu"] = g
                g = self._gemm_args(H, d["down"].k, R)
                g.n_active, g.active_ids, g.probs, g.max_slots = (self.n_active.data_ptr(), self.active_ids.data_ptr(),
                                                                 self.probs.data_ptr(), self.max_slots)
                g.n_experts = rt.expert_count
                g.w_scale0, g.a_scale = d["down"].s.data_ptr(), self.ys.data_ptr()
                g.out_bf16, g.ld_out, g.resid = self.x.data_ptr(), H, self.x.data_ptr()
                g.out_copy, g.ld_copy = copy_ptr, self.feats.shape[1]
                g.fab = self.fab.fabric_args(2 * L + 1, H)
                g.ssq_out = self.ssq.data_ptr() if self.fused else None
                d["args_down"] = g
                if self.moe_fused:
                    m = K.MoeArgs()
                    m.r = d["args_router"]
                    if self.moe_split_router:          # the router kernel runs first; the fused kernel reads its lists
                        m.r.w = None
                    m.inter = d["gate"].n
                    m.gate_s, m.up_s, m.down_s = d["gate"].s.data_ptr(), d["up"].s.data_ptr(), d["down"].s.data_ptr()
                    m.y8, m.ys = self.y8.data_ptr(), self.ys.data_ptr()
                    m.sync, m.slot_flags = self.moe_sync.data_ptr(), self.moe_slot_flags.data_ptr()
                    m.part, m.part_flags = self.moe_part.data_ptr(), self.moe_part_flags.data_ptr()
                    m.ar = d["args_down"]
                    d["args_moe"] = m
        g = self._gemm_args(self.lm_head.shape[0], H, R)
        g.out_f32, g.ld_out = self.logits.data_ptr(), self.logits.shape[1]
        self.args_head = g
        # Weights of the next projection are requested into L2 by the kernel before it, at the point where that
        # kernel's own HBM stream is over: the q/k/v projection asks for o_proj's weights, the MoE block (or the dense
        # down projection) for the next layer's q/k/v weights.  NAIVERT_NEXT_WEIGHTS_L2=0 turns it off.
        import os
        if self.fused and os.environ.get("NAIVERT_NEXT_WEIGHTS_L2", "1") == "1":
            for L, d in enumerate(self.layers):
                wo = d["wo"].w
                d["args_qkv"].pf_ptr, d["args_qkv"].pf_bytes = wo.data_ptr(), wo.numel() * wo.element_size()
                if L + 1 < len(self.layers):
                    nq = self.layers[L + 1]["wqkv"]
                    tail = d["args_moe"].ar if "args_moe" in d else d["args_down"]
                    tail.pf_ptr, tail.pf_bytes = nq.data_ptr(), nq.numel() * nq.element_size()
        pa = K.PrologueArgs()
        pa.tokens, pa.table, pa.x, pa.ssq = self.tokens.data_ptr(), self.embed.data_ptr(), self.x.data_ptr(), self.ssq.data_ptr()
        pa.hidden, pa.rows, pa.vocab, pa.mode = H, R, self.embed.shape[0], 0
        tabs = [(s.attention[kind].rope_dim, s.attention[kind].rope_theta, tab) for kind, tab in self.rope.items()]
        if FULL_DSA in self.rope:
            tabs.append((ix.rope_dim, s.attention[FULL_DSA].rope_theta, self.idx_rope))
        pa.n_tabs = len(tabs)
        for i, (dim, theta, tab) in enumerate(tabs):
            pa.tab_pos0[i], pa.tab_dim[i], pa.tab_theta[i], pa.tab_out[i] = pos0, dim, theta, tab.data_ptr()
        self.args_prologue = pa

    # ------------------------------------------------------------------ the step
    V_FP8_STORE = K.gemm_variant(True, False, K.EPI_STORE_F32, K.GROUP_NONE)
    V_FP8_AR = K.gemm_variant(True, False, K.EPI_ALLREDUCE, K.GROUP_NONE)
    V_FP8_GU = K.gemm_variant(True, True, K.EPI_SILU_QUANT, K.GROUP_NONE)
    V_FP8_GU_ITEM = K.gemm_variant(True, True, K.EPI_SILU_QUANT, K.GROUP_ITEM)
    V_FP8_DOWN_LOOP = K.gemm_variant(True, False, K.EPI_ALLREDUCE, K.GROUP_LOOP)
    V_BF16_STORE = K.gemm_variant(False, False, K.EPI_STORE_F32, K.GROUP_NONE)
    V_QKV_POST = K.gemm_variant(False, False, K.EPI_QKV_POST, K.GROUP_NONE, K.B_NORM)
    V_FP8_GU_NORM = K.gemm_variant(True, True, K.EPI_SILU_QUANT, K.GROUP_NONE, K.B_NORM)
    V_FP8_GU_ITEM_NORM = K.gemm_variant(True, True, K.EPI_SILU_QUANT, K.GROUP_ITEM, K.B_NORM)

    def step(self, head: bool = True, stop_after=None) -> None:
        if not self.fused:
            return self._step_legacy(head, stop_after)
        s, R, pdl = self.spec, self.rows, self.pdl
        K.step_prologue(self.args_prologue, pdl=pdl)
        for L, d in enumerate(self.layers):
            nt = d["wqkv"].shape[0] // 128
            K.gemm(self.V_QKV_POST, d["map_qkv"], None, None, d["args_qkv"], nt, K.norm_split(nt, s.hidden, False, False), pdl=pdl)
            if d["kind"] == FULL_DSA:
                if self.use_sweep:
                    K.index_sweep(*d["sweep_maps"], d["args_sweep"], min(148, -(-self.capacity // 128)), pdl=pdl)
                else:
                    K.index_logits_simple(d["args_index"], 148, pdl=pdl)
                if self.topk_grid:
                    K.topk_rows_grid(self.idx_logits, self.ctrl, R, s.indexer.top_k, self.sel, self.topk_state, 16, pdl=pdl)
                else:
                    K.topk_rows(self.idx_logits, self.ctrl, R, s.indexer.top_k, self.sel, pdl=pdl)
            if d["attn_tc"]:
                K.attn_decode(d["args_attn"], self.dsa_splits if d["kind"] == FULL_DSA else 1, pdl=pdl)
            else:
                K.attn_rows(d["args_attn"], self.attn_splits if d["kind"] == FULL_DSA else 1, pdl=pdl)
            K.gemm(self.V_FP8_AR, d["wo"].map, None, self.map_o8, d["args_o"], s.hidden // 128,
                   K.pick_split(s.hidden // 128, d["wo"].k // 128), pdl=pdl)
            if stop_after == (L, "attn"):
                return
            if "dense" in d:
                dn = d["dense"]
                nt = dn["gate"].n // 128
                K.gemm(self.V_FP8_GU_NORM, dn["gate"].map, dn["up"].map, None, d["args_gu"], nt,
                       K.norm_split(nt, s.hidden, True, True, max_split=4), pdl=pdl)
                K.gemm(self.V_FP8_AR, dn["down"].map, None, self.map_yd8, d["args_down"], s.hidden // 128,
                       K.pick_split(s.hidden // 128, dn["down"].k // 128), pdl=pdl)
            elif self.moe_fused and self._moe_fused_layer(d, pdl):
                pass
            else:
                self.moe_fused = False           # geometry or occupancy does not fit the fused kernel: separate launches
                K.router(d["args_router"], pdl=pdl)
                K.gemm(self.V_FP8_GU_ITEM, d["gate"].map, d["up"].map, self.map_x8, d["args_gu"], d["gate"].n // 128,
                       self.step_slots, pdl=pdl)
                K.gemm(self.V_FP8_DOWN_LOOP, d["down"].map, None, self.map_y8, d["args_down"], s.hidden // 128,
                       K.pick_split(s.hidden // 128, 4), pdl=pdl)
        if head:
            K.prep_norm(self.x, self.g_final, R, s.norm_eps, xn=self.xn, pdl=pdl)
            K.gemm(self.V_BF16_STORE, self.map_lm, None, self.map_xn, self.args_head, -(-self.lm_head.shape[0] // 128), pdl=pdl)

    def _moe_fused_layer(self, d, pdl) -> bool:
        if self.moe_split_router:
            K.router(d["args_router"], pdl=pdl)
        return K.moe_layer(d["gate"].map, d["up"].map, d["down"].map, self.map_x8, self.map_y8, d["args_moe"], pdl=pdl) == 0

    def _step_legacy(self, head: bool = True, stop_after=None) -> None:
        s, R, pdl = self.spec, self.rows, self.pdl
        K.embed_rows(self.tokens, self.embed, self.x, R, pdl=pdl)
        for kind, tab in self.rope.items():
            a = s.attention[kind]
            K.rope_table(self.ctrl, R, a.rope_dim, a.rope_theta, tab, pdl=pdl)
        if FULL_DSA in self.rope:
            K.rope_table(self.ctrl, R, s.indexer.rope_dim, s.attention[FULL_DSA].rope_theta, self.idx_rope, pdl=pdl)
        for L, d in enumerate(self.layers):
            K.prep_norm(self.x, d["g_in"], R, s.norm_eps, xn=self.xn, pdl=pdl)
            nt = d["wqkv"].shape[0] // 128
            K.gemm(self.V_BF16_STORE, d["map_qkv"], None, self.map_xn, d["args_qkv"], nt, K.pick_split(nt, s.hidden // 64), pdl=pdl)
            K.attn_post(d["args_post"], pdl=pdl)
            if d["kind"] == FULL_DSA:
                if self.use_sweep:
                    K.index_sweep(*d["sweep_maps"], d["args_sweep"], min(148, -(-self.capacity // 128)), pdl=pdl)
                else:
                    K.index_logits_simple(d["args_index"], 148, pdl=pdl)
                if self.topk_grid:
                    K.topk_rows_grid(self.idx_logits, self.ctrl, R, s.indexer.top_k, self.sel, self.topk_state, 16, pdl=pdl)
                else:
                    K.topk_rows(self.idx_logits, self.ctrl, R, s.indexer.top_k, self.sel, pdl=pdl)
            K.attn_rows(d["args_attn"], self.attn_splits if d["kind"] == FULL_DSA else 1, pdl=pdl)
            K.gemm(self.V_FP8_AR, d["wo"].map, None, self.map_o8, d["args_o"], s.hidden // 128,
                   K.pick_split(s.hidden // 128, d["wo"].k // 128), pdl=pdl)
            if stop_after == (L, "attn"):
                return
            if "dense" in d:
                dn = d["dense"]
                K.prep_norm(self.x, d["g_post"], R, s.norm_eps, x8=self.x8, xs=self.xs, pdl=pdl)
                K.gemm(self.V_FP8_GU, dn["gate"].map, dn["up"].map, self.map_x8, d["args_gu"], dn["gate"].n // 128, pdl=pdl)
                K.gemm(self.V_FP8_AR, dn["down"].map, None, self.map_yd8, d["args_down"], s.hidden // 128,
                       K.pick_split(s.hidden // 128, dn["down"].k // 128), pdl=pdl)
            else:
                if not d["router_fused"]:
                    K.prep_norm(self.x, d["g_post"], R, s.norm_eps, xn=self.xn, x8=self.x8, xs=self.xs, pdl=pdl)
                K.router(d["args_router"], pdl=pdl)
                K.gemm(self.V_FP8_GU_ITEM, d["gate"].map, d["up"].map, self.map_x8, d["args_gu"], d["gate"].n // 128,
                       self.step_slots, pdl=pdl)
                K.gemm(self.V_FP8_DOWN_LOOP, d["down"].map, None, self.map_y8, d["args_down"], s.hidden // 128,
                       K.pick_split(s.hidden // 128, 4), pdl=pdl)
        if head:
            K.prep_norm(self.x, self.g_final, R, s.norm_eps, xn=self.xn, pdl=pdl)
            K.gemm(self.V_BF16_STORE, self.map_lm, None, self.map_xn, self.args_head, -(-self.lm_head.shape[0] // 128), pdl=pdl)

    ARGMAX_CALL = 60                                  # small-exchange call index (unique inside one epoch)

    def greedy_argmax(self) -> torch.Tensor:
        """Enqueue the tensor-parallel arg-max of the current logits rows; returns the device tensor that will hold
        the global token ids (identical on every rank).  Capturable; one exchange per epoch."""
        a = K.ArgmaxArgs()
        V = self.logits.shape[1]
        a.logits, a.ld, a.rows, a.vlocal, a.vbase = self.logits.data_ptr(), V, self.rows, V, self.rank * V
        a.tokens, a.keys, a.ticket = self.greedy.data_ptr(), self._argmax_keys.data_ptr(), self._argmax_ticket.data_ptr()
        a.call, a.x = self.ARGMAX_CALL, self.fab.xchg_args()
        K.argmax_rows(a, pdl=self.pdl)
        return self.greedy

    # ------------------------------------------------------------------ host helpers (not on the hot path)
    def set_inputs(self, tokens, pos0: int) -> None:
        t = torch.as_tensor(tokens, dtype=torch.int32)
        self.tokens[: t.numel()].copy_(t.to(self.dev))
        self.ctrl[0] = pos0

    def kv_bytes(self) -> int:
        n = 0
        for d in self.layers:
            for k in ("k", "v", "ik", "iks"):
                if k in d:
                    n += d[k].numel() * d[k].element_size()
        return n
