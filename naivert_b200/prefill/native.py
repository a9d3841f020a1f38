"""Chunked native prefill: whole chunks of prompt rows go through every layer in one pass.

A chunk of ``R`` rows (a multiple of 16, up to ``chunk``) is processed layer by layer with the same
kernels and caches as the decode/verify step, launched over row groups:

    RMSNorm -> q/k/v(/indexer) projection (tcgen05, grid.y = 16-row groups) -> RoPE / KV append /
    indexer keys -> [tcgen05 indexer sweep per row group -> exact top-k per row] -> row attention ->
    o_proj partials -> tensor-parallel reduction -> MoE -> draft feature ingest at the tap layers

Parallel layout (``tp`` ranks, one process per GPU):

* attention is tensor parallel (heads split, KV caches of this rank's heads), the partial o_proj
  outputs are reduced with NCCL: all-reduce for dense layers, reduce-scatter for MoE layers;
* with expert-parallel weights (``ep_weights``) the MoE rows are sequence parallel (``R / tp`` rows per
  rank) and the experts are whole and split over the ranks: count / dispatch / grouped GEMMs / return /
  combine run inside the kernels of ``EPMoE`` over peer memory, then the residual rows are all-gathered;
* without them every rank runs all rows through its intermediate slice of every expert (the same
  grouped kernels on a single-rank exchange) and the partial sums are all-reduced.

The caches it fills are the decode caches, so decoding continues from the chunk boundary
(``SpeculativeRound.initialize(start_pos=...)`` replays what is left of the prompt).

Parity: ``NativePrefill`` (naivert/prefill/native/executor.py: chunk body :479-537, ``run``,
``warm_chunks``, ``resume_from_decode``, ``close``), ``TPMoE`` (naivert/prefill/native/moe_tp.py),
``DraftFeaturePrefillExecutor`` (naivert/prefill/draft_features.py:24-103), chunk planning
(naivert/prefill/planning.py).
"""
from __future__ import annotations

import os
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..models.spec import FULL_DSA, ModelSpec
from ..ops import kernels as K
from ..runtime.target import LocalFabric, TargetRuntime
from .ep_moe import EPMoE, EPWeights

ROWS = K.K_TOK


@dataclass
class Chunk:
    pos0: int
    rows: int


def plan_chunks(start: int, end: int, chunk: int, quantum: int) -> List[Chunk]:
    """Split positions [start, end) into chunks of at most ``chunk`` rows; every chunk is a multiple of
    ``quantum`` rows, the remainder (< quantum) is left to the caller (prompt replay).
    Parity: naivert/prefill/planning.py (bucketed chunk plan)."""
    if chunk % quantum:
        raise ValueError(f"chunk {chunk} is not a multiple of {quantum}")
    out, p = [], start
    while end - p >= quantum:
        r = min(chunk, (end - p) // quantum * quantum)
        out.append(Chunk(p, r))
        p += r
    return out


class NativePrefill:
    V_BF16_F32 = K.gemm_variant(False, False, K.EPI_STORE_F32, K.GROUP_ITEM)
    V_BF16_BF16 = K.gemm_variant(False, False, K.EPI_STORE_BF16, K.GROUP_ITEM)
    V_FP8_BF16 = K.gemm_variant(True, False, K.EPI_STORE_BF16, K.GROUP_ITEM)
    V_FP8_GU = K.gemm_variant(True, True, K.EPI_SILU_QUANT, K.GROUP_ITEM)

    def __init__(self, spec: ModelSpec, target: TargetRuntime, draft=None, chunk: int = 4096,
                 ep_weights: Optional[list] = None, group=None):
        t = target
        self.spec, self.t, self.draft, self.group = spec, target, draft, group
        self.tp, self.rank, self.dev = t.fab.tp, t.fab.rank, t.dev
        if t.tp != t.fab.tp:
            raise ValueError("shape emulation has no peers to reduce with")
        self.ep = ep_weights is not None and self.tp > 1
        self.quantum = ROWS * (self.tp if self.ep else 1)
        if chunk % self.quantum or chunk < self.quantum:
            raise ValueError(f"chunk must be a multiple of {self.quantum}")
        if t.prefill_chunk < chunk:
            raise ValueError("the target's sliding-window rings were not sized for this chunk (prefill_chunk)")
        if FULL_DSA in spec.layer_kinds and not t.use_sweep:
            raise ValueError("the chunked indexer needs the tcgen05 sweep geometry (16 heads x 128)")
        self.C = C = chunk
        # 64-column chunk GEMM (a weight tile feeds 64 rows) unless NAIVERT_PREFILL_WIDE=0 or the chunk is not a
        # multiple of 64 rows; otherwise the step engine's 16-column tiles in item mode
        self.wide = os.environ.get("NAIVERT_PREFILL_WIDE", "1") == "1" and chunk % K.WIDE_TOK == 0
        self.step = K.WIDE_TOK if self.wide else ROWS
        self._gemm = self._wide_gemm if self.wide else K.gemm
        s, dev = spec, self.dev
        H = s.hidden
        bf, f32, i32, u8 = torch.bfloat16, torch.float32, torch.int32, torch.uint8
        self.pos = torch.zeros(4, dtype=i32, device=dev)                 # [0] = position of the chunk's row 0
        self.tokens = torch.zeros(C, dtype=i32, device=dev)
        self.x = torch.zeros(C, H, dtype=bf, device=dev)
        self.xn = torch.zeros(C, H, dtype=bf, device=dev)
        self.x8 = torch.zeros(C, H, dtype=u8, device=dev)
        self.xs = torch.ones(C, H // 128, dtype=f32, device=dev)
        self.part = torch.zeros(C, H, dtype=bf, device=dev)
        self.map_xn, self.map_x8 = K.act_tmap(self.xn, self.step), K.act_tmap(self.x8, self.step)
        self.qkv = torch.zeros(C, t.qkv.shape[1], dtype=f32, device=dev)
        self.q = torch.zeros(C, t.q.shape[1], t.q.shape[2], dtype=bf, device=dev)
        self.o8 = torch.zeros(C, t.o8.shape[1], dtype=u8, device=dev)
        self.os = torch.ones(C, t.os.shape[1], dtype=f32, device=dev)
        self.map_o8 = K.act_tmap(self.o8, self.step)
        self.rope = {k: torch.zeros(C, v.shape[1], 2, dtype=f32, device=dev) for k, v in t.rope.items()}
        self.idx_rope = torch.zeros(C, t.idx_rope.shape[1], 2, dtype=f32, device=dev)
        self.items = C // self.step
        self.row_offsets = (torch.arange(self.items, dtype=i32, device=dev) * self.step).contiguous()
        self.zero_ids = torch.zeros(self.items, dtype=i32, device=dev)
        self.n_items = torch.zeros(1, dtype=i32, device=dev)
        ix = s.indexer
        if FULL_DSA in s.layer_kinds:
            self.iq8 = torch.zeros(C * ix.head_count, ix.head_dim, dtype=u8, device=dev)
            self.ihw = torch.zeros(C, ix.head_count, dtype=f32, device=dev)
            self.idx_logits = torch.zeros(C, t.capacity, dtype=f32, device=dev)
            self.sel = torch.zeros(C, ix.top_k, dtype=i32, device=dev)
            # the indexer is replicated, so ranks split the query rows of a chunk for the sweep and the top-k and
            # all-gather the selection lists (NAIVERT_PREFILL_SHARD_INDEX=0: every rank selects for every row)
            self.shard_index = self.tp > 1 and os.environ.get("NAIVERT_PREFILL_SHARD_INDEX", "1") == "1"
            self.sel_local = torch.zeros(C // self.tp, ix.top_k, dtype=i32, device=dev) if self.shard_index else None
            self.topk_state = torch.zeros(C * K.topk_grid_state_bytes() // 4, dtype=i32, device=dev) if t.topk_grid else None
        if s.dense_layer_count:
            Id = s.dense_inter_local(self.tp)
            self.yd8 = torch.zeros(C, Id, dtype=u8, device=dev)
            self.yds = torch.ones(C, Id // 128, dtype=f32, device=dev)
            self.map_yd8 = K.act_tmap(self.yd8, self.step)
        # ---- MoE
        rt = s.routing
        self.T = C // self.tp if self.ep else C                            # rows a rank routes
        self.scores = torch.zeros(self.T, rt.expert_count, dtype=f32, device=dev)
        self.tickets = torch.zeros(-(-self.T // ROWS), dtype=i32, device=dev)
        self.topk_ids = torch.zeros(self.T, rt.top_k, dtype=i32, device=dev)
        self.topk_p = torch.zeros(self.T, rt.top_k, dtype=f32, device=dev)
        self.xl = torch.zeros(self.T, H, dtype=bf, device=dev)             # this rank's rows between scatter and gather
        self.rs = torch.zeros(self.T, H, dtype=bf, device=dev)
        self.zeros = torch.zeros(self.T, H, dtype=bf, device=dev) if (self.tp > 1 and not self.ep) else None
        has_moe = any("gate" in d for d in t.layers)
        self.moe_fab = t.fab if (self.ep or self.tp == 1) else LocalFabric(dev)
        self.moe: Optional[EPMoE] = None
        self.moe_w: List[Optional[EPWeights]] = []
        if has_moe:
            inter = rt.intermediate if self.ep else s.expert_inter_local(self.tp)
            self.moe = EPMoE(self.moe_fab, H, inter, rt.expert_count, rt.top_k, self.T, eps=s.norm_eps, item_rows=self.step)
            for L, d in enumerate(t.layers):
                if "gate" not in d:
                    self.moe_w.append(None)
                elif self.ep:
                    w = ep_weights[L]
                    self.moe_w.append(EPWeights(*({"w": w[n]["w"].to(dev), "s": w[n]["s"].to(dev)} for n in ("gate", "up", "down"))))
                else:
                    self.moe_w.append(EPWeights(*({"w": d[n].w, "s": d[n].s} for n in ("gate", "up", "down"))))
        # ---- draft feature ingest
        if draft is not None:
            taps = len(s.draft.target_layer_ids)
            Hd = s.draft.hidden
            self.feats = torch.zeros(C, max(1, taps) * H, dtype=bf, device=dev)
            self.map_feats = K.act_tmap(self.feats[:, self.rank * draft.kf:(self.rank + 1) * draft.kf], self.step)
            self.dh = torch.zeros(C, Hd, dtype=bf, device=dev)
            self.dxn = torch.zeros(C, Hd, dtype=bf, device=dev)
            self.map_dxn = K.act_tmap(self.dxn, self.step)
            self.draw = torch.zeros(C, draft.wkv.shape[0], dtype=f32, device=dev)
            self.drope = torch.zeros(C, s.draft.head_dim // 2, 2, dtype=f32, device=dev)
        self.phases: dict = {}
        # grouped-head attention kernel; NAIVERT_PREFILL_GROUP_ATTN=0 keeps the per-head row kernel of the step
        # path (bitwise-comparable with replay)
        self.group_attn = os.environ.get("NAIVERT_PREFILL_GROUP_ATTN", "1") == "1"
        self.profile = False                         # per-stage CUDA-event timing (adds an event pair per stage)
        self._timed: Dict[str, list] = {}
        self._build_args()

    @staticmethod
    def _wide_gemm(variant, a0, a1, b, args, n_tiles, items, pdl=False):
        """Plain projections share one weight matrix over all items.  A matrix that fits the L2 (126 MB) stays
        resident while feature tiles vary fastest (tokens stream once); a larger one is walked item-fastest so
        that each weight tile is fetched from HBM once and the (smaller) token operand stays resident instead."""
        wbytes = a0.tensor.numel() * a0.tensor.element_size() * (2 if a1 is not None else 1)
        K.wide_gemm(variant, a0, a1, b, args, n_tiles, items, pdl=pdl, items_fastest=wbytes > (96 << 20))

    # ------------------------------------------------------------------ argument blocks
    def _item_args(self, n, k) -> K.GemmArgs:
        g = K.GemmArgs()
        g.n_total, g.k_total, g.rows, g.a_group, g.out_scale = n, k, self.step, 0, 1.0
        g.n_active, g.active_ids, g.max_slots = self.n_items.data_ptr(), self.zero_ids.data_ptr(), self.items
        g.row_offsets = self.row_offsets.data_ptr()
        g.status = self.t.fab.status.data_ptr()
        return g

    def _build_args(self):
        s, t = self.spec, self.t
        H, ix = s.hidden, s.indexer
        pos0 = self.pos.data_ptr()
        self.L: List[dict] = []
        for L, d in enumerate(t.layers):
            a, nh, nkv, cols = d["a"], d["nh"], d["nkv"], d["cols"]
            e: dict = {}
            g = self._item_args(d["wqkv"].shape[0], H)
            g.out_f32, g.ld_out = self.qkv.data_ptr(), self.qkv.shape[1]
            e["qkv"] = g
            p = K.AttnPostArgs.from_buffer_copy(d["args_post"])
            p.qkv, p.ld, p.pos0, p.rope, p.q_out = self.qkv.data_ptr(), self.qkv.shape[1], pos0, self.rope[d["kind"]].data_ptr(), self.q.data_ptr()
            if d["kind"] == FULL_DSA:
                p.idx_rope_tab, p.iq8, p.ihw = self.idx_rope.data_ptr(), self.iq8.data_ptr(), self.ihw.data_ptr()
                # the step runtime keeps the query quantisation scale in a 16-row side buffer; a chunk has more rows,
                # so here the scale is folded into the head weights (the kernel's form without that buffer)
                p.iq_scale = None
                e["sweep_maps"] = K.sweep_maps(d["ik"], self.iq8)
                sw = K.SweepArgs()
                sw.ihw, sw.iks, sw.pos0 = self.ihw.data_ptr(), d["iks"].data_ptr(), pos0
                sw.heads, sw.top_k = ix.head_count, ix.top_k
                sw.logits, sw.ld, sw.status = self.idx_logits.data_ptr(), self.idx_logits.shape[1], t.fab.status.data_ptr()
                e["sweep"] = sw
            e["post"] = p
            q = K.AttnArgs.from_buffer_copy(d["args_attn"])
            q.q, q.pos0, q.o8, q.o_scale, q.part, q.tickets = self.q.data_ptr(), pos0, self.o8.data_ptr(), self.os.data_ptr(), None, None
            if d["kind"] == FULL_DSA:
                q.sel = self.sel.data_ptr()
            e["attn"] = q
            # one CTA per (KV head, row) shares every gathered key among the group's query heads
            e["group_attn"] = self.group_attn and a.head_dim == 192 and a.v_head_dim == 128 and nh // nkv <= 16
            g = self._item_args(H, d["wo"].k)
            g.w_scale0, g.a_scale = d["wo"].s.data_ptr(), self.os.data_ptr()
            g.out_bf16, g.ld_out = self.part.data_ptr(), H
            e["o"] = g
            if "dense" in d:
                dn = d["dense"]
                g = self._item_args(dn["gate"].n, H)
                g.w_scale0, g.w_scale1, g.a_scale = dn["gate"].s.data_ptr(), dn["up"].s.data_ptr(), self.xs.data_ptr()
                g.out_q, g.out_qscale = self.yd8.data_ptr(), self.yds.data_ptr()
                e["gu"] = g
                g = self._item_args(H, dn["down"].k)
                g.w_scale0, g.a_scale = dn["down"].s.data_ptr(), self.yds.data_ptr()
                g.out_bf16, g.ld_out = self.part.data_ptr(), H
                e["down"] = g
            else:
                rt = s.routing
                r = K.RouterArgs()
                r.w, r.bias, r.xn = None, d["router_b"].data_ptr(), self.xn.data_ptr()      # selection only (scores by torch.mm)
                if "router_wt" not in d:
                    d["router_wt"] = d["router_w"].float().t().contiguous()                 # [hidden][experts]
                r.hidden, r.experts, r.top_k = H, rt.expert_count, rt.top_k
                r.sigmoid, r.normalize, r.route_scale = int(rt.score_func == "sigmoid"), int(rt.normalize_top_k), rt.route_scale
                r.scores, r.ticket = self.scores.data_ptr(), self.tickets.data_ptr()
                r.topk_ids, r.topk_p, r.max_slots = self.topk_ids.data_ptr(), self.topk_p.data_ptr(), 0
                e["router"] = r
            self.L.append(e)
        if self.draft is not None:
            dr, dd = self.draft, s.draft
            g = self._item_args(dd.hidden, dr.kf)
            g.out_bf16, g.ld_out = self.dh.data_ptr(), dd.hidden
            self.args_fc = g
            g = self._item_args(dr.wkv.shape[0], dd.hidden)
            g.out_f32, g.ld_out = self.draw.data_ptr(), self.draw.shape[1]
            self.args_kv = g
            self.args_ingest = []
            for Ld in dr.layers:
                p = K.AttnPostArgs.from_buffer_copy(Ld["args_ingest_post"])
                p.qkv, p.ld, p.pos0, p.rope = self.draw.data_ptr(), self.draw.shape[1], pos0, self.drope.data_ptr()
                self.args_ingest.append(p)

    @contextmanager
    def _stage(self, name: str):
        if not self.profile:
            yield
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        yield
        b.record()
        self._timed.setdefault(name, []).append((a, b))

    def stage_ms(self) -> Dict[str, float]:
        """Device milliseconds per stage since the last call (``profile`` must be on); waits for the stream."""
        torch.cuda.current_stream().synchronize()
        out = {k: round(sum(a.elapsed_time(b) for a, b in v), 3) for k, v in self._timed.items()}
        self._timed = {}
        return out

    # ------------------------------------------------------------------ collectives (NCCL on the current stream)
    def _all_reduce(self, buf: torch.Tensor) -> None:
        if self.tp > 1:
            dist.all_reduce(buf, group=self.group)

    # ------------------------------------------------------------------ one chunk
    def _chunk(self, pos0: int, R: int) -> None:
        s, t, tp = self.spec, self.t, self.tp
        H, pdl = s.hidden, False
        items = -(-R // self.step)
        self.pos.fill_(pos0)
        if getattr(self, "shard_index", False) and R % (ROWS * tp) == 0:
            self.pos[1:2].fill_(pos0 + self.rank * (R // tp))
        self.n_items.fill_(items)
        x, xn, part = self.x, self.xn, self.part
        K.embed_rows(self.tokens, t.embed, x, R, pdl=pdl)
        for kind, tab in self.rope.items():
            a = s.attention[kind]
            K.rope_table(self.pos, R, a.rope_dim, a.rope_theta, tab, pdl=pdl)
        if FULL_DSA in self.rope:
            K.rope_table(self.pos, R, s.indexer.rope_dim, s.attention[FULL_DSA].rope_theta, self.idx_rope, pdl=pdl)
        T = R // tp if self.ep else R
        xl = x[self.rank * T:(self.rank + 1) * T] if self.ep else x[:R]
        for L, (d, e) in enumerate(zip(t.layers, self.L)):
            # ---- attention (tensor parallel)
            with self._stage("norm"):
                K.prep_norm(x, d["g_in"], R, s.norm_eps, xn=xn, pdl=pdl)
            with self._stage("qkv_gemm"):
                self._gemm(self.V_BF16_F32, d["map_qkv"], None, self.map_xn, e["qkv"], d["wqkv"].shape[0] // 128, items, pdl=pdl)
            e["post"].rows = R
            with self._stage("attn_post"):
                K.attn_post(e["post"], pdl=pdl)
            if d["kind"] == FULL_DSA and pos0 + R > s.indexer.top_k:
                sw = e["sweep"]
                sw.rows = R
                shard = self.shard_index and R % (ROWS * tp) == 0
                Rl = R // tp if shard else R                         # rows this rank selects for
                row0 = self.rank * Rl if shard else 0
                sw.group0, sw.ngroups = row0 // ROWS, Rl // ROWS
                tiles = -(-(pos0 + R) // 128)
                with self._stage("index_sweep"):
                    K.index_sweep(*e["sweep_maps"], sw, max(1, min(tiles, 592 // (Rl // ROWS))), pdl=pdl)
                with self._stage("topk"):
                    logits, pos_l = self.idx_logits[row0:row0 + Rl], self.pos[1:]          # pos[1] = pos0 + row0
                    sel = self.sel_local if shard else self.sel
                    if t.topk_grid:
                        K.topk_rows_grid(logits, pos_l, Rl, s.indexer.top_k, sel, self.topk_state, 16, pdl=pdl)
                    else:
                        K.topk_rows(logits, pos_l, Rl, s.indexer.top_k, sel, pdl=pdl)
                    if shard:
                        dist.all_gather_into_tensor(self.sel[:R], self.sel_local[:Rl], group=self.group)
            e["attn"].rows = R
            with self._stage("attn_dsa" if d["kind"] == FULL_DSA else "attn_swa"):
                if e["group_attn"]:
                    K.attn_group(e["attn"], pdl=pdl)
                else:
                    K.attn_rows(e["attn"], 1, pdl=pdl)
            with self._stage("o_gemm"):
                self._gemm(self.V_FP8_BF16, d["wo"].map, None, self.map_o8, e["o"], H // 128, items, pdl=pdl)
            moe = "dense" not in d
            with self._stage("tp_reduce"):
                if self.ep and moe:
                    # sequence parallel from here to the end of the layer: this rank keeps rows [rank*T, (rank+1)*T)
                    dist.reduce_scatter_tensor(self.rs[:T], part[:R], group=self.group)
                    torch.add(xl, self.rs[:T], out=self.xl[:T])
                else:
                    self._all_reduce(part[:R])
                    torch.add(x[:R], part[:R], out=x[:R])
            # ---- MLP
            if not moe:
                dn = d["dense"]
                with self._stage("dense_mlp"):
                    K.prep_norm(x, d["g_post"], R, s.norm_eps, x8=self.x8, xs=self.xs, pdl=pdl)
                    self._gemm(self.V_FP8_GU, dn["gate"].map, dn["up"].map, self.map_x8, e["gu"], dn["gate"].n // 128, items, pdl=pdl)
                    self._gemm(self.V_FP8_BF16, dn["down"].map, None, self.map_yd8, e["down"], H // 128, items, pdl=pdl)
                with self._stage("tp_reduce"):
                    self._all_reduce(part[:R])
                    torch.add(x[:R], part[:R], out=x[:R])
            else:
                src = self.xl if self.ep else x
                with self._stage("router"):
                    K.prep_norm(src, d["g_post"], T, s.norm_eps, xn=xn, pdl=pdl)
                    # scores of all chunk rows as one fp32 matrix product (library GEMM, no TF32: the same products as
                    # the step's FMA loop, summed in another order), selection by the router kernel per 16 rows
                    tf32 = torch.backends.cuda.matmul.allow_tf32
                    torch.backends.cuda.matmul.allow_tf32 = False
                    torch.mm(xn[:T].float(), d["router_wt"], out=self.scores[:T])
                    torch.backends.cuda.matmul.allow_tf32 = tf32
                    e["router"].rows = T
                    K.router(e["router"], pdl=pdl)
                self.moe.stage = self._stage if self.profile else None
                with self._stage("moe"):
                    if self.ep or tp == 1:
                        self.moe.run(src, d["g_post"], self.topk_ids, self.topk_p, src, src, weights=self.moe_w[L], tokens=T)
                    else:
                        self.moe.run(src, d["g_post"], self.topk_ids, self.topk_p, self.zeros, part, weights=self.moe_w[L], tokens=T)
                with self._stage("tp_reduce"):
                    if self.ep:
                        dist.all_gather_into_tensor(x[:R], src[:T], group=self.group)
                    elif tp > 1:
                        self._all_reduce(part[:R])
                        torch.add(x[:R], part[:R], out=x[:R])
            tap = t.tap_of_layer.get(L)
            if tap is not None and self.draft is not None:
                self.feats[:R, tap * H:(tap + 1) * H].copy_(x[:R])
        if self.draft is not None:
            with self._stage("draft_ingest"):
                self._ingest(R, items)

    def _ingest(self, R: int, items: int) -> None:
        """Draft context for the chunk's rows: fc over this rank's feature taps (reduced over the ranks),
        RMSNorm, every draft layer's k/v projection in one GEMM, k-norm + RoPE + append."""
        dr, dd, pdl = self.draft, self.spec.draft, False
        K.rope_table(self.pos, R, dd.head_dim, dd.rope_theta, self.drope, pdl=pdl)
        self._gemm(self.V_BF16_BF16, dr.map_fc, None, self.map_feats, self.args_fc, dd.hidden // 128, items, pdl=pdl)
        self._all_reduce(self.dh[:R])
        K.prep_norm(self.dh, dr.hidden_norm, R, dd.norm_eps, xn=self.dxn, pdl=pdl)
        self._gemm(self.V_BF16_F32, dr.map_kv, None, self.map_dxn, self.args_kv, dr.wkv.shape[0] // 128, items, pdl=pdl)
        for p in self.args_ingest:
            p.rows = R
            K.attn_post(p, pdl=pdl)

    # ------------------------------------------------------------------ public API
    def run(self, prompt: torch.Tensor, start: int = 0, end: Optional[int] = None) -> int:
        """Ingest prompt positions [start, end) in whole chunks on the current stream; returns the first
        position that was *not* ingested (the remainder, fewer than ``quantum`` rows, is left to replay).
        ``prompt`` may live in pinned host memory.  Caches before ``start`` must be valid."""
        n = int(prompt.numel())
        end = n if end is None else end
        if not 0 <= start <= end <= n or end > self.t.capacity:
            raise ValueError(f"prefill range [{start}, {end}) outside the prompt / cache capacity")
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        p = start
        chunks = plan_chunks(start, end, self.C, self.quantum)
        for c in chunks:
            self.tokens[:c.rows].copy_(prompt[c.pos0:c.pos0 + c.rows].to(torch.int32), non_blocking=True)
            self._chunk(c.pos0, c.rows)
            p = c.pos0 + c.rows
        ev1.record()
        self.phases = {"chunks": len(chunks), "rows": p - start, "events": (ev0, ev1)}
        return p

    def executor_ms(self) -> float:
        """Device time of the last ``run`` (waits for it)."""
        ev0, ev1 = self.phases["events"]
        ev1.synchronize()
        return ev0.elapsed_time(ev1)

    def warm_chunks(self, sizes=None) -> None:
        """Run every chunk size once on scratch positions so that module loading, kernel attributes and NCCL
        channels are paid before the first request.  The rows it writes into the caches start at position 0 and
        are overwritten by the next request."""
        for r in sorted(set(sizes or [self.quantum, self.C])):
            self.tokens.zero_()
            self._chunk(0, r)
        torch.cuda.current_stream().synchronize()
        self.check()

    def resume_from_decode(self, position: int) -> int:
        """A session that was decoding continues with a long new turn: every cache is position indexed (or a
        ring keyed by position), so chunks simply resume at ``position``; returns it for symmetry with the
        reference's executor (which rebuilds its swizzled shadows here)."""
        if not 0 <= position <= self.t.capacity:
            raise ValueError("resume position outside the cache")
        return position

    def check(self) -> None:
        self.t.fab.check()
        if self.moe_fab is not self.t.fab:
            self.moe_fab.check()

    def close(self) -> None:
        if self.moe_fab is not self.t.fab:
            self.moe_fab.close()
