"""Per-rank block-draft runtime: context ingest (D12), the 8-row draft block (attention + MLP
per layer, every row-parallel projection fused with its all-reduce) and the Markov head that
emits seven proposals.

Parity: ``DraftCore`` (naivert/backends/naive_n0p5_draft.py:5-98: fc_ctx_kv, attn_rows8_swa, mlp,
head_markov), kernels naivert/body/dspark_{context,attention,mlp,head_markov}/, buffers
``DraftBuffers`` (naivert/models/naive_n0p5/dspark.py:144).
"""
from __future__ import annotations

from typing import List

import torch

from ..models.spec import ModelSpec
from ..ops import kernels as K
from .target import PAD_ROWS, TargetRuntime, _pad128

DRAFT_CALL_BASE = 200          # all-reduce call indices of the draft inside one round


class DraftRuntime:
    def __init__(self, spec: ModelSpec, draft_weights: dict, target: TargetRuntime, capacity: int, seed_buf, params_buf,
                 block_ids, pdl: bool = True):
        d = spec.draft
        if d.hidden != spec.hidden:
            raise ValueError("the draft shares the target LM head: hidden sizes must match")
        self.spec, self.d, self.t, self.fab, self.pdl = spec, d, target, target.fab, pdl
        self.tp, self.rank, dev = target.tp, target.rank, target.dev
        self.capacity = capacity
        bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
        Hd, hd = d.hidden, d.head_dim
        w = draft_weights
        self.rows = d.rows
        self.nh = d.head_count // self.tp
        self.nkv = max(1, d.kv_head_count // self.tp)
        self.I = d.intermediate // self.tp
        taps = len(d.target_layer_ids)
        self.kf = taps // self.tp * spec.hidden
        self.block_ids = block_ids
        self.ctrl = target.ctrl
        self.ctrl_ingest_pos = target.ctrl[2:]          # device view: [0] = first ingest position

        def dv(t):
            return t.to(dev).to(bf).contiguous()

        self.fc = dv(w["fc"])
        self.map_fc = K.weight_tmap(self.fc)
        self.hidden_norm, self.g_final, self.mask = dv(w["hidden_norm"]), dv(w["norm"]), dv(w["mask_embedding"])
        self.w1, self.w2 = dv(w["markov_w1"]), dv(w["markov_w2"])
        kv_rows = self.nkv * hd * 2
        wkv = torch.zeros(_pad128(d.layer_count * kv_rows), Hd, dtype=bf, device=dev)
        self.fused = target.fused
        # draft KV of all layers in one allocation: the context ingest appends every layer's rows from one GEMM epilogue
        self.kc = torch.zeros(d.layer_count, capacity, self.nkv, hd, dtype=bf, device=dev)
        self.vc = torch.zeros(d.layer_count, capacity, self.nkv, hd, dtype=bf, device=dev)
        self.k_norms = torch.stack([dv(lw["k_norm"]) for lw in w["layers"]]).contiguous()
        self.layers: List[dict] = []
        for l, lw in enumerate(w["layers"]):
            wkv[l * kv_rows:(l + 1) * kv_rows] = torch.cat([dv(lw["wk"]), dv(lw["wv"])])
            n = (self.nh + 2 * self.nkv) * hd
            wqkv = torch.zeros(_pad128(n), Hd, dtype=bf, device=dev)
            wqkv[:n] = torch.cat([dv(lw["wq"]), dv(lw["wk"]), dv(lw["wv"])])
            L = {"wqkv": wqkv, "map_qkv": K.weight_tmap(wqkv), "g_in": dv(lw["g_in"]), "g_post": dv(lw["g_post"]),
                 "q_norm": dv(lw["q_norm"]), "k_norm": dv(lw["k_norm"]),
                 "wo": dv(lw["wo"]), "gate": dv(lw["gate"]), "up": dv(lw["up"]), "down": dv(lw["down"]),
                 "k": self.kc[l], "v": self.vc[l]}
            for nme in ("wo", "gate", "up", "down"):
                L["map_" + nme] = K.weight_tmap(L[nme])
            self.layers.append(L)
        self.wkv, self.map_kv = wkv, K.weight_tmap(wkv)

        # ---- activations
        self.h = torch.zeros(PAD_ROWS, Hd, dtype=bf, device=dev)          # fc output / block residual
        self.xd = torch.zeros(PAD_ROWS, Hd, dtype=bf, device=dev)
        self.xn = torch.zeros(PAD_ROWS, Hd, dtype=bf, device=dev)
        self.map_xn = K.act_tmap(self.xn)
        self.raw = torch.zeros(PAD_ROWS, max(wkv.shape[0], self.layers[0]["wqkv"].shape[0]), dtype=f32, device=dev)
        self.q = torch.zeros(PAD_ROWS, self.nh, hd, dtype=bf, device=dev)
        self.k_blk = torch.zeros(PAD_ROWS, self.nkv, hd, dtype=bf, device=dev)
        self.v_blk = torch.zeros(PAD_ROWS, self.nkv, hd, dtype=bf, device=dev)
        self.o = torch.zeros(PAD_ROWS, self.nh * hd, dtype=bf, device=dev)
        self.map_o = K.act_tmap(self.o)
        self.y = torch.zeros(PAD_ROWS, self.I, dtype=bf, device=dev)
        self.map_y = K.act_tmap(self.y)
        self.attn_splits = 3
        # one 128-key chunk per CTA: the context window plus the block's own rows
        self.tc_splits = max(1, -(-(d.window + PAD_ROWS) // 128))
        self.attn_part = torch.zeros(max(PAD_ROWS * self.nh * self.attn_splits * (hd + 2),
                                         K.attn_decode_part_floats(PAD_ROWS, self.nkv, self.tc_splits)), dtype=f32, device=dev)
        self.attn_tickets = torch.zeros(PAD_ROWS * self.nh, dtype=i32, device=dev)
        self.rope_blk = torch.zeros(PAD_ROWS, hd // 2, 2, dtype=f32, device=dev)
        self.rope_ing = torch.zeros(PAD_ROWS, hd // 2, 2, dtype=f32, device=dev)
        feats = target.feats[:, self.rank * self.kf:(self.rank + 1) * self.kf]
        self.map_feats = K.act_tmap(feats)
        V = spec.vocab_shard(self.tp)
        self.dlogits = torch.zeros(PAD_ROWS, V, dtype=f32, device=dev)
        self.zq = torch.zeros(8, V, dtype=f32, device=dev)
        self.best = torch.zeros(8, dtype=torch.int64, device=dev)
        self.markov_sync = torch.zeros(2, dtype=torch.int64, device=dev)
        import os
        self.markov_chain = target.fused and os.environ.get("NAIVERT_MARKOV_CHAIN", "1") == "1"
        self.ticket = torch.zeros(1, dtype=i32, device=dev)
        self.seed_buf, self.params_buf = seed_buf, params_buf
        # per-tile sums of squares of h (fc output) and of the block residual xd for the fused RMSNorms
        self.ssq_h = torch.zeros(Hd // 128, PAD_ROWS, dtype=f32, device=dev)
        self.ssq_x = torch.zeros(Hd // 128, PAD_ROWS, dtype=f32, device=dev)
        self._build_args()

    def _g(self, n, k, rows):
        g = K.GemmArgs()
        g.n_total, g.k_total, g.rows, g.out_scale = n, k, rows, 1.0
        g.status = self.fab.status.data_ptr()
        return g

    def _build_args(self):
        d, R = self.d, self.rows
        Hd, hd = d.hidden, d.head_dim
        # ---- ingest
        g = self._g(Hd, self.kf, R)
        g.out_bf16, g.ld_out = self.h.data_ptr(), Hd
        g.fab = self.fab.fabric_args(DRAFT_CALL_BASE, Hd)
        g.ssq_out = self.ssq_h.data_ptr() if self.fused else None
        self.args_fc = g
        g = self._g(self.wkv.shape[0], Hd, R)
        g.out_f32, g.ld_out = self.raw.data_ptr(), self.raw.shape[1]
        kv_rows = self.nkv * hd * 2
        if self.fused:
            # RMSNorm(h) in the operand build; k-norm + RoPE + append of every layer in the epilogue
            g.n_total = d.layer_count * kv_rows
            g.nx, g.ngamma, g.nssq, g.neps = self.h.data_ptr(), self.hidden_norm.data_ptr(), self.ssq_h.data_ptr(), d.norm_eps
            p = g.post
            p.rows, p.pos0 = R, self.ctrl_ingest_pos.data_ptr()
            p.heads, p.kv_heads, p.head_dim, p.v_dim, p.rope_dim = 0, self.nkv, hd, hd, hd
            p.value_scale, p.rope = 1.0, self.rope_ing.data_ptr()
            p.k_cache, p.v_cache, p.ring = self.kc.data_ptr(), self.vc.data_ptr(), 0
            p.k_norm, p.norm_eps = self.k_norms.data_ptr(), d.norm_eps
            p.col_q, p.col_k, p.col_v = 0, 0, self.nkv * hd
            p.group_cols, p.norm_group_stride = kv_rows, hd
            p.k_group_stride = p.v_group_stride = self.capacity * self.nkv * hd
        self.args_kv = g
        for l, L in enumerate(self.layers):
            p = K.AttnPostArgs()
            p.qkv, p.ld, p.rows, p.pos0 = self.raw.data_ptr(), self.raw.shape[1], R, self.ctrl_ingest_pos.data_ptr()
            p.heads, p.kv_heads, p.head_dim, p.v_dim, p.rope_dim = 0, self.nkv, hd, hd, hd
            p.value_scale, p.rope = 1.0, self.rope_ing.data_ptr()
            p.k_cache, p.v_cache, p.ring = L["k"].data_ptr(), L["v"].data_ptr(), 0
            p.k_norm, p.norm_eps = L["k_norm"].data_ptr(), d.norm_eps
            p.col_q, p.col_k, p.col_v = 0, l * kv_rows, l * kv_rows + self.nkv * hd
            L["args_ingest_post"] = p
            # ---- block
            g = self._g(L["wqkv"].shape[0], Hd, R)
            g.out_f32, g.ld_out = self.raw.data_ptr(), self.raw.shape[1]
            L["args_qkv"] = g
            p = g.post if self.fused else K.AttnPostArgs()
            if self.fused:
                g.nx, g.ngamma, g.nssq, g.neps = self.xd.data_ptr(), L["g_in"].data_ptr(), self.ssq_x.data_ptr(), d.norm_eps
            p.qkv, p.ld, p.rows, p.pos0 = self.raw.data_ptr(), self.raw.shape[1], R, self.ctrl.data_ptr()
            p.heads, p.kv_heads, p.head_dim, p.v_dim, p.rope_dim = self.nh, self.nkv, hd, hd, hd
            p.value_scale, p.rope = 1.0, self.rope_blk.data_ptr()
            p.q_out, p.k_cache, p.v_cache, p.ring = self.q.data_ptr(), self.k_blk.data_ptr(), self.v_blk.data_ptr(), -1
            p.q_norm, p.k_norm, p.norm_eps = L["q_norm"].data_ptr(), L["k_norm"].data_ptr(), d.norm_eps
            p.col_q, p.col_k, p.col_v = 0, self.nh * hd, (self.nh + self.nkv) * hd
            L["args_post"] = p
            t = K.AttnArgs()
            t.q, t.k_cache, t.v_cache, t.pos0 = self.q.data_ptr(), L["k"].data_ptr(), L["v"].data_ptr(), self.ctrl.data_ptr()
            t.rows, t.heads, t.kv_heads, t.head_dim, t.v_dim = R, self.nh, self.nkv, hd, hd
            t.scale, t.mode, t.window, t.ring = hd ** -0.5, 2, d.window, 0
            t.k_blk, t.v_blk, t.o_bf16 = self.k_blk.data_ptr(), self.v_blk.data_ptr(), self.o.data_ptr()
            t.part, t.tickets = self.attn_part.data_ptr(), self.attn_tickets.data_ptr()
            L["args_attn"] = t
            L["attn_tc"] = self.fused and K.attn_decode_ok(t)
            g = self._g(Hd, self.nh * hd, R)
            g.out_bf16, g.ld_out, g.resid = self.xd.data_ptr(), Hd, self.xd.data_ptr()
            g.fab = self.fab.fabric_args(DRAFT_CALL_BASE + 1 + 2 * l, Hd)
            g.ssq_out = self.ssq_x.data_ptr() if self.fused else None
            L["args_o"] = g
            g = self._g(self.I, Hd, R)
            g.out_bf16, g.ld_out = self.y.data_ptr(), self.I
            if self.fused:
                g.nx, g.ngamma, g.nssq, g.neps = self.xd.data_ptr(), L["g_post"].data_ptr(), self.ssq_x.data_ptr(), d.norm_eps
            L["args_gu"] = g
            g = self._g(Hd, self.I, R)
            g.out_bf16, g.ld_out, g.resid = self.xd.data_ptr(), Hd, self.xd.data_ptr()
            g.fab = self.fab.fabric_args(DRAFT_CALL_BASE + 2 + 2 * l, Hd)
            g.ssq_out = self.ssq_x.data_ptr() if self.fused else None
            L["args_down"] = g
        g = self._g(self.t.lm_head.shape[0], Hd, R)
        g.out_f32, g.ld_out = self.dlogits.data_ptr(), self.dlogits.shape[1]
        self.args_head = g
        m = K.MarkovArgs()
        m.logits, m.ld = self.dlogits.data_ptr(), self.dlogits.shape[1]
        m.w1, m.w2, m.rank_dim = self.w1.data_ptr(), self.w2.data_ptr(), d.markov_rank
        V = self.spec.vocab_shard(self.tp)
        m.vlocal, m.vbase, m.vocab = V, self.rank * V, self.spec.vocab
        m.block_ids, m.zq = self.block_ids.data_ptr(), self.zq.data_ptr()
        m.params, m.seed, m.ctrl = self.params_buf.data_ptr(), self.seed_buf.data_ptr(), self.ctrl.data_ptr()
        m.best, m.ticket = self.best.data_ptr(), self.ticket.data_ptr()
        m.x = self.fab.xchg_args()
        self.args_markov = m
        pa = K.PrologueArgs()
        pa.tokens, pa.table, pa.mask = self.block_ids.data_ptr(), self.t.embed.data_ptr(), self.mask.data_ptr()
        pa.x, pa.ssq = self.xd.data_ptr(), self.ssq_x.data_ptr()
        pa.hidden, pa.rows, pa.vocab, pa.mode, pa.n_tabs = Hd, R, self.t.embed.shape[0], 1, 2
        pa.tab_pos0[0], pa.tab_dim[0], pa.tab_theta[0], pa.tab_out[0] = (self.ctrl_ingest_pos.data_ptr(), hd, d.rope_theta,
                                                                         self.rope_ing.data_ptr())
        pa.tab_pos0[1], pa.tab_dim[1], pa.tab_theta[1], pa.tab_out[1] = self.ctrl.data_ptr(), hd, d.rope_theta, self.rope_blk.data_ptr()
        self.args_prologue = pa

    V_STORE = K.gemm_variant(False, False, K.EPI_STORE_F32, K.GROUP_NONE)
    V_AR = K.gemm_variant(False, False, K.EPI_ALLREDUCE, K.GROUP_NONE)
    V_GU = K.gemm_variant(False, True, K.EPI_SILU_BF16, K.GROUP_NONE)
    V_QKV_POST = K.gemm_variant(False, False, K.EPI_QKV_POST, K.GROUP_NONE, K.B_NORM)
    V_GU_NORM = K.gemm_variant(False, True, K.EPI_SILU_BF16, K.GROUP_NONE, K.B_NORM)

    def ingest(self) -> None:
        """Draft KV for the (up to 8) feature rows the last target step produced, at positions
        ctrl[2].. ; rows beyond the committed count land beyond the context and are rewritten later."""
        d, R, pdl = self.d, self.rows, self.pdl
        if self.fused:
            # prologue: block input rows + both RoPE tables (the block that follows in a round reuses them; the
            # control words they depend on do not change before the round's tail)
            K.step_prologue(self.args_prologue, pdl=pdl)
            K.gemm(self.V_AR, self.map_fc, None, self.map_feats, self.args_fc, d.hidden // 128,
                   K.pick_split(d.hidden // 128, self.kf // 64), pdl=pdl)
            nt = self.wkv.shape[0] // 128
            K.gemm(self.V_QKV_POST, self.map_kv, None, None, self.args_kv, nt, K.norm_split(nt, d.hidden, False, False), pdl=pdl)
            return
        K.rope_table(self.ctrl_ingest_pos, R, d.head_dim, d.rope_theta, self.rope_ing, pdl=pdl)
        K.gemm(self.V_AR, self.map_fc, None, self.map_feats, self.args_fc, d.hidden // 128,
               K.pick_split(d.hidden // 128, self.kf // 64), pdl=pdl)
        K.prep_norm(self.h, self.hidden_norm, R, d.norm_eps, xn=self.xn, pdl=pdl)
        K.gemm(self.V_STORE, self.map_kv, None, self.map_xn, self.args_kv, self.wkv.shape[0] // 128,
               K.pick_split(self.wkv.shape[0] // 128, d.hidden // 64), pdl=pdl)
        for L in self.layers:
            K.attn_post(L["args_ingest_post"], pdl=pdl)

    def block(self, prologue: bool = False) -> None:
        d, R, pdl = self.d, self.rows, self.pdl
        if self.fused:
            if prologue:                   # standalone use (no ingest before it)
                K.step_prologue(self.args_prologue, pdl=pdl)
            for L in self.layers:
                nt = L["wqkv"].shape[0] // 128
                K.gemm(self.V_QKV_POST, L["map_qkv"], None, None, L["args_qkv"], nt, K.norm_split(nt, d.hidden, False, False), pdl=pdl)
                if L["attn_tc"]:
                    K.attn_decode(L["args_attn"], self.tc_splits, pdl=pdl)
                else:
                    K.attn_rows(L["args_attn"], self.attn_splits, pdl=pdl)
                K.gemm(self.V_AR, L["map_wo"], None, self.map_o, L["args_o"], d.hidden // 128,
                       K.pick_split(d.hidden // 128, self.nh * d.head_dim // 64), pdl=pdl)
                K.gemm(self.V_GU_NORM, L["map_gate"], L["map_up"], None, L["args_gu"], self.I // 128,
                       K.norm_split(self.I // 128, d.hidden, False, True), pdl=pdl)
                K.gemm(self.V_AR, L["map_down"], None, self.map_y, L["args_down"], d.hidden // 128,
                       K.pick_split(d.hidden // 128, self.I // 64), pdl=pdl)
            return
        K.draft_block_input(self.block_ids, self.t.embed, self.mask, self.xd, R, pdl=pdl)
        K.rope_table(self.ctrl, R, d.head_dim, d.rope_theta, self.rope_blk, pdl=pdl)
        for L in self.layers:
            K.prep_norm(self.xd, L["g_in"], R, d.norm_eps, xn=self.xn, pdl=pdl)
            K.gemm(self.V_STORE, L["map_qkv"], None, self.map_xn, L["args_qkv"], L["wqkv"].shape[0] // 128,
                   K.pick_split(L["wqkv"].shape[0] // 128, d.hidden // 64), pdl=pdl)
            K.attn_post(L["args_post"], pdl=pdl)
            K.attn_rows(L["args_attn"], self.attn_splits, pdl=pdl)
            K.gemm(self.V_AR, L["map_wo"], None, self.map_o, L["args_o"], d.hidden // 128,
                   K.pick_split(d.hidden // 128, self.nh * d.head_dim // 64), pdl=pdl)
            K.prep_norm(self.xd, L["g_post"], R, d.norm_eps, xn=self.xn, pdl=pdl)
            K.gemm(self.V_GU, L["map_gate"], L["map_up"], self.map_xn, L["args_gu"], self.I // 128, pdl=pdl)
            K.gemm(self.V_AR, L["map_down"], None, self.map_y, L["args_down"], d.hidden // 128,
                   K.pick_split(d.hidden // 128, self.I // 64), pdl=pdl)

    def propose(self) -> None:
        """Head logits of all rows, then seven sequential Markov / Gumbel-max steps."""
        d, R, pdl = self.d, self.rows, self.pdl
        K.prep_norm(self.xd, self.g_final, R, d.norm_eps, xn=self.xn, pdl=pdl)
        K.gemm(self.V_STORE, self.t.map_lm, None, self.map_xn, self.args_head, -(-self.t.lm_head.shape[0] // 128), pdl=pdl)
        if self.markov_chain and K.markov_chain(self.args_markov, d.block_size, self.markov_sync, pdl=pdl) == 0:
            return
        self.markov_chain = False
        for step in range(d.block_size):
            K.markov_step(self.args_markov, step, pdl=pdl)

    def kv_bytes(self) -> int:
        return sum(L[k].numel() * 2 for L in self.layers for k in ("k", "v"))
