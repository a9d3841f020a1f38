"""Torch oracle of the target and draft models with explicit rounding points.

This is the numerical contract every CUDA kernel is tested against and the whole
CPU reference configuration (fp32, no rounding).  It restates, on plain torch ops,
the math the reference pins in its own oracle
(tests/gpu/naive_n0p5_e2e/run_naive_n0p5_decode.py:442-591, tests/gpu/attn_dsa/run_attn_dsa.py:215-302,
naivert/models/naive_n0p5/training_moe.py) with the following recipe ("fp8" mode):

* RMSNorm in fp32, result rounded to bf16.
* q/k/v = bf16(x_norm @ W^T) (v scaled by ``value_scale`` before rounding); RoPE on adjacent
  pairs of the first ``rope_dim`` channels, rounded to bf16; softmax in fp32; o rounded to bf16.
* Every fp8 linear (o_proj, dense MLP, experts) quantises its activation to e4m3 with one
  power-of-two scale per 128-wide K block and promotes each K block in fp32.
* SiLU(gate)*up stays fp32 until it is quantised for the down projection.
* Each tensor-parallel rank rounds its partial of a row-parallel linear (o_proj, down,
  expert mixture) to bf16; partials are added in rank order in fp32, the residual is added
  in fp32 and the sum is rounded once to bf16.
* Experts of a token are accumulated in ascending expert-id order, shared experts last.
* Indexer: key = LayerNorm -> bf16 -> RoPE -> e4m3 with per-row scale amax/448; query e4m3 with
  a per-(row, head) scale folded into the head weights; logit = sum_h relu(q_h.k) w_h * k_scale;
  selection = top-k by (value desc, index asc); dense attention while <= top_k keys are visible.

In "fp32" mode every rounding and quantisation step is the identity.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from ..ops.quant import dequant_block, quantize_act_pow2, quantize_rows_e4m3
from .spec import FULL_DSA, ModelSpec


def rope_table(positions: torch.Tensor, rope_dim: int, theta: float) -> torch.Tensor:
    """[n] int positions -> [n, rope_dim/2, 2] (cos, sin), computed in fp64 then fp32."""
    i = torch.arange(rope_dim // 2, dtype=torch.float64, device=positions.device)
    inv = theta ** (-2.0 * i / rope_dim)
    ang = positions.double()[:, None] * inv[None, :]
    return torch.stack((ang.cos(), ang.sin()), dim=-1).float()


def apply_rope(x: torch.Tensor, table: torch.Tensor, rope_dim: int) -> torch.Tensor:
    """x [n, heads, dim]; rotates adjacent pairs (2i, 2i+1) of the first rope_dim channels."""
    xr = x[..., :rope_dim].float().reshape(*x.shape[:-1], rope_dim // 2, 2)
    c, s = table[:, None, :, 0], table[:, None, :, 1]
    re = xr[..., 0] * c - xr[..., 1] * s
    im = xr[..., 0] * s + xr[..., 1] * c
    rot = torch.stack((re, im), dim=-1).reshape(*x.shape[:-1], rope_dim)
    return torch.cat((rot, x[..., rope_dim:].float()), dim=-1)


def topk_stable(values: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k largest values, ties to the lowest index, returned ascending."""
    order = torch.sort(-values, stable=True).indices[:k]
    return torch.sort(order).values


class _Recipe:
    def __init__(self, mode: str):
        self.fp8 = mode == "fp8"

    def r(self, x: torch.Tensor) -> torch.Tensor:
        return x.to(torch.bfloat16).float() if self.fp8 else x.float()

    def rmsnorm(self, x, g, eps):
        xf = x.float()
        return self.r(xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * g.float())

    def linear(self, x, w):
        """bf16/fp32 weight linear with fp32 accumulation (no output rounding)."""
        return x.float() @ w.float().T

    def qlinear(self, x, q):
        """fp8 block-scaled linear in the W8A8 recipe (or plain fp32 when un-quantised)."""
        if q["s"] is None:
            return x.float() @ q["w"].float().T
        x8, xs = quantize_act_pow2(x)
        m, k = x8.shape
        kb = k // 128
        n = q["w"].shape[0]
        xa = x8.float().reshape(m, kb, 128)
        wa = q["w"].float().reshape(n, kb, 128)
        ws = q["s"].repeat_interleave(128, dim=0)[:n]
        out = torch.zeros(m, n, dtype=torch.float32, device=x.device)
        for b in range(kb):
            out = out + (xa[:, b] @ wa[:, b].T) * (xs[:, b, None] * ws[None, :, b])
        return out


def _slice_q(q, dim, lo, hi):
    w = q["w"]
    if dim == 0:
        return {"w": w[lo:hi], "s": None if q["s"] is None else q["s"][lo // 128: -(-hi // 128)]}
    return {"w": w[:, lo:hi], "s": None if q["s"] is None else q["s"][:, lo // 128: -(-hi // 128)]}


class ReferenceModel:
    """Target model oracle.  ``tp`` only moves the bf16 rounding of rank partials; it runs
    on one device.  Caches are plain growing tensors indexed by absolute position."""

    def __init__(self, spec: ModelSpec, weights: dict, tp: int = 1, capacity: int = 4096, device="cpu"):
        self.spec, self.w, self.tp = spec, weights, tp
        self.rc = _Recipe(spec.weight_dtype)
        self.device = device
        self.capacity = capacity
        self.reset()

    def reset(self):
        s = self.spec
        self.k: List[torch.Tensor] = []
        self.v: List[torch.Tensor] = []
        self.ik: List[Optional[torch.Tensor]] = []
        self.iks: List[Optional[torch.Tensor]] = []
        for L, kind in enumerate(s.layer_kinds):
            a = s.attention[kind]
            self.k.append(torch.zeros(self.capacity, a.kv_head_count, a.head_dim, device=self.device))
            self.v.append(torch.zeros(self.capacity, a.kv_head_count, a.v_head_dim, device=self.device))
            if kind == FULL_DSA:
                self.ik.append(torch.zeros(self.capacity, s.indexer.head_dim, device=self.device))
                self.iks.append(torch.ones(self.capacity, device=self.device))
            else:
                self.ik.append(None)
                self.iks.append(None)
        self.last_selection = {}
        self.trace = {}

    # ------------------------------------------------------------------ attention
    def _attention(self, L: int, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        s, rc, lw = self.spec, self.rc, self.w["layers"][L]
        a = s.attention[lw["kind"]]
        R = x.shape[0]
        xn = rc.rmsnorm(x, lw["g_in"], s.norm_eps)
        tab = rope_table(pos, a.rope_dim, a.rope_theta)
        q = rc.r(rc.linear(xn, lw["wq"])).reshape(R, a.head_count, a.head_dim)
        k = rc.r(rc.linear(xn, lw["wk"])).reshape(R, a.kv_head_count, a.head_dim)
        v = rc.r(rc.linear(xn, lw["wv"]) * a.value_scale).reshape(R, a.kv_head_count, a.v_head_dim)
        q = rc.r(apply_rope(q, tab, a.rope_dim))
        k = rc.r(apply_rope(k, tab, a.rope_dim))
        self.k[L][pos] = k
        self.v[L][pos] = v
        sel = None
        if lw["kind"] == FULL_DSA:
            sel = self._index_select(L, xn, pos, tab_positions=pos)
        group = a.head_count // a.kv_head_count
        o = torch.zeros(R, a.head_count, a.v_head_dim, device=x.device)
        for r in range(R):
            p = int(pos[r])
            if a.sliding_window is not None:
                keys = torch.arange(max(0, p - a.sliding_window + 1), p + 1, device=x.device)
            elif sel is not None and sel[r] is not None:
                keys = sel[r]
            else:
                keys = torch.arange(0, p + 1, device=x.device)
            kk = self.k[L][keys]            # [T, kvh, d]
            vv = self.v[L][keys]
            for h in range(a.head_count):
                g = h // group
                sc = (kk[:, g] @ q[r, h]) * a.softmax_scale
                if a.sink_bias:
                    sc = torch.cat((sc, lw["sink"][h].float().reshape(1)))
                pr = torch.softmax(sc.float(), dim=0)
                if a.sink_bias:
                    pr = pr[:-1]
                o[r, h] = pr @ vv[:, g]
        o = rc.r(o).reshape(R, a.head_count * a.v_head_dim)
        out = self._row_parallel(x, o, lw["wo"], a.head_count * a.v_head_dim)
        self.trace[(L, "q")], self.trace[(L, "o")], self.trace[(L, "attn")] = q, o, out
        return out

    def _index_select(self, L, xn, pos, tab_positions):
        s, rc, lw = self.spec, self.rc, self.w["layers"][L]
        ix = s.indexer
        a = s.attention[FULL_DSA]
        R = xn.shape[0]
        tab = rope_table(tab_positions, ix.rope_dim, a.rope_theta)
        iq = rc.r(rc.linear(xn, lw["iwq"])).reshape(R, ix.head_count, ix.head_dim)
        iq = rc.r(apply_rope(iq, tab, ix.rope_dim))
        kraw = rc.linear(xn, lw["iwk"])
        mu = kraw.mean(-1, keepdim=True)
        var = (kraw - mu).pow(2).mean(-1, keepdim=True)
        kn = rc.r((kraw - mu) * torch.rsqrt(var + s.norm_eps) * lw["ik_w"].float() + lw["ik_b"].float())
        kn = rc.r(apply_rope(kn[:, None, :], tab, ix.rope_dim))[:, 0]
        hw = rc.linear(xn, lw["iww"]) * ix.weight_scale            # [R, heads] fp32
        if rc.fp8:
            k8, ks = quantize_rows_e4m3(kn)
            q8, qs = quantize_rows_e4m3(iq)
            self.ik[L][pos] = k8.float()
            self.iks[L][pos] = ks
            iqv, hw = q8.float(), hw * qs
        else:
            self.ik[L][pos] = kn
            self.iks[L][pos] = torch.ones(R, device=xn.device)
            iqv = iq
        out = []
        for r in range(R):
            p = int(pos[r])
            if p + 1 <= ix.top_k:
                out.append(None)
                continue
            keys = self.ik[L][: p + 1]                               # [T, d]
            dots = torch.relu(torch.einsum("hd,td->ht", iqv[r], keys))
            logit = (dots * hw[r][:, None]).sum(0) * self.iks[L][: p + 1]
            out.append(topk_stable(logit, ix.top_k))
        self.last_selection[L] = out
        return out

    # ------------------------------------------------------------------ row-parallel helper
    def _row_parallel(self, resid, act, q, k_total):
        """bf16-rounded per-rank partials of act @ W^T (K split over ranks), fp32 rank-order
        sum plus residual, one bf16 rounding."""
        rc = self.rc
        kk = k_total // self.tp
        total = resid.float().clone()
        for rank in range(self.tp):
            part = rc.qlinear(act[:, rank * kk:(rank + 1) * kk], _slice_q(q, 1, rank * kk, (rank + 1) * kk))
            total = total + rc.r(part)
        return rc.r(total)

    # ------------------------------------------------------------------ MLP / MoE
    def _ffn_partial(self, xn, gate, up, down, lo, hi):
        rc = self.rc
        g = rc.qlinear(xn, _slice_q(gate, 0, lo, hi))
        u = rc.qlinear(xn, _slice_q(up, 0, lo, hi))
        y = torch.nn.functional.silu(g) * u
        return rc.qlinear(y, _slice_q(down, 1, lo, hi))

    def route(self, L, xn):
        rt, lw = self.spec.routing, self.w["layers"][L]
        sc = xn.float() @ lw["router_w"].float().T
        if rt.score_func == "sigmoid":
            score = torch.sigmoid(sc)
            choice = score + lw["router_b"].float()
        else:
            score = torch.softmax(sc, dim=-1)
            choice = score
        idx = torch.stack([torch.sort(-choice[r], stable=True).indices[: rt.top_k] for r in range(xn.shape[0])])
        p = torch.gather(score, 1, idx)
        if rt.normalize_top_k:
            p = p / (p.sum(-1, keepdim=True) + 1e-20)
        return idx, p * rt.route_scale

    def _mlp(self, L, x):
        s, rc, lw = self.spec, self.rc, self.w["layers"][L]
        xn = rc.rmsnorm(x, lw["g_post"], s.norm_eps)
        total = x.float().clone()
        if "dense" in lw:
            I = s.dense_intermediate // self.tp
            for rank in range(self.tp):
                d = lw["dense"]
                total = total + rc.r(self._ffn_partial(xn, d["gate"], d["up"], d["down"], rank * I, (rank + 1) * I))
            return rc.r(total)
        rt = s.routing
        idx, p = self.route(L, xn)
        self.trace[(L, "route")] = (idx, p)
        I = rt.intermediate // self.tp
        R = x.shape[0]
        for rank in range(self.tp):
            mix = torch.zeros(R, s.hidden, device=x.device)
            for r in range(R):
                order = torch.sort(idx[r]).indices
                for j in order.tolist():
                    e = int(idx[r, j])
                    ge = {"w": lw["gate"]["w"][e], "s": None if lw["gate"]["s"] is None else lw["gate"]["s"][e]}
                    ue = {"w": lw["up"]["w"][e], "s": None if lw["up"]["s"] is None else lw["up"]["s"][e]}
                    de = {"w": lw["down"]["w"][e], "s": None if lw["down"]["s"] is None else lw["down"]["s"][e]}
                    mix[r] = mix[r] + p[r, j] * self._ffn_partial(xn[r:r + 1], ge, ue, de, rank * I, (rank + 1) * I)[0]
                for sh in range(rt.shared_expert_count):
                    e = rt.expert_count + sh
                    ge = {"w": lw["gate"]["w"][e], "s": None if lw["gate"]["s"] is None else lw["gate"]["s"][e]}
                    ue = {"w": lw["up"]["w"][e], "s": None if lw["up"]["s"] is None else lw["up"]["s"][e]}
                    de = {"w": lw["down"]["w"][e], "s": None if lw["down"]["s"] is None else lw["down"]["s"][e]}
                    mix[r] = mix[r] + self._ffn_partial(xn[r:r + 1], ge, ue, de, rank * I, (rank + 1) * I)[0]
            total = total + rc.r(mix)
        return rc.r(total)

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, tokens: torch.Tensor, pos0: int, return_features: bool = False):
        """Run ``R`` consecutive rows (tokens at positions pos0..pos0+R-1).  Returns fp32
        logits [R, vocab] (and the residual stream after each layer when asked)."""
        s, rc = self.spec, self.rc
        R = tokens.shape[0]
        pos = torch.arange(pos0, pos0 + R, device=self.device)
        x = rc.r(self.w["embed"][tokens].float())
        feats = []
        for L in range(s.layer_count):
            x = self._attention(L, x, pos)
            x = self._mlp(L, x)
            feats.append(x)
        xn = rc.rmsnorm(x, self.w["norm"], s.norm_eps)
        logits = rc.linear(xn, self.w["lm_head"])
        if return_features:
            return logits, feats
        return logits

    @torch.no_grad()
    def greedy_decode(self, prompt: torch.Tensor, n: int, chunk: int = 8):
        """Prompt ingestion in ``chunk``-row steps followed by ``n`` greedy tokens."""
        self.reset()
        logits = None
        for i in range(0, prompt.shape[0], chunk):
            logits = self.step(prompt[i:i + chunk], i)
        out, all_logits = [], []
        p = prompt.shape[0]
        tok = int(logits[-1].argmax())
        for _ in range(n):
            out.append(tok)
            logits = self.step(torch.tensor([tok], device=self.device), p)
            all_logits.append(logits[0])
            p += 1
            tok = int(logits[0].argmax())
        return torch.tensor(out), torch.stack(all_logits)


class ReferenceDraft:
    """Block-draft oracle (bf16 everywhere in fp8 mode, fp32 otherwise).

    Context: target features of committed positions go through ``fc`` + ``hidden_norm`` and
    each layer's K/V projection (k-norm + RoPE) into the draft KV.  A block of ``rows`` rows
    (row 0 = embedding of the anchor token, the others the mask embedding) at positions
    pos0..pos0+rows-1 attends to the last ``window`` context positions before pos0 and to all
    block rows; rows 0..block_size-1 produce the proposal logits (plus the low-rank Markov
    bias of the previous token).  Reference: naivert/body/dspark_{context,attention,mlp,
    head_markov}/ and naivert/backends/naive_n0p5_draft.py:35-88."""

    def __init__(self, spec: ModelSpec, dw: dict, target_w: dict, tp: int = 1, capacity: int = 4096, device="cpu"):
        self.spec, self.d, self.w, self.tw, self.tp = spec, spec.draft, dw, target_w, tp
        self.rc = _Recipe(spec.weight_dtype)
        self.device, self.capacity = device, capacity
        self.reset()

    def reset(self):
        d = self.d
        self.k = [torch.zeros(self.capacity, d.kv_head_count, d.head_dim, device=self.device) for _ in range(d.layer_count)]
        self.v = [torch.zeros(self.capacity, d.kv_head_count, d.head_dim, device=self.device) for _ in range(d.layer_count)]

    def _headnorm(self, x, g):
        xf = x.float()
        return self.rc.r(xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.d.norm_eps) * g.float())

    def _tp_linear(self, act, w, resid=None):
        """Row-parallel linear: each rank's fp32 partial is rounded to bf16, partials are added
        in rank order in fp32 on top of the residual, and the sum is rounded once."""
        kk = act.shape[1] // self.tp
        tot = torch.zeros(act.shape[0], w.shape[0], device=act.device) if resid is None else resid.float().clone()
        for r in range(self.tp):
            tot = tot + self.rc.r(act[:, r * kk:(r + 1) * kk].float() @ w[:, r * kk:(r + 1) * kk].float().T)
        return self.rc.r(tot)

    @torch.no_grad()
    def ingest(self, feats: torch.Tensor, pos0: int):
        """feats [n, taps*hidden] (bf16-valued) for positions pos0.. -> draft KV."""
        d, rc = self.d, self.rc
        n = feats.shape[0]
        pos = torch.arange(pos0, pos0 + n, device=self.device)
        h = self._tp_linear(feats, self.w["fc"])
        c = rc.rmsnorm(h, self.w["hidden_norm"], d.norm_eps)
        tab = rope_table(pos, d.head_dim, d.rope_theta)
        for l, lw in enumerate(self.w["layers"]):
            k = rc.r(rc.linear(c, lw["wk"])).reshape(n, d.kv_head_count, d.head_dim)
            k = self._headnorm(k, lw["k_norm"])
            k = rc.r(apply_rope(k, tab, d.head_dim))
            v = rc.r(rc.linear(c, lw["wv"])).reshape(n, d.kv_head_count, d.head_dim)
            self.k[l][pos] = k
            self.v[l][pos] = v

    @torch.no_grad()
    def block(self, anchor: int, pos0: int) -> torch.Tensor:
        """Hidden states [rows, hidden] of the draft block whose row 0 sits at position pos0."""
        d, rc = self.d, self.rc
        R = d.rows
        x = self.w["mask_embedding"].float().repeat(R, 1)
        x[0] = self.tw["embed"][anchor].float()
        x = rc.r(x)
        pos = torch.arange(pos0, pos0 + R, device=self.device)
        tab = rope_table(pos, d.head_dim, d.rope_theta)
        lo = max(0, pos0 - d.window)
        group = d.head_count // d.kv_head_count
        for l, lw in enumerate(self.w["layers"]):
            xn = rc.rmsnorm(x, lw["g_in"], d.norm_eps)
            q = self._headnorm(rc.r(rc.linear(xn, lw["wq"])).reshape(R, d.head_count, d.head_dim), lw["q_norm"])
            k = self._headnorm(rc.r(rc.linear(xn, lw["wk"])).reshape(R, d.kv_head_count, d.head_dim), lw["k_norm"])
            v = rc.r(rc.linear(xn, lw["wv"])).reshape(R, d.kv_head_count, d.head_dim)
            q = rc.r(apply_rope(q, tab, d.head_dim))
            k = rc.r(apply_rope(k, tab, d.head_dim))
            kk = torch.cat((self.k[l][lo:pos0], k), 0)
            vv = torch.cat((self.v[l][lo:pos0], v), 0)
            o = torch.zeros(R, d.head_count, d.head_dim, device=self.device)
            for h in range(d.head_count):
                g = h // group
                sc = (q[:, h] @ kk[:, g].T) * (d.head_dim ** -0.5)
                o[:, h] = torch.softmax(sc.float(), -1) @ vv[:, g]
            o = rc.r(o).reshape(R, -1)
            x = self._tp_linear(o, lw["wo"], resid=x)
            xn = rc.rmsnorm(x, lw["g_post"], d.norm_eps)
            I = d.intermediate // self.tp
            tot = x.float().clone()
            for r in range(self.tp):
                g_ = rc.linear(xn, lw["gate"][r * I:(r + 1) * I])
                u_ = rc.linear(xn, lw["up"][r * I:(r + 1) * I])
                y = rc.r(torch.nn.functional.silu(g_) * u_)
                tot = tot + rc.r(y @ lw["down"][:, r * I:(r + 1) * I].float().T)
            x = rc.r(tot)
        return x

    @torch.no_grad()
    def head_logits(self, x: torch.Tensor) -> torch.Tensor:
        xn = self.rc.rmsnorm(x, self.w["norm"], self.d.norm_eps)
        return self.rc.linear(xn, self.tw["lm_head"])

    @torch.no_grad()
    def markov_bias(self, prev: int) -> torch.Tensor:
        return self.rc.r(self.w["markov_w1"][prev].float() @ self.w["markov_w2"].float().T)
