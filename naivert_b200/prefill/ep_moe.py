"""Expert-parallel MoE layer for prefill chunks: tokens are row-sharded over the ranks (sequence
parallel), experts are whole and sharded over the ranks (expert parallel).

    count -> dispatch (RMSNorm + e4m3 quantisation + expert-sorted placement in the expert rank's memory)
          -> grouped gate/up GEMM (tcgen05, SiLU, e4m3 re-quantisation)
          -> grouped down GEMM whose epilogue returns bf16 rows to the token owner (tagged words)
          -> combine (probability-weighted fixed-order sum + residual)

Everything between ranks is peer stores issued by these kernels; no NCCL call.  Buffers are sized for the
worst case (every token of every rank routed to one rank).

Parity: the EP8 expert path of the reference's native prefill (naivert/prefill/native/executor.py:431-474:
DeepEP dispatch, DeepGEMM contiguous grouped GEMM, ``native_combine``) and naivert/prefill/operands.py
(``load_expert_rank``: whole experts per rank).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from ..ops import kernels as K
from ..parallel.fabric import Fabric

CALL_DISPATCH, CALL_RETURN = 900, 901


def _raw_map(ptr: int, rows: int, cols_bytes: int, box_rows: int = 16) -> K.TensorMap:
    """Tensor map over a fabric allocation viewed as [rows, cols_bytes] bytes (``box_rows`` x 128-byte boxes)."""
    m = K.TensorMap.__new__(K.TensorMap)
    m.tensor, m.buf = None, (C.c_ubyte * 128)()
    d = (C.c_uint64 * 5)(cols_bytes, rows)
    st = (C.c_uint64 * 5)(cols_bytes)
    bx = (C.c_uint32 * 5)(128, box_rows)
    K.check(K.lib().nrt_tmap_encode(C.byref(m.buf), 0, 2, d, st, bx, 3, C.c_void_p(ptr)), "tensor map")
    return m


class EPWeights:
    """One MoE layer's experts held by this rank, with their tensor maps.
    ``gate/up`` {"w": e4m3 [E_local, inter, hidden], "s": [E_local, inter/128, hidden/128]},
    ``down`` {"w": [E_local, hidden, inter], "s": ...}."""

    def __init__(self, gate: dict, up: dict, down: dict):
        self.gate_w, self.up_w, self.down_w = gate["w"].contiguous(), up["w"].contiguous(), down["w"].contiguous()
        self.gate_s, self.up_s, self.down_s = gate["s"].float().contiguous(), up["s"].float().contiguous(), down["s"].float().contiguous()
        self.map_gate = K.weight_tmap(self.gate_w.view(torch.uint8))
        self.map_up = K.weight_tmap(self.up_w.view(torch.uint8))
        self.map_down = K.weight_tmap(self.down_w.view(torch.uint8))


class EPMoE:
    def __init__(self, fabric: Fabric, hidden: int, inter: int, experts: int, top_k: int, tokens_local: int,
                 gate: Optional[dict] = None, up: Optional[dict] = None, down: Optional[dict] = None, eps: float = 1e-5,
                 item_rows: int = 16):
        """Exchange buffers for up to ``tokens_local`` rows per rank; the experts of a layer are passed to
        ``run`` (``EPWeights``) or, for a single layer, given here.  ``item_rows`` = 64 pads expert segments to
        64 rows and runs the grouped GEMMs on the 64-column chunk engine (16: the step engine's tile)."""
        if item_rows not in (16, K.WIDE_TOK):
            raise ValueError("item_rows must be 16 or 64")
        self.fab, self.H, self.I, self.E, self.K, self.T, self.eps = fabric, hidden, inter, experts, top_k, tokens_local, eps
        self.item_rows = item_rows
        tp, dev = fabric.tp, fabric.device
        self.El = experts // tp
        self.cap_rows = -(-(tokens_local * tp * top_k) // item_rows) * item_rows + item_rows * self.El    # worst case + segment padding
        self.max_items = self.cap_rows // item_rows + self.El
        i32, f32 = torch.int32, torch.float32
        self._keep: List[torch.Tensor] = []          # single-rank buffers (no fabric allocation needed)
        self.slot_of = torch.zeros(tokens_local * top_k, dtype=i32, device=dev)
        self.n_items = torch.zeros(1, dtype=i32, device=dev)
        self.item_expert = torch.zeros(self.max_items, dtype=i32, device=dev)
        self.item_row = torch.zeros(self.max_items, dtype=i32, device=dev)
        self.seg_rows = torch.zeros(self.El, dtype=i32, device=dev)
        self.ticket = torch.zeros(1, dtype=i32, device=dev)
        one = tp == 1
        alloc = (lambda n: self._local(n)) if one else fabric._symmetric
        self.recv8 = alloc(self.cap_rows * hidden)
        self.recvs = alloc(self.cap_rows * (hidden // 128) * 4)
        self.meta = alloc(self.cap_rows * 16)
        self.flags = alloc(4096)
        self.combine = alloc(tokens_local * top_k * (hidden // 2) * 8)
        self.y8 = torch.zeros(self.cap_rows, inter, dtype=torch.uint8, device=dev)
        self.ys = torch.ones(self.cap_rows, inter // 128, dtype=f32, device=dev)
        self.w = EPWeights(gate, up, down) if gate is not None else None
        self.stage = None                              # optional context-manager factory: per-kernel timing
        self.map_recv = _raw_map(self.recv8[fabric.rank], self.cap_rows, hidden, item_rows)
        self.map_y = K.act_tmap(self.y8, item_rows)

    def _local(self, nbytes: int) -> List[int]:
        t = torch.zeros(nbytes, dtype=torch.uint8, device=self.fab.device)
        self._keep.append(t)
        return [t.data_ptr()] + [0] * (K.K_MAX_PEERS - 1)

    def _ep_args(self, x, gamma, ids, probs, tokens) -> K.EpArgs:
        a = K.EpArgs()
        a.topk_ids, a.topk_p = ids.data_ptr(), probs.data_ptr()
        a.tokens, a.top_k, a.experts, a.experts_local, a.hidden = tokens, self.K, self.E, self.El, self.H
        a.slot_of, a.n_items = self.slot_of.data_ptr(), self.n_items.data_ptr()
        a.item_expert, a.item_row, a.seg_rows = self.item_expert.data_ptr(), self.item_row.data_ptr(), self.seg_rows.data_ptr()
        a.max_items, a.cap_rows = self.max_items, self.cap_rows
        a.x, a.gamma, a.eps = x.data_ptr(), None if gamma is None else gamma.data_ptr(), self.eps
        for i in range(K.K_MAX_PEERS):
            a.recv8[i], a.recvs[i], a.meta[i], a.flags[i] = self.recv8[i], self.recvs[i], self.meta[i], self.flags[i]
        a.ticket, a.call, a.item_rows = self.ticket.data_ptr(), CALL_DISPATCH, self.item_rows
        a.x_args = self.fab.xchg_args()
        return a

    def run(self, x: torch.Tensor, gamma: Optional[torch.Tensor], ids: torch.Tensor, probs: torch.Tensor,
            resid: torch.Tensor, out: torch.Tensor, pdl: bool = False, weights: Optional[EPWeights] = None,
            tokens: Optional[int] = None) -> None:
        """x [T, H] bf16 residual rows of this rank, ids/probs [T, top_k]; out = resid + sum_k p_k * expert_k(norm(x)).
        ``tokens`` (<= tokens_local, the same on every rank) rows take part; ``weights`` selects the layer."""
        fab, rank = self.fab, self.fab.rank
        w = weights or self.w
        T = self.T if tokens is None else tokens
        if not 0 < T <= self.T:
            raise ValueError(f"{T} rows exceed the exchange buffers sized for {self.T}")
        from contextlib import nullcontext
        stage = self.stage or (lambda name: nullcontext())
        a = self._ep_args(x, gamma, ids, probs, T)
        with stage("moe.count"):
            K.ep_count(a, pdl=pdl)
        with stage("moe.dispatch"):
            K.ep_dispatch(a, pdl=pdl)
        st = fab.status.data_ptr()
        g = K.GemmArgs()
        g.n_total, g.k_total, g.rows, g.out_scale = self.I, self.H, self.item_rows, 1.0
        g.n_active, g.active_ids, g.max_slots = self.n_items.data_ptr(), self.item_expert.data_ptr(), self.max_items
        g.row_offsets = self.item_row.data_ptr()
        g.w_scale0, g.w_scale1, g.a_scale = w.gate_s.data_ptr(), w.up_s.data_ptr(), self.recvs[rank]
        g.out_q, g.out_qscale = self.y8.data_ptr(), self.ys.data_ptr()
        g.fab = fab.fabric_args(0, self.H)
        g.fab.ag_call, g.fab.ag_flags = CALL_DISPATCH, self.flags[rank]
        g.status = st
        launch = K.wide_gemm if self.item_rows == K.WIDE_TOK else K.gemm
        with stage("moe.gate_up"):
            launch(K.gemm_variant(True, True, K.EPI_SILU_QUANT, K.GROUP_ITEM), w.map_gate, w.map_up, self.map_recv, g,
                   self.I // 128, self.max_items, pdl=pdl)
        d = K.GemmArgs()
        d.n_total, d.k_total, d.rows, d.out_scale = self.H, self.I, self.item_rows, 1.0
        d.n_active, d.active_ids, d.max_slots = self.n_items.data_ptr(), self.item_expert.data_ptr(), self.max_items
        d.row_offsets = self.item_row.data_ptr()
        d.w_scale0, d.a_scale = w.down_s.data_ptr(), self.ys.data_ptr()
        d.fab = fab.fabric_args(0, self.H)
        d.status = st
        d.ep_meta, d.ep_top_k = self.meta[rank], self.K
        for i in range(K.K_MAX_PEERS):
            d.ep_combine[i] = self.combine[i]
        d.ep_dispatch_call, d.ep_return_call = CALL_DISPATCH, CALL_RETURN
        with stage("moe.down_return"):
            launch(K.gemm_variant(True, False, K.EPI_RETURN, K.GROUP_ITEM), w.map_down, None, self.map_y, d,
                   self.H // 128, self.max_items, pdl=pdl)
        c = K.EpCombineArgs()
        c.slots, c.topk_p, c.resid, c.out = self.combine[rank], probs.data_ptr(), resid.data_ptr(), out.data_ptr()
        c.epoch, c.status = fab.epoch.data_ptr(), st
        c.tokens, c.top_k, c.hidden, c.call, c.timeout_ns = T, self.K, self.H, CALL_RETURN, fab.timeout_ns
        with stage("moe.combine"):
            K.ep_combine(c, pdl=pdl)
            K.epoch_advance(fab.epoch, pdl=pdl)


def ep_layout_reference(ids_per_rank: List[torch.Tensor], experts: int, item_rows: int = 16):
    """Host restatement of the layout ``ep_count`` computes on the device (for tests and debugging).

    ``ids_per_rank[s]`` are source rank s's routing choices [tokens, top_k] (global expert ids).  Returns, for every
    destination rank d: ``seg_base[d][el]`` (first receive-buffer row of local expert el, segments padded to
    ``item_rows``), ``seg_rows[d][el]`` (rows received), the work list ``items[d]`` = [(local expert, first row)], and
    ``slot[s]`` = destination row of every (token, k) pair of source s: segment base + rows of lower source ranks +
    the pair's rank among the source's pairs of that expert in (token, k) order."""
    tp = len(ids_per_rank)
    if experts % tp:
        raise ValueError("experts must divide over the ranks")
    el_n = experts // tp
    counts = torch.stack([torch.bincount(i.flatten().long(), minlength=experts) for i in ids_per_rank])   # [tp, E]
    seg_base, seg_rows, items = [], [], []
    for d in range(tp):
        base, bases, rows_d, work = 0, [], [], []
        for el in range(el_n):
            e = d * el_n + el
            rows = int(counts[:, e].sum())
            bases.append(base)
            rows_d.append(rows)
            work += [(el, base + r0) for r0 in range(0, rows, item_rows)]
            base += -(-rows // item_rows) * item_rows
        seg_base.append(bases); seg_rows.append(rows_d); items.append(work)
    slots = []
    for s, ids in enumerate(ids_per_rank):
        flat = ids.flatten().long()
        cursor = {}
        out = torch.empty_like(flat)
        for i, e in enumerate(flat.tolist()):
            d, el = divmod(e, el_n)
            start = seg_base[d][el] + int(counts[:s, e].sum())
            k = cursor.get(e, 0)
            out[i] = start + k
            cursor[e] = k + 1
        slots.append(out.reshape(ids.shape))
    return {"seg_base": seg_base, "seg_rows": seg_rows, "items": items, "slot": slots}
