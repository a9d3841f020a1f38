"""Peer-memory fabric: one process per GPU, symmetric device buffers exported over CUDA IPC.

Each rank allocates two regions that every peer maps: the *mailbox* (tagged-word partials of
the fused GEMM -> all-reduce epilogues) and the *exchange box* (small integer reductions of
the sampler, draft head and tail).  Handles are exchanged once through ``torch.distributed``
(any backend); afterwards all traffic is issued from inside kernels with plain system-scope
stores into peer memory - no NCCL call sits on the decode path.  A status word collects
the first bounded wait that gave up, an epoch word (advanced once per step / round) makes
every tag unique.

Parity: naivert/common/tp8_mailbox.cuh (tagged-word mailbox, generation tags, bounded waits,
watchdog word) and the single-process peer enablement of the reference harness.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from ..ops import kernels as K

MAILBOX_FEATURES_MAX = 8192


def mailbox_bytes(tp: int, features: int) -> int:
    """slabs x source ranks x features x row pairs x 8-byte tagged words."""
    return K.K_MAILBOX_SLABS * tp * features * K.K_ROW_PAIRS * 8


def xchg_bytes(tp: int) -> int:
    return 4 * tp * 4096 * 2 * 8


class Fabric:
    def __init__(self, rank: int, tp: int, features: int, group=None, device: Optional[torch.device] = None,
                 timeout_ns: int = 2_000_000_000):
        self.rank, self.tp, self.features, self.group = rank, tp, features, group
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.timeout_ns = timeout_ns
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.epoch = torch.ones(1, dtype=torch.int32, device=self.device)
        self._local: List[int] = []
        self._opened: List[int] = []
        self.mailbox_ptrs = [0] * K.K_MAX_PEERS
        self.xchg_ptrs = [0] * K.K_MAX_PEERS
        if tp > 1:
            self.mailbox_ptrs = self._symmetric(mailbox_bytes(tp, features))
            self.xchg_ptrs = self._symmetric(xchg_bytes(tp))

    # -------------------------------------------------------------- symmetric allocation
    def _symmetric(self, nbytes: int) -> List[int]:
        import torch.distributed as dist
        L = K.lib()
        p = C.c_void_p()
        K.check(L.nrt_ipc_alloc(C.byref(p), C.c_size_t(nbytes)), "fabric alloc")
        self._local.append(p.value)
        hs = L.nrt_ipc_handle_size()
        buf = (C.c_ubyte * hs)()
        K.check(L.nrt_ipc_get_handle(p, C.byref(buf)), "cudaIpcGetMemHandle")
        handles: List[Optional[bytes]] = [None] * self.tp
        dist.all_gather_object(handles, bytes(buf), group=self.group)
        ptrs = [0] * K.K_MAX_PEERS
        for r, h in enumerate(handles):
            if r == self.rank:
                ptrs[r] = p.value
                continue
            q = C.c_void_p()
            hb = (C.c_ubyte * hs).from_buffer_copy(h)
            K.check(L.nrt_ipc_open(C.byref(hb), C.byref(q)), f"cudaIpcOpenMemHandle(rank {r})")
            self._opened.append(q.value)
            ptrs[r] = q.value
        dist.barrier(group=self.group)
        return ptrs

    # -------------------------------------------------------------- kernel argument blocks
    def fabric_args(self, call_idx: int, features: int) -> K.FabricArgs:
        if self.tp > 1 and features > self.features:
            raise ValueError(f"all-reduce width {features} exceeds the mailbox width {self.features}")
        f = K.FabricArgs()
        for i, p in enumerate(self.mailbox_ptrs):
            f.mailbox[i] = p
        f.epoch, f.status = self.epoch.data_ptr(), self.status.data_ptr()
        f.tp, f.rank, f.call_idx, f.features = self.tp, self.rank, call_idx, self.features
        f.timeout_ns = self.timeout_ns
        f.mode, f.ag_call = 0, -1
        return f

    def xchg_args(self) -> K.XchgArgs:
        x = K.XchgArgs()
        for i, p in enumerate(self.xchg_ptrs):
            x.box[i] = p
        x.epoch, x.status = self.epoch.data_ptr(), self.status.data_ptr()
        x.tp, x.rank, x.timeout_ns = self.tp, self.rank, self.timeout_ns
        return x

    def check(self) -> None:
        code = int(self.status[0])
        if code:
            raise RuntimeError(f"device wait gave up at site 0x{code:x} (rank {self.rank}): {explain_status(code)}")

    def close(self) -> None:
        L = K.lib()
        for q in self._opened:
            L.nrt_ipc_close(C.c_void_p(q))
        for p in self._local:
            L.nrt_ipc_free(C.c_void_p(p))
        self._opened, self._local = [], []


# status word = site class (bits 8..11, csrc/ptx.cuh) | detail (low byte)
_SITE_CLASSES = {
    0x100: "a consumer waited for a TMA stage that never filled (detail: stage; 0x10+: MoE down slots, 0x40: operand build, 0x80: sweep queries)",
    0x200: "a producer waited for a pipeline stage that was never released (detail: stage; 0x10+: MoE down slots)",
    0x300: "an epilogue waited for an accumulator commit (detail: TMEM buffer; 0x10+: MoE down)",
    0x400: "the MMA issuer waited for an accumulator buffer (detail: TMEM buffer; 0x10+: MoE down)",
    0x500: "a peer's tagged mailbox word did not arrive",
    0x600: "a cluster partner did not arrive",
    0x700: "a small-message exchange did not complete",
    0x800: "an in-grid hand-over did not complete",
}


def explain_status(code: int) -> str:
    """What a non-zero status word says: which bounded device wait gave up first (site codes of csrc/ptx.cuh and the
    details the kernels add to them)."""
    code = int(code)
    if code == 0:
        return "ok"
    cls, detail = code & 0xF00, code & 0xFF
    text = _SITE_CLASSES.get(cls, "unknown site class")
    if cls == 0x500:
        if detail & 0x80:
            text += f": expert-parallel return slot {detail & 0x7F} (a rank did not push its expert output)"
        elif detail & 0x60 == 0x60:
            text += f": all-gather flag of source rank {detail & 0x1F}"
        elif detail & 0x40:
            text += f": all-gather rows of source rank {detail & 0x1F}"
        else:
            text += f": all-reduce, first missing word slot {detail - 1} of the poll mask" if detail else ""
    elif cls == 0x700:
        names = {0: "sampler maxima", 1: "sampler totals", 10: "acceptance", 11: "rank totals of the draw", 12: "drawn token",
                 13: "tail pause consensus", 60: "greedy arg-max"}
        if 2 <= detail <= 9:
            what = f"nucleus pass {(detail - 2) // 2}: " + ("bins to the owning rank" if detail % 2 == 0 else "threshold digit")
        elif 16 <= detail <= 23:
            what = f"Markov step {detail - 16}"
        elif 32 <= detail <= 47:
            what = "expert-parallel token counts"
        else:
            what = names.get(detail, f"call {detail}")
        text += f": {what}"
    elif cls == 0x800:
        if detail & 0x40:
            text += f": sampler phase {detail & 0x3F}"
        elif detail & 0x20:
            text += f": Markov step {detail & 0x1F}"
        else:
            text += {1: ": fused MoE arrival (scores of all CTAs)", 2: ": fused MoE gate/up tile flag",
                     3: ": fused MoE expert-range partial"}.get(detail, f": detail {detail}")
    return text
