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
            raise RuntimeError(f"device wait gave up at site 0x{code:x} (rank {self.rank})")

    def close(self) -> None:
        L = K.lib()
        for q in self._opened:
            L.nrt_ipc_close(C.c_void_p(q))
        for p in self._local:
            L.nrt_ipc_free(C.c_void_p(p))
        self._opened, self._local = [], []
