"""NCCL baseline collectives (the measured baseline, not the product path) and helpers of the
fused paths.

``TPComm`` wraps ``torch.distributed`` all-reduce / reduce-scatter / all-gather on the rank's
process group with a warm-up, mirroring what the reference's prefill uses
(naivert/prefill/comms.py:54-147 ``TP8Comm``).  The fused counterparts live in the GEMM engine
(``FabricArgs.mode`` = reduce-scatter, ``ag_call`` = all-gathered operand) and ``ops.kernels.ag_push``.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class TPComm:
    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0

    def warmup(self, device) -> None:
        if self.world > 1:
            t = torch.ones(1024, device=device)
            dist.all_reduce(t, group=self.group)
            torch.cuda.synchronize(device) if t.is_cuda else None

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return t

    def reduce_scatter(self, t: torch.Tensor, dim_rows: bool = False) -> torch.Tensor:
        """[M, N] -> this rank's [M, N/world] column slice (or row slice) of the sum."""
        if self.world == 1:
            return t
        if dim_rows:
            out = torch.empty(t.shape[0] // self.world, *t.shape[1:], dtype=t.dtype, device=t.device)
            dist.reduce_scatter_tensor(out, t.contiguous(), group=self.group)
            return out
        cols = t.shape[1] // self.world
        chunks = t.reshape(t.shape[0], self.world, cols).permute(1, 0, 2).contiguous()
        out = torch.empty(t.shape[0], cols, dtype=t.dtype, device=t.device)
        dist.reduce_scatter_tensor(out, chunks, group=self.group)
        return out

    def all_gather_cols(self, t: torch.Tensor) -> torch.Tensor:
        """[M, K/world] slices -> [M, K]."""
        if self.world == 1:
            return t
        out = torch.empty(self.world, *t.shape, dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
        return out.permute(1, 0, 2).reshape(t.shape[0], -1)
