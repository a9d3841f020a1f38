"""Canary-fenced tensor allocations: a debugging aid that replaces a memory checker.

``GuardedPool.alloc`` returns a tensor whose storage is surrounded by 4096-byte guard zones filled
with 0xA5 (front) / 0x5A (back); ``verify`` raises when any guard byte changed, naming the
allocation - i.e. which kernel output overran its buffer.  Works on CPU and CUDA tensors.

Parity: naivert/guarded_tensors.py (4096-byte 0xA5/0x5A guards, ``verify_canaries``).
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch

GUARD_BYTES = 4096
FRONT, BACK = 0xA5, 0x5A


class CanaryError(RuntimeError):
    pass


class GuardedPool:
    def __init__(self, device="cpu"):
        self.device = device
        self._items: List[Tuple[str, torch.Tensor, int]] = []

    def alloc(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        elem = torch.empty((), dtype=dtype).element_size()
        n = 1
        for d in shape:
            n *= d
        nbytes = n * elem
        padded = -(-nbytes // 256) * 256
        raw = torch.empty(2 * GUARD_BYTES + padded, dtype=torch.uint8, device=self.device)
        raw[:GUARD_BYTES] = FRONT
        raw[GUARD_BYTES + nbytes:] = BACK
        raw[GUARD_BYTES:GUARD_BYTES + nbytes] = 0
        self._items.append((name, raw, nbytes))
        return raw[GUARD_BYTES:GUARD_BYTES + nbytes].view(dtype).reshape(*shape)

    def like(self, t: torch.Tensor, name: str = "") -> torch.Tensor:
        """A fenced, zero-filled tensor with the shape and dtype of ``t`` (contiguous)."""
        return self.alloc(name or f"buf{len(self._items)}", tuple(t.shape), t.dtype)

    def verify(self) -> None:
        bad = []
        for name, raw, nbytes in self._items:
            front_ok = bool((raw[:GUARD_BYTES] == FRONT).all())
            back_ok = bool((raw[GUARD_BYTES + nbytes:] == BACK).all())
            if not (front_ok and back_ok):
                bad.append(f"{name} ({'underrun' if not front_ok else ''}{' ' if not front_ok and not back_ok else ''}{'overrun' if not back_ok else ''})")
        if bad:
            raise CanaryError("guard zones overwritten: " + ", ".join(bad))

    def names(self) -> List[str]:
        return [n for n, _, _ in self._items]
