"""CPU model of the tagged-word fabric protocol: threads stand in for ranks.

The model follows the device code word for word at the protocol level - 64-bit words
``{tag, payload}`` pushed into the *destination's* mailbox, consumers polling their own memory,
slab = call % 4, tag = epoch * 1024 + call + 1, bounded waits that record the first failing site in
a status word and make every later wait return at once - so the failure paths that must never be
provoked on a GPU of the shared pool (a rank that never publishes, a rank that leaves between
steps) are exercised here.

Parity: naivert/common/tp8_mailbox.cuh:122-195 (bounded waits + watchdog word); failures are injected on
the host only (a simulated rank withholds one publish).
"""
from __future__ import annotations

import threading
import time
from typing import Callable, List, Optional, Sequence

import numpy as np

SLABS = 4
SITE_MAILBOX = 0x500


class SimFabric:
    """Shared 'peer memory' of ``tp`` simulated ranks."""

    def __init__(self, tp: int, features: int, pairs: int = 4):
        self.tp, self.features, self.pairs = tp, features, pairs
        # mailbox[dst][slab][src][pair][feature] -> (tag, payload)
        self.tag = np.zeros((tp, SLABS, tp, pairs, features), dtype=np.uint32)
        self.payload = np.zeros((tp, SLABS, tp, pairs, features), dtype=np.uint32)
        self.status = np.zeros(tp, dtype=np.uint32)
        self.epoch = np.ones(tp, dtype=np.uint32)
        self.lock = threading.Lock()

    def report(self, rank: int, site: int) -> None:
        with self.lock:
            if self.status[rank] == 0:
                self.status[rank] = site            # first writer wins


def _bf16_round(x: np.ndarray) -> np.ndarray:
    u = x.astype(np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) & 0xFFFF0000).view(np.float32)


def _pack(lo: np.ndarray, hi: np.ndarray) -> np.ndarray:
    return (lo.view(np.uint32) >> 16) | (hi.view(np.uint32) & 0xFFFF0000)


def _unpack(w: np.ndarray):
    return (w << 16).view(np.float32), (w & 0xFFFF0000).view(np.float32)


def all_reduce(fab: SimFabric, rank: int, partial: np.ndarray, resid: np.ndarray, call: int,
               timeout_s: float = 1.0, publish: bool = True, delay_s: float = 0.0) -> Optional[np.ndarray]:
    """One rank's side of the fused all-reduce epilogue.  ``partial`` [rows, features] fp32,
    ``resid`` [rows, features] bf16-valued fp32.  Returns the new residual, or None when the wait
    gave up (the status word then holds the site)."""
    rows = partial.shape[0]
    pairs = (rows + 1) // 2
    tag = np.uint32(int(fab.epoch[rank]) * 1024 + call + 1)
    slab = call % SLABS
    p = np.zeros((2 * pairs, fab.features), dtype=np.float32)
    p[:rows] = _bf16_round(partial)
    own = _pack(p[0::2], p[1::2])                                   # [pairs, features]
    if delay_s:
        time.sleep(delay_s)                                         # a late (but live) peer
    if publish:
        for d in range(1, fab.tp):
            peer = (rank + d) % fab.tp
            fab.payload[peer, slab, rank, :pairs] = own
            fab.tag[peer, slab, rank, :pairs] = tag                  # payload first, tag last
    deadline = time.monotonic() + timeout_s
    words = np.zeros((fab.tp, pairs, fab.features), dtype=np.uint32)
    words[rank] = own
    missing = [s for s in range(fab.tp) if s != rank]
    while missing:
        if fab.status[rank] != 0:
            return None                                             # someone already failed: do not spin
        for s in list(missing):
            if np.all(fab.tag[rank, slab, s, :pairs] == tag):
                words[s] = fab.payload[rank, slab, s, :pairs]
                missing.remove(s)
        if missing and time.monotonic() > deadline:
            fab.report(rank, SITE_MAILBOX | missing[0])
            return None
        if missing:
            time.sleep(1e-4)
    total = resid.astype(np.float32).copy()
    for s in range(fab.tp):                                         # fixed rank order
        lo, hi = _unpack(words[s])
        both = np.empty((2 * pairs, fab.features), dtype=np.float32)
        both[0::2], both[1::2] = lo, hi
        total += both[:rows]
    return _bf16_round(total)


def run_ranks(tp: int, fn: Callable[[int], object]) -> List[object]:
    out: List[object] = [None] * tp
    errs: List[BaseException] = []

    def body(r):
        try:
            out[r] = fn(r)
        except BaseException as e:      # noqa: BLE001
            errs.append(e)

    ts = [threading.Thread(target=body, args=(r,)) for r in range(tp)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    if errs:
        raise errs[0]
    return out
