"""CPU model of the tagged-word fabric protocol: threads stand in for ranks.

The model follows the device code word for word at the protocol level - 64-bit words
``{tag, payload}`` pushed into the *destination's* mailbox, consumers polling their own memory,
slab = call % 4, tag = epoch * 1024 + call + 1, bounded waits that record the first failing site in
a status word and make every later wait return at once - so the failure paths that must never be
provoked on a GPU of the shared pool (a rank that never publishes, a rank that leaves between
steps) are exercised here.  The small-message exchange of the sampler / Markov head (``SimExchange``: all-to-all and
reduce-scatter forms, tag = epoch * 64 + call + 1) is modelled the same way; the tests run a whole round's call plan
under random rank skew and show what the slab rule (consecutive calls differ modulo 4) protects against.

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


# --------------------------------------------------------------------------- small exchange (csrc/fabric.cuh)
SITE_RENDEZVOUS = 0x700
XCHG_SLABS = 4


class SimExchange:
    """The small-message boxes of ``tp`` simulated ranks: box[dst][slab][src][value index] -> (tag, value).  A value
    is one 64-bit integer here (the device splits it into two tagged 32-bit words; both carry the same tag)."""

    def __init__(self, tp: int, max_values: int = 4096):
        self.tp, self.max_values = tp, max_values
        self.tag = np.zeros((tp, XCHG_SLABS, tp, max_values), dtype=np.uint32)
        self.val = np.zeros((tp, XCHG_SLABS, tp, max_values), dtype=np.uint64)
        self.status = np.zeros(tp, dtype=np.uint32)
        self.epoch = np.ones(tp, dtype=np.uint32)
        self.lock = threading.Lock()

    def report(self, rank: int, site: int) -> None:
        with self.lock:
            if self.status[rank] == 0:
                self.status[rank] = site


def _collect(x: SimExchange, rank: int, idx: np.ndarray, tag, slab: int, call: int, timeout_s: float):
    """Poll this rank's box until every peer's words for the value indices ``idx`` carry ``tag``; -> [tp, len(idx)] or None."""
    got = np.zeros((x.tp, len(idx)), dtype=np.uint64)
    missing = [s for s in range(x.tp) if s != rank] if len(idx) else []
    deadline = time.monotonic() + timeout_s
    while missing:
        if x.status[rank] != 0:
            return None
        for s in list(missing):
            if np.all(x.tag[rank, slab, s, idx] == tag):
                got[s] = x.val[rank, slab, s, idx]
                missing.remove(s)
        if missing and time.monotonic() > deadline:
            x.report(rank, SITE_RENDEZVOUS | call)
            return None
        if missing:
            time.sleep(1e-4)
    return got


def xchg_reduce(x: SimExchange, rank: int, vals: np.ndarray, call: int, op: str = "sum", timeout_s: float = 1.0,
                delay_s: float = 0.0) -> Optional[np.ndarray]:
    """All-to-all form: every rank pushes all values to every peer and reduces locally."""
    if x.tp <= 1:
        return vals.copy()
    tag, slab = np.uint32(int(x.epoch[rank]) * 64 + call + 1), call % XCHG_SLABS
    idx = np.arange(len(vals))
    if delay_s:
        time.sleep(delay_s)
    for d in range(1, x.tp):
        peer = (rank + d) % x.tp
        x.val[peer, slab, rank, idx] = vals
        x.tag[peer, slab, rank, idx] = tag
    got = _collect(x, rank, idx, tag, slab, call, timeout_s)
    if got is None:
        return None
    got[rank] = vals
    return got.sum(0, dtype=np.uint64) if op == "sum" else got.max(0)


def xchg_reduce_scatter(x: SimExchange, rank: int, vals: np.ndarray, groups: int, gsize: int, live: int, call: int,
                        timeout_s: float = 1.0, delay_s: float = 0.0) -> Optional[np.ndarray]:
    """Reduce-scatter form: group g (values g * gsize ..) is owned by rank g % tp; values of live groups go to their
    owners only, an owner's groups come back summed, the others keep the local values."""
    if x.tp <= 1:
        return vals.copy()
    tag, slab = np.uint32(int(x.epoch[rank]) * 64 + call + 1), call % XCHG_SLABS
    if delay_s:
        time.sleep(delay_s)
    out = vals.copy()
    own_idx = []
    for g in range(groups):
        if not (live >> g) & 1:
            continue
        idx = np.arange(g * gsize, (g + 1) * gsize)
        owner = g % x.tp
        if owner == rank:
            own_idx.append(idx)
        else:
            x.val[owner, slab, rank, idx] = vals[idx]
            x.tag[owner, slab, rank, idx] = tag
    if own_idx:
        idx = np.concatenate(own_idx)
        got = _collect(x, rank, idx, tag, slab, call, timeout_s)
        if got is None:
            return None
        got[rank] = vals[idx]
        out[idx] = got.sum(0, dtype=np.uint64)
    return out
