"""Session prefix parking: per-session snapshots of the KV state so a later request that
shares a token prefix resumes instead of re-reading its prompt.

A *park* holds, for ``position`` context rows: rows [0, position) of every full-length cache
(DSA k / v / indexer key + scale, draft k / v), every sliding-window ring in full, and the
token list.  A *checkpoint* holds only the rings (and the position), taken at prompt end,
so a branching conversation can rewind to that point: full-length caches are position
indexed and rewind for free, rings are not.  Entries are evicted least-recently-used down to
a byte budget per rank.

Parity: naivert/backends/naive_n0p5_prefix_store.py (``clear/checkpoint/save/restore/evict/bytes``
:21-143) and the selection rule of naivert/backends/naive_n0p5_session_engine.py:52-118.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch


@dataclass
class RingCheckpoint:
    position: int
    rings: List[torch.Tensor]


@dataclass
class ParkedPrefix:
    key: str
    tokens: List[int]
    position: int                              # context rows held (tokens[:position] are in the caches)
    rows: List[torch.Tensor]                   # full-length caches, first `position` rows each
    rings: List[torch.Tensor]
    checkpoints: List[RingCheckpoint] = field(default_factory=list)
    last_used: float = 0.0

    def nbytes(self) -> int:
        n = sum(t.numel() * t.element_size() for t in self.rows + self.rings)
        n += sum(t.numel() * t.element_size() for c in self.checkpoints for t in c.rings)
        return n


def common_prefix(a: Sequence[int], b: Sequence[int]) -> int:
    n = 0
    for x, y in zip(a, b):
        if x != y:
            break
        n += 1
    return n


@dataclass
class ResumeChoice:
    key: str
    position: int                 # rows to restore
    checkpoint: Optional[int]     # index into entry.checkpoints, None = the park itself
    matched: int                  # common token prefix with the entry


def select_resume(entries: Dict[str, ParkedPrefix], tokens: Sequence[int], session_id: Optional[str],
                  min_gain: int = 16) -> Optional[ResumeChoice]:
    """Longest usable prefix.  A resume point must not exceed the common token prefix (and must
    leave the last prompt token for the anchor); the request's own session key wins ties; entries
    named ``key#N`` are siblings of ``key`` (branches of one conversation)."""
    best: Optional[ResumeChoice] = None
    limit = len(tokens) - 1
    for key, e in entries.items():
        m = common_prefix(e.tokens, tokens)
        points: List[Tuple[int, Optional[int]]] = [(e.position, None)]
        points += [(c.position, i) for i, c in enumerate(e.checkpoints)]
        for pos, ck in points:
            if pos > min(m, limit) or pos < min_gain:
                continue
            own = session_id is not None and (key == session_id or key.split("#")[0] == session_id)
            cand = ResumeChoice(key, pos, ck, m)
            if best is None or (pos, own) > (best.position, session_id is not None and
                                             (best.key == session_id or best.key.split("#")[0] == session_id)):
                best = cand
    return best


def best_prefix_match(entries: Dict[str, "ParkedPrefix"], tokens: Sequence[int]) -> Optional[tuple]:
    """(key, common prefix length) of the parked entry that shares the longest prefix with ``tokens``, or None.  Only a
    diagnostic: when nothing resumes, the entry that came closest says where the client's re-rendered history first
    departs from what the model produced (naivert/backends/naive_n0p5_session_engine.py:88-99)."""
    best = None
    for key, e in entries.items():
        c = common_prefix(e.tokens[:e.position], tokens)
        if best is None or c > best[1]:
            best = (key, c)
    return best


def park_name(entries: Dict[str, ParkedPrefix], session_id: Optional[str], tokens: Sequence[int]) -> str:
    """Name under which a finished request is parked: the session key when the stored sequence is a
    prefix of the new one (the conversation continued), else a ``key#N`` sibling (it branched)."""
    base = session_id or "anon"
    cur = entries.get(base)
    if cur is None or common_prefix(cur.tokens, tokens) >= min(len(cur.tokens), cur.position):
        return base
    n = 1
    while f"{base}#{n}" in entries:
        n += 1
    return f"{base}#{n}"


class PrefixStore:
    """``full`` are the position-indexed caches, ``rings`` the sliding-window rings (live tensors
    of the runtime; snapshots are clones on ``device`` - the cache device or pinned host)."""

    def __init__(self, full: List[torch.Tensor], rings: List[torch.Tensor], budget_bytes: int, host: bool = False):
        self.full, self.rings, self.budget, self.host = full, rings, budget_bytes, host
        self.entries: Dict[str, ParkedPrefix] = {}

    def _keep(self, t: torch.Tensor) -> torch.Tensor:
        if self.host:
            out = torch.empty(t.shape, dtype=t.dtype, pin_memory=t.is_cuda)
            out.copy_(t)
            return out
        return t.clone()

    def clear(self) -> None:
        self.entries.clear()

    def bytes(self) -> int:
        return sum(e.nbytes() for e in self.entries.values())

    def make_checkpoint(self, position: int) -> RingCheckpoint:
        """Snapshot of the rings at ``position``, owned by the caller (a session keeps the one taken at its prompt
        end and hands it to ``save`` together with the tokens it belongs to)."""
        return RingCheckpoint(position, [self._keep(r) for r in self.rings])

    def save(self, key: str, tokens: Sequence[int], position: int,
             checkpoints: Optional[Sequence[RingCheckpoint]] = None) -> ParkedPrefix:
        """Park ``tokens[:position]``.  A checkpoint must belong to the saved prefix: those handed in were taken
        while this very sequence was in the caches; those of the entry being replaced are kept only inside the
        token prefix the old and the new sequence share."""
        old = self.entries.get(key)
        shared = min(position, common_prefix(old.tokens, tokens)) if old else 0
        cks = [c for c in (old.checkpoints if old else []) if c.position <= shared]
        for c in checkpoints or ():
            if c is not None and c.position <= position:
                cks = [k for k in cks if k.position != c.position] + [c]
        cks = sorted(cks, key=lambda c: c.position)[-4:]
        e = ParkedPrefix(key, list(tokens), position, [self._keep(t[:position]) for t in self.full],
                         [self._keep(r) for r in self.rings], cks, time.monotonic())
        self.entries[key] = e
        self.evict_to_budget(keep=key)
        return e

    def restore(self, choice: ResumeChoice) -> int:
        e = self.entries[choice.key]
        pos = choice.position
        for live, kept in zip(self.full, e.rows):
            live[:pos].copy_(kept[:pos], non_blocking=True)
        rings = e.rings if choice.checkpoint is None else e.checkpoints[choice.checkpoint].rings
        for live, kept in zip(self.rings, rings):
            live.copy_(kept, non_blocking=True)
        e.last_used = time.monotonic()
        return pos

    def evict(self, key: str) -> None:
        self.entries.pop(key, None)

    def evict_to_budget(self, keep: Optional[str] = None) -> List[str]:
        gone = []
        while self.bytes() > self.budget and len(self.entries) > (1 if keep in self.entries else 0):
            victim = min((e for k, e in self.entries.items() if k != keep), key=lambda e: e.last_used, default=None)
            if victim is None:
                break
            gone.append(victim.key)
            del self.entries[victim.key]
        return gone
