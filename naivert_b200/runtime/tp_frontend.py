"""Driving a tensor-parallel engine from one process: rank 0 owns the HTTP server and the
request logic, the other ranks mirror its engine calls.

Commands travel through the job's key-value store (the one ``torch.distributed`` rendezvoused on) as small
pickled objects, not through a collective: a collective with a dead peer can block for as long as the backend
likes, a store wait has the time-out we give it.  Every follower acknowledges the receipt of a command; a
follower that has left (crashed rank, closed connection) makes the leader's next command fail after
``ack_timeout_s`` with an error that names the missing ranks - the serving layer answers 500 and resets the slot
instead of hanging.  The decode itself needs no host coordination - every rank polls its own ring (all tails write
the same record) and launches the same number of rounds; a cancel set on rank 0 reaches the others through the tail
kernel's cross-rank consensus.

The reference runs all eight GPUs from one process (naivert/prefill/comms.py:12-15); one
process per GPU with ``torch.distributed`` is the layout here.
"""
from __future__ import annotations

import pickle
from datetime import timedelta
from typing import Any, Optional, Sequence

import torch.distributed as dist

from ..models.spec import SamplingParams
from .session_engine import Session, SessionEngine


class FollowerLost(RuntimeError):
    """A follower rank did not acknowledge a command in time."""


class Commands:
    """Command channel rank 0 -> followers over the rendezvous store, with receipt acknowledgements."""

    def __init__(self, group=None, store=None, rank: Optional[int] = None, world: Optional[int] = None,
                 ack_timeout_s: float = 30.0, prefix: str = "nrt"):
        self.group = group                         # kept for callers that pass the CPU group; not used for transport
        self.store = store if store is not None else dist.distributed_c10d._get_default_store()
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.ack_timeout_s = ack_timeout_s
        self.prefix = prefix
        self.seq = 0

    def _key(self, kind: str, seq: int, rank: Optional[int] = None) -> str:
        return f"{self.prefix}/{kind}/{seq}" + ("" if rank is None else f"/{rank}")

    def send(self, obj: Any) -> None:
        self.seq += 1
        self.store.set(self._key("cmd", self.seq), pickle.dumps(obj))
        acks = [self._key("ack", self.seq, r) for r in range(1, self.world)]
        try:
            if acks:
                self.store.wait(acks, timedelta(seconds=self.ack_timeout_s))
        except Exception as e:                      # noqa: BLE001 - the store raises backend-specific timeout types
            missing = [r for r in range(1, self.world) if not self._has(self._key("ack", self.seq, r))]
            raise FollowerLost(f"ranks {missing} did not acknowledge command {self.seq} ({obj.get('op') if isinstance(obj, dict) else '?'}) "
                               f"within {self.ack_timeout_s:.0f} s") from e
        if self.seq > 2:                            # the store does not grow with the number of requests
            old = self.seq - 2
            for k in [self._key("cmd", old)] + [self._key("ack", old, r) for r in range(1, self.world)]:
                try:
                    self.store.delete_key(k)
                except Exception:                   # noqa: BLE001 - not every store backend can delete
                    pass

    def _has(self, key: str) -> bool:
        try:
            return bool(self.store.check([key]))
        except Exception:                           # noqa: BLE001
            return False

    def recv(self, idle_poll_s: float = 5.0) -> Any:
        self.seq += 1
        key = self._key("cmd", self.seq)
        while True:                                 # an idle server waits here for hours: poll in short store waits
            try:
                self.store.wait([key], timedelta(seconds=idle_poll_s))
                break
            except Exception:                       # noqa: BLE001 - time-out of an idle wait
                continue
        obj = pickle.loads(self.store.get(key))
        self.store.set(self._key("ack", self.seq, self.rank), b"1")
        return obj


class LeaderEngine:
    """Duck-type compatible with ``SessionEngine`` for the serving layer; mirrors calls to followers."""

    def __init__(self, engine: SessionEngine, channel: Commands):
        self.inner, self.ch = engine, channel
        self.config = engine.config

    def align_prompt(self, tokens: Sequence[int], session_id: Optional[str], text: Optional[str] = None):
        return self.inner.align_prompt(tokens, session_id, text=text)

    def open_session(self, tokens, max_decode, session_id, sampling: Optional[SamplingParams] = None) -> "LeaderSession":
        self.ch.send({"op": "open", "tokens": list(tokens), "max_decode": int(max_decode), "session_id": session_id,
                      "sampling": sampling})
        return LeaderSession(self.inner.open_session(tokens, max_decode, session_id, sampling), self.ch)

    def close(self) -> None:
        self.ch.send({"op": "close"})
        self.inner.close()


class LeaderSession:
    def __init__(self, s: Session, ch: Commands):
        self.s, self.ch = s, ch

    def __getattr__(self, name):
        return getattr(self.s, name)

    def step(self, timeout_s: float = 120.0):
        return self.s.step(timeout_s)

    def cancel(self) -> None:
        self.s.cancel()

    def finish(self) -> dict:
        self.ch.send({"op": "finish"})
        return self.s.finish()


def follower_loop(engine: SessionEngine, channel: Commands, step_timeout_s: float = 300.0) -> None:
    """Run on every rank but 0 until the leader closes."""
    while True:
        cmd = channel.recv()
        if cmd["op"] == "close":
            engine.close()
            return
        if cmd["op"] == "open":
            s = engine.open_session(cmd["tokens"], cmd["max_decode"], cmd["session_id"], cmd["sampling"])
            while not s.done:
                s.step(step_timeout_s)
            nxt = channel.recv()
            if nxt["op"] != "finish":
                raise RuntimeError(f"protocol error: expected finish, got {nxt['op']}")
            s.finish()
