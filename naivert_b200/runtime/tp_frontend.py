"""Driving a tensor-parallel engine from one process: rank 0 owns the HTTP server and the
request logic, the other ranks mirror its engine calls.

Commands travel over a CPU (gloo) process group as small Python objects; the decode itself
needs no host coordination - every rank polls its own ring (all tails write the same record)
and launches the same number of rounds; a cancel set on rank 0 reaches the others through the
tail kernel's cross-rank consensus.

The reference runs all eight GPUs from one process (naivert/prefill/comms.py:12-15); one
process per GPU with ``torch.distributed`` is the layout here.
"""
from __future__ import annotations

from typing import Any, Optional, Sequence

import torch.distributed as dist

from ..models.spec import SamplingParams
from .session_engine import Session, SessionEngine


class Commands:
    """Broadcast channel rank 0 -> followers."""

    def __init__(self, group=None):
        self.group = group

    def send(self, obj: Any) -> None:
        dist.broadcast_object_list([obj], src=0, group=self.group)

    def recv(self) -> Any:
        box = [None]
        dist.broadcast_object_list(box, src=0, group=self.group)
        return box[0]


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
