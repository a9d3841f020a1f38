"""Exact assistant-turn replay.

Clients often send history back with the assistant text trimmed or re-serialised; the prompt
then no longer reproduces the tokens that were generated and the parked prefix of the session
cannot be reused.  ``AssistantReplay`` remembers each generated reply under a digest of the
conversation that led to it and, when a later request contains the same turn up to
whitespace, substitutes the exact generated text.

Parity: naivert/serve/replay.py (``AssistantReplay.restore`` :38, ``remember`` :57).
"""
from __future__ import annotations

import hashlib
import json
from collections import OrderedDict
from typing import Any, Dict, List


def _digest(prev: str, msg: Dict[str, Any]) -> str:
    h = hashlib.sha256(prev.encode())
    h.update(json.dumps({k: msg.get(k) for k in ("role", "content", "reasoning_content", "tool_calls")},
                        sort_keys=True, ensure_ascii=False, default=str).encode())
    return h.hexdigest()


def _squash(s: str) -> str:
    return "".join((s or "").split())


class AssistantReplay:
    def __init__(self, max_bytes: int = 16 << 20, max_entries: int = 256):
        self.max_bytes, self.max_entries = max_bytes, max_entries
        self.store: "OrderedDict[str, Dict[str, str]]" = OrderedDict()
        self.bytes = 0

    def _walk(self, messages: List[dict]):
        d = ""
        for i, m in enumerate(messages):
            yield i, d
            d = _digest(d, m)

    def restore(self, task) -> int:
        """Replace assistant turns that match a remembered reply up to whitespace; returns the count."""
        n = 0
        for i, d in self._walk(task.messages):
            m = task.messages[i]
            if m["role"] != "assistant":
                continue
            kept = self.store.get(d)
            if kept is None:
                continue
            self.store.move_to_end(d)
            if _squash(kept["content"]) == _squash(m.get("content", "")) and \
                    _squash(kept.get("reasoning_content", "")) == _squash(m.get("reasoning_content", "")):
                if kept["content"] != m.get("content") or kept.get("reasoning_content", "") != m.get("reasoning_content", ""):
                    n += 1
                m["content"] = kept["content"]
                if kept.get("reasoning_content"):
                    m["reasoning_content"] = kept["reasoning_content"]
        return n

    def remember(self, task, blocks: List[dict]) -> None:
        d = ""
        for m in task.messages:
            d = _digest(d, m)
        entry = {"content": "".join(b.get("text", "") for b in blocks if b["type"] == "text"),
                 "reasoning_content": "".join(b.get("thinking", "") for b in blocks if b["type"] == "thinking")}
        size = len(entry["content"]) + len(entry["reasoning_content"])
        if size > self.max_bytes:
            return
        self.store[d] = entry
        self.bytes += size
        while len(self.store) > self.max_entries or self.bytes > self.max_bytes:
            _, old = self.store.popitem(last=False)
            self.bytes -= len(old["content"]) + len(old["reasoning_content"])
