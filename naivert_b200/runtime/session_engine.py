"""Session engine: the object the serving layer talks to.  Adds session-prefix reuse, the
resume policy and per-request statistics on top of ``Engine``.

    engine = SessionEngine(Engine.build(...), store_gb=8)
    session = engine.open_session(tokens, max_decode, session_id, sampling)
    while not session.done: tokens += session.step(timeout)
    stats = session.finish()           # parks the KV state under the session key

Parity: ``SessionEngine`` / ``Session`` (naivert/backends/naive_n0p5_session_engine.py:52-118
resume selection, :123-212 prefill cost model and path policy, :263-340 step loop, :411-454
``align_prompt``, :590-630 ``_finish``).
"""
from __future__ import annotations

import logging
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..models.spec import FULL_DSA, SamplingParams
from .engine import Engine
from .prefix_store import PrefixStore, best_prefix_match, common_prefix, park_name, select_resume
from .round import RuntimeContractError

log = logging.getLogger("naivert_b200.session")

# Measured on B200 (ms); inputs of the resume / prefill-path policy.
REPLAY_MS_PER_TOKEN = 1.2            # 8-row verify replay per prompt token (tp8, 48 layers: 9.6 ms per 8 rows)
NATIVE_FIXED_MS = 90.0               # chunked native prefill at tp8, 48 layers: a chunk is bound by per-layer latencies
NATIVE_MS_PER_TOKEN = 0.003          # ... (launches, NCCL and peer exchanges: ~2 ms per layer), rows add little on top
NATIVE_MS_PER_TOKEN_PER_64K_CONTEXT = 0.001  # sweep + top-k grow with the context (131072 tokens: 3.2 s measured)
NATIVE_CHUNK = 4096
RESTORE_MS_PER_GB = 2.0


def prefill_estimate(new_tokens: int, path: str) -> float:
    """Estimated milliseconds to ingest ``new_tokens`` prompt tokens on ``path``."""
    if new_tokens <= 0:
        return 0.0
    if path == "replay":
        return new_tokens * REPLAY_MS_PER_TOKEN
    chunks = -(-new_tokens // NATIVE_CHUNK)
    context_term = NATIVE_MS_PER_TOKEN_PER_64K_CONTEXT * new_tokens * (new_tokens / 2.0) / 65536.0
    return chunks * NATIVE_FIXED_MS + new_tokens * NATIVE_MS_PER_TOKEN + context_term


def prefill_path(new_tokens: int, policy: str = "cost", native_ready: bool = False) -> str:
    """``replay`` (verify-8 replay) or ``native`` (chunked TP/EP prefill); ``cost`` picks the cheaper."""
    if policy in ("replay", "native"):
        return policy if (policy == "replay" or native_ready) else "replay"
    if not native_ready:
        return "replay"
    return "native" if prefill_estimate(new_tokens, "native") < prefill_estimate(new_tokens, "replay") else "replay"


@dataclass
class EngineConfig:
    capacity: int
    max_output_tokens: int
    eos_token_ids: Sequence[int]
    think_end_token_id: int


def segment_stats(tokens: Sequence[int], round_sizes: Sequence[int], round_ns: Sequence[int], think_end: int,
                  accepted: Sequence[int]) -> Dict[str, dict]:
    """Think / answer / total statistics from per-round device timestamps: the reply is split at the
    first ``think_end`` token; a round belongs to the segment its first token falls into."""
    out: Dict[str, dict] = {}
    split = tokens.index(think_end) + 1 if think_end in tokens else 0
    segs = {"think": (0, split), "answer": (split, len(tokens)), "total": (0, len(tokens))}
    starts, pos = [], 0
    for n in round_sizes:
        starts.append(pos)
        pos += n
    for name, (lo, hi) in segs.items():
        idx = [i for i, s in enumerate(starts) if lo <= s < hi and i > 0]
        toks = sum(round_sizes[i] for i in idx)
        ns = sum(round_ns[i] - round_ns[i - 1] for i in idx)
        if hi - lo <= 0:
            continue
        out[name] = {"tokens": hi - lo, "rounds": len(idx), "tokens_per_round": round(toks / max(1, len(idx)), 3),
                     "device_ms": round(ns * 1e-6, 3), "device_tok_s": round(toks / (ns * 1e-9), 2) if ns > 0 else 0.0,
                     "acceptance": round(sum(accepted[i] for i in idx) / max(1, 7 * len(idx)), 4)}
    return out


def acceptance_histogram(accepted: Sequence[int], block: int = 7) -> List[int]:
    """Rounds by accepted draft prefix length 0..block (the reference keeps this as a device counter array,
    ``verify_counts``; here it is derived from the ring records the host already reads)."""
    hist = [0] * (block + 1)
    for a in accepted:
        hist[min(max(int(a), 0), block)] += 1
    return hist


class Session:
    def __init__(self, owner: "SessionEngine", tokens: List[int], cached: int, session_id: Optional[str], info: dict):
        self.owner, self.prompt, self.cached_tokens, self.session_id = owner, tokens, cached, session_id
        self.prefill_info = info
        self.done, self.stop_reason = False, None
        self.out: List[int] = []
        self.round_sizes: List[int] = []
        self.round_ns: List[int] = []
        self.accepted: List[int] = []
        self._launched = False
        self.closed = False

    def step(self, timeout_s: float = 120.0) -> List[int]:
        """Tokens of the next published round (launches rounds ahead of the host as needed)."""
        if self.done:
            return []
        r = self.owner.engine.round
        if not self._launched:
            r.launch(self.owner.ahead)
            self._launched = True
        rec = r.wait_round(timeout_s)
        self.out.extend(rec.tokens)
        self.round_sizes.append(len(rec.tokens))
        self.round_ns.append(rec.t_end_ns)
        self.accepted.append(rec.accepted)
        if rec.stop_reason is not None:
            self.done, self.stop_reason = True, rec.stop_reason
        else:
            r.launch(1)
        return rec.tokens

    def cancel(self) -> None:
        if not self.done:
            self.owner.engine.round.cancel()

    def finish(self) -> dict:
        """Drain the chain, check the fabric, park the KV state; returns device statistics."""
        if self.closed:
            return {}
        self.closed = True
        eng = self.owner.engine
        r = eng.round
        if self._launched and not self.done:
            r.cancel()
            deadline = time.monotonic() + self.owner.cancel_timeout_s
            while not self.done:
                rec = r.poll()
                if rec is None:
                    if time.monotonic() > deadline:
                        raise RuntimeError("the running chain did not honour the cancel request")
                    time.sleep(1e-4)
                    continue
                self.out.extend(rec.tokens)
                self.round_sizes.append(len(rec.tokens))
                self.round_ns.append(rec.t_end_ns)
                self.accepted.append(rec.accepted)
                if rec.stop_reason is not None:
                    self.done, self.stop_reason = True, rec.stop_reason
        if self._launched:
            r.launch(1, force=True)                       # one more pass completes the draft context of the last rows
        r.stream.synchronize()
        eng.fabric.check()
        stats = {"prefill_path": self.prefill_info.get("path"), "initialize_ms": self.prefill_info.get("init_ms"),
                 "segments": segment_stats(self.out, self.round_sizes, self.round_ns, self.owner.config.think_end_token_id,
                                           self.accepted)}
        stats["accepted_prefix_histogram"] = acceptance_histogram(self.accepted)
        tot = stats["segments"].get("total")
        if tot:
            stats["decode_tok_s_device"] = tot["device_tok_s"]
        self.owner._park(self)
        return stats


class SessionEngine:
    def __init__(self, engine: Engine, store_gb: float = 8.0, ahead: int = 4, max_output_tokens: int = 524288,
                 resume_policy: str = "cost", cancel_timeout_s: float = 30.0, host_store: bool = False, tokenizer=None):
        self.engine, self.ahead, self.resume_policy, self.cancel_timeout_s = engine, ahead, resume_policy, cancel_timeout_s
        self.tokenizer = tokenizer                       # optional: enables incremental tokenisation in align_prompt
        spec = engine.spec
        self.config = EngineConfig(engine.round.capacity, max_output_tokens, tuple(spec.stop_token_ids), spec.think_end_token_id)
        full, rings = [], []
        for d in engine.target.layers:
            if d["kind"] == FULL_DSA:
                full += [d["k"], d["v"], d["ik"], d["iks"]]
            else:
                rings += [d["k"], d["v"]]
        for L in engine.round.draft.layers:
            full += [L["k"], L["v"]]
        self.store = PrefixStore(full, rings, int(store_gb * (1 << 30)), host=host_store)
        self.active: Optional[Session] = None
        self._sampled: Dict[str, List[int]] = {}

    # ------------------------------------------------------------------
    def _entry_text(self, key: str, position: int) -> str:
        """Decoded text of a parked sequence up to ``position`` (cached on the entry)."""
        e = self.store.entries[key]
        cache = e.__dict__.setdefault("_text", {})
        if position not in cache:
            cache[position] = self.tokenizer.decode(list(e.tokens[:position]))
        return cache[position]

    def align_prompt(self, tokens: Sequence[int], session_id: Optional[str], text: Optional[str] = None) -> List[int]:
        """Incremental tokenisation: keep the ids the model actually wrote for a parked history.

        ``tokens`` is the canonical encoding of the rendered prompt ``text``.  Re-encoding text that the model
        generated need not reproduce the sampled ids (the sampler may have split a word differently from the
        encoder); the token-level prefix match then stops early and the parked KV is wasted.  When no parked
        sequence matches by ids but the decoded text of one (at its park position or at one of its ring
        checkpoints, longest first, the session's own key first on ties) is a proper prefix of ``text``, the
        result is the parked ids up to that position followed by the encoding of the remaining text alone.
        Needs ``self.tokenizer`` (``decode(ids) -> str``, ``encode(str) -> ids``); without it, without ``text`` or
        without a match the canonical ids are returned unchanged.
        Parity: naivert/backends/naive_n0p5_session_engine.py:411-454."""
        tokens = [int(t) for t in tokens]
        if self.tokenizer is None or text is None or not self.store.entries:
            return tokens
        if select_resume(self.store.entries, tokens, session_id) is not None:
            return tokens
        keys = list(self.store.entries)
        own = [k for k in keys if session_id is not None and (k == session_id or k.split("#")[0] == session_id)]
        keys = own + [k for k in keys if k not in own]
        points = []
        for order, k in enumerate(keys):
            e = self.store.entries[k]
            for pos in {e.position, *(c.position for c in e.checkpoints)}:
                if 0 < pos <= len(e.tokens):
                    points.append((-pos, order, k, pos))
        for _, _, k, pos in sorted(points):
            parked = self._entry_text(k, pos)
            if not parked or len(parked) >= len(text) or not text.startswith(parked):
                continue
            enc = self.tokenizer.encode(text[len(parked):])
            suffix = [int(t) for t in (enc if not hasattr(enc, "input_ids") else enc.input_ids)]
            aligned = list(self.store.entries[k].tokens[:pos]) + suffix
            vocab = self.engine.spec.vocab
            if not suffix or any(not 0 <= t < vocab for t in aligned):
                return tokens
            return aligned
        return tokens

    def open_session(self, tokens: Sequence[int], max_decode: int, session_id: Optional[str],
                     sampling: Optional[SamplingParams] = None, use_graphs: bool = True) -> Session:
        if self.active is not None and not self.active.closed:
            raise RuntimeContractError("one sequence at a time: finish the active session first")
        tokens = [int(t) for t in tokens]
        n = len(tokens)
        cap = self.config.capacity
        if n < 1 or n + max_decode + 32 > cap:
            raise RuntimeContractError(f"prompt {n} + decode {max_decode} exceeds capacity {cap}")
        t0 = time.perf_counter()
        choice = select_resume(self.store.entries, tokens, session_id)
        start = 0
        if choice is not None:
            new_after = n - 1 - choice.position
            # restoring costs a device copy; replaying a handful of tokens can be cheaper
            gb = self.store.entries[choice.key].nbytes() / (1 << 30)
            if prefill_estimate(n - 1, "replay") - prefill_estimate(new_after, "replay") > gb * RESTORE_MS_PER_GB:
                start = self.store.restore(choice)
        near = None
        if start == 0 and self.store.entries:
            near = best_prefix_match(self.store.entries, tokens)
            if near is not None and near[1] >= 16:
                log.info("no parked prefix resumes this prompt; closest is %s: %d of its %d parked tokens match, the prompt "
                         "departs at token %d", near[0], near[1], self.store.entries[near[0]].position, near[1])
        t1 = time.perf_counter()
        path = prefill_path(n - 1 - start, self.resume_policy, native_ready=self.engine.prefill is not None)
        prompt = torch.tensor(tokens, dtype=torch.int32)
        replay_from = start
        if path == "native":
            replay_from = self.engine.prefill_native(prompt, start)
        self.engine.round.initialize(prompt, max_decode, sampling or SamplingParams(), use_graphs=use_graphs,
                                     start_pos=replay_from)
        t2 = time.perf_counter()
        # ring state at prompt end, for later rewinds; it stays with this session until the sequence it belongs to
        # is parked (a checkpoint filed under the bare session key could end up beside another branch's tokens)
        ring_ck = self.store.make_checkpoint(n - 1) if n - 1 >= 16 else None
        info = {"path": path, "restore_ms": round((t1 - t0) * 1e3, 3), "init_ms": round((t2 - t1) * 1e3, 3),
                "resumed_from": choice.key if start else None,
                "closest_parked": {"key": near[0], "common_tokens": near[1]} if near is not None else None, "estimate_ms": round(prefill_estimate(n - 1 - start, path), 2),
                "phases": {"restore_ms": round((t1 - t0) * 1e3, 3), "executor_ms": self.engine.last_prefill.get("executor_ms", 0.0),
                           "native_rows": self.engine.last_prefill.get("native_rows", 0), "replay_rows": n - 1 - replay_from,
                           "init_ms": round((t2 - t1) * 1e3, 3)}}
        self.active = Session(self, tokens, start, session_id, info)
        self.active.ring_checkpoint = ring_ck
        return self.active

    def _park(self, s: Session) -> None:
        ctrl = self.engine.target.ctrl.tolist()
        position = int(ctrl[0])                           # rows valid in the caches (the anchor row is not)
        seq = s.prompt + s.out
        if position < 16 or position > len(seq):
            return
        name = park_name(self.store.entries, s.session_id, seq)
        ck = getattr(s, "ring_checkpoint", None)
        self.store.save(name, seq, position, checkpoints=[ck] if ck is not None else None)

    def close(self) -> None:
        self.store.clear()
        self.engine.close()
