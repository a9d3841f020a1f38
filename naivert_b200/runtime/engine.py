"""Public engine API: build a (tensor-parallel) speculative decoding engine and generate.

``Engine.build`` sets up one rank (one process per GPU): the peer-memory fabric, the
rank's target and draft weights (random-init on device, or loaded from checkpoints in the
reference layout), KV caches, the verify runtime and the captured speculative round.
``Engine.generate`` runs one request: prompt replay, then rounds launched ahead of the host
while a pinned ring is polled for committed tokens.

Parity: ``SessionEngine.build/open_session`` and ``Session.step/finish``
(naivert/backends/naive_n0p5_session_engine.py:263-340,456-573,590-630,649-748).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Iterator, List, Optional

import torch

from ..models.spec import ModelSpec, SamplingParams
from ..parallel.fabric import Fabric
from .round import RING_SIZE, RoundRecord, RuntimeContractError, SpeculativeRound
from .target import TargetRuntime


@dataclass
class GenerationResult:
    tokens: List[int] = field(default_factory=list)
    rounds: int = 0
    accepted: int = 0
    stop_reason: Optional[str] = None
    device_ns: int = 0                   # first to last round-end device timestamp
    prefill_s: float = 0.0
    decode_s: float = 0.0

    @property
    def acceptance(self) -> float:
        return self.accepted / max(1, 7 * self.rounds)

    @property
    def device_tok_s(self) -> float:
        return 0.0 if self.device_ns <= 0 else (len(self.tokens) - self.first_round_tokens) / (self.device_ns * 1e-9)

    first_round_tokens: int = 0


class Engine:
    def __init__(self, spec: ModelSpec, fabric: Fabric, target: TargetRuntime, rnd: SpeculativeRound, prefill=None):
        self.spec, self.fabric, self.target, self.round = spec, fabric, target, rnd
        self.tp, self.rank = fabric.tp, fabric.rank
        self.prefill = prefill                       # NativePrefill (chunked prompt ingestion) or None: replay only
        self.native_min_rows = 96                    # shorter prompts are cheaper to replay eight rows at a time (~1.2 ms per row vs ~90 ms per chunk)
        self.last_prefill = {}

    # ------------------------------------------------------------------ construction
    @classmethod
    def build(cls, spec: ModelSpec, rank: int = 0, tp: int = 1, group=None, capacity: int = 16384, seed: int = 0,
              target_ckpt: Optional[str] = None, draft_ckpt: Optional[str] = None, device=None,
              weights: Optional[dict] = None, draft_weights: Optional[dict] = None, pdl: Optional[bool] = None,
              shape_tp: int = 0, device_chain: Optional[bool] = None, prefill_chunk: int = 0,
              ep_weights: Optional[list] = None, ring_size: int = 0) -> "Engine":
        """``prefill_chunk`` > 0 adds the chunked native prefill (rows per chunk); ``ep_weights`` (whole experts of
        this rank per layer, ``models.weights.shard_expert_weights``) selects its expert-parallel MoE path."""
        device = device or torch.device("cuda", torch.cuda.current_device())
        if pdl is None:
            # Programmatic dependent launch on every kernel (NAIVERT_PDL=0 turns it off): the next kernel's launch,
            # barrier / TMEM set-up and first weight requests run under the predecessor's tail.  Measured 4.31 vs
            # 4.43 ms per round at 8-way shapes on one GPU and 6.56 vs 6.68 ms on two GPUs (32 layers).
            import os
            pdl = os.environ.get("NAIVERT_PDL", "1") == "1"
        if spec.draft is None:
            raise RuntimeContractError("the engine needs a model with a draft specification")
        # fail closed before anything is captured if the loaded library was built from other sources than this package
        from ..ops import kernels as K, variants
        try:
            from .modes import MODES
            need = MODES["speculative_round"].entries + MODES["greedy_step"].entries
            if prefill_chunk:
                need += MODES["prefill_native"].entries
            variants.require_entries(K.lib(), dict.fromkeys(need))
        except ValueError as e:
            raise RuntimeContractError(str(e)) from e
        fabric = Fabric(rank, tp, max(spec.hidden, spec.draft.hidden), group=group, device=device)
        if shape_tp:
            if tp != 1:
                raise RuntimeContractError("shape_tp emulation needs a single-rank fabric")
            rank, tp = 0, shape_tp
        if weights is None:
            if target_ckpt is not None:
                from ..models.checkpoint import load_rank_weights
                weights, _ = load_rank_weights(spec, target_ckpt, rank, tp, device=device)
            else:
                from ..models.device_init import init_rank_weights_device
                weights = init_rank_weights_device(spec, rank, tp, seed=seed, device=device)
        if draft_weights is None:
            if draft_ckpt is not None:
                from ..models.checkpoint import load_draft_rank_weights
                draft_weights, _ = load_draft_rank_weights(spec, draft_ckpt, rank, tp, device=device)
            else:
                from ..models.device_init import init_draft_rank_weights_device
                draft_weights = init_draft_rank_weights_device(spec, rank, tp, seed=seed + 1, device=device)
        target = TargetRuntime(spec, weights, fabric, rows=spec.draft.rows, capacity=capacity, device=device, pdl=pdl,
                               shape_tp=shape_tp, prefill_chunk=prefill_chunk)
        del weights
        if device_chain is None:
            import os
            device_chain = os.environ.get("NAIVERT_DEVICE_CHAIN", "0") == "1"
        rnd = SpeculativeRound(spec, target, draft_weights, capacity, pdl=pdl, device_chain=device_chain,
                               ring_size=ring_size or RING_SIZE)
        prefill = None
        if prefill_chunk:
            from ..prefill.native import NativePrefill
            prefill = NativePrefill(spec, target, rnd.draft, chunk=prefill_chunk, ep_weights=ep_weights, group=group)
        return cls(spec, fabric, target, rnd, prefill)

    # ------------------------------------------------------------------ one request
    def prefill_native(self, prompt: torch.Tensor, start: int = 0) -> int:
        """Ingest prompt context rows [start, n - 1) in whole chunks where that pays; returns the position from
        which the eight-row replay has to continue."""
        n = int(prompt.numel())
        self.last_prefill = {"path": "replay", "native_rows": 0}
        if self.prefill is None or n - 1 - start < max(self.native_min_rows, self.prefill.quantum):
            return start
        if n > self.target.capacity:
            raise RuntimeContractError(f"prompt {n} exceeds the cache capacity {self.target.capacity}")
        with torch.cuda.stream(self.round.stream):
            pos = self.prefill.run(prompt, start, n - 1)
        self.last_prefill = {"path": "native", "native_rows": pos - start, "executor_ms": round(self.prefill.executor_ms(), 3)}
        self.prefill.check()
        return pos

    def open(self, prompt: torch.Tensor, max_tokens: int, sampling: Optional[SamplingParams] = None,
             use_graphs: bool = True) -> None:
        start = self.prefill_native(prompt)
        self.round.initialize(prompt, max_tokens, sampling or SamplingParams(), use_graphs=use_graphs, start_pos=start)

    def stream_rounds(self, ahead: int = 4, timeout_s: float = 120.0) -> Iterator[RoundRecord]:
        """Launch rounds ``ahead`` of the host and yield each round's record as it is published."""
        r = self.round
        r.launch(ahead)
        while True:
            rec = r.wait_round(timeout_s)
            yield rec
            if rec.stop_reason is not None:
                break
            r.launch(1)
        r.stream.synchronize()
        self.fabric.check()

    def generate(self, prompt: torch.Tensor, max_tokens: int, sampling: Optional[SamplingParams] = None,
                 ahead: int = 4, use_graphs: bool = True) -> GenerationResult:
        res = GenerationResult()
        t0 = time.perf_counter()
        self.open(prompt, max_tokens, sampling, use_graphs=use_graphs)
        t1 = time.perf_counter()
        first_ns = None
        last_ns = 0
        for rec in self.stream_rounds(ahead=ahead):
            res.tokens.extend(rec.tokens)
            res.rounds += 1
            res.accepted += rec.accepted
            if first_ns is None:
                first_ns = rec.t_end_ns
                res.first_round_tokens = len(rec.tokens)
            last_ns = rec.t_end_ns
            res.stop_reason = rec.stop_reason
        res.device_ns = last_ns - (first_ns or last_ns)
        res.prefill_s, res.decode_s = t1 - t0, time.perf_counter() - t1
        return res

    def kv_bytes(self) -> int:
        return self.target.kv_bytes() + self.round.draft.kv_bytes()

    def close(self) -> None:
        if self.prefill is not None:
            self.prefill.close()
        self.round.close()
        self.fabric.close()
