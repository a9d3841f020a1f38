"""The speculative round: draft ingest -> draft block -> 7 proposals -> target verify-8 ->
sharded sampler / verify -> tail commit, captured once as a CUDA graph per rank whose kernels
are chained with programmatic dependent launch.  Ranks stay in lockstep purely through the
tagged words of the fabric; the host only launches graphs ahead and polls a pinned ring.

Control block (int32, device): [0] position of the anchor row, [1] rows to ingest,
[2] first ingest position, [4] stopped, [5] stop reason, [6] tokens produced, [7] token limit,
[8] round counter, [9] KV capacity, [10] prompt replay cursor, [11] prompt rows to replay.

Parity: ``DraftRound`` (naivert/backends/naive_n0p5_draft_round.py:17-191: phase list :49-58,
``set_sampling`` :97-123, ``initialize`` :125-179, ``launch`` :181-184), ``DraftTarget`` and
``DraftTail`` (naivert/backends/naive_n0p5_draft_target.py, ..._draft_tail.py), the host ring
poll of ``Session.step`` (naivert/backends/naive_n0p5_session_engine.py:288-323).
"""
from __future__ import annotations

import ctypes as C
import time
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ..models.spec import ModelSpec, SamplingParams
from ..ops import kernels as K
from .contract import (CTRL_CAPACITY, CTRL_CURSOR, CTRL_MAX_TOKENS, CTRL_PROMPT_CTX, STOP_REASONS)
from .draft import DraftRuntime
from .modes import request_fits
from .target import PAD_ROWS, TargetRuntime

RING_SIZE = 1024


class RuntimeContractError(RuntimeError):
    """A request violates a bound the captured graphs were built for."""


@dataclass
class RoundRecord:
    round: int
    tokens: List[int]
    pos0: int
    accepted: int
    stop_reason: Optional[str]
    t_end_ns: int


class HostRing:
    """Pinned, device-mapped ring of fixed-size round records plus the cancel word."""

    def __init__(self, size: int = RING_SIZE):
        self.size = size
        nbytes = size * C.sizeof(K.RingRecord) + 64
        self.host, self.dev = K.host_alloc_mapped(nbytes)
        self.records = (K.RingRecord * size).from_address(self.host)
        self.cancel_host = self.host + size * C.sizeof(K.RingRecord)
        self.cancel_dev = self.dev + size * C.sizeof(K.RingRecord)
        self.cancel = C.c_int.from_address(self.cancel_host)
        self.consumed = C.c_int.from_address(self.cancel_host + 16)      # rounds the host has read (device chain backpressure)
        self.consumed_dev = self.cancel_dev + 16

    def clear(self):
        C.memset(self.host, 0, self.size * C.sizeof(K.RingRecord) + 64)

    def poll(self, rnd: int) -> Optional[RoundRecord]:
        rec = self.records[rnd % self.size]
        if rec.generation != rnd + 1:
            return None
        toks = [int(t) for t in rec.tokens[: rec.count]]
        return RoundRecord(rnd, toks, rec.pos0, rec.accepted, STOP_REASONS.get(rec.stop_reason, "unknown"), rec.t_end_ns)

    def close(self):
        if self.host:
            K.host_free(self.host)
            self.host = 0


class SpeculativeRound:
    def __init__(self, spec: ModelSpec, target: TargetRuntime, draft_weights: dict, capacity: int, pdl: bool = True,
                 device_chain: bool = False, ring_size: int = RING_SIZE):
        if target.rows != spec.draft.rows:
            raise RuntimeContractError("the verify runtime must run block_size + 1 rows")
        self.spec, self.t, self.fab, self.pdl = spec, target, target.fab, pdl
        dev = target.dev
        self.tp, self.rank = target.tp, target.rank
        V = spec.vocab_shard(self.tp)
        self.vlocal, self.vbase = V, self.rank * V
        self.block_ids = target.tokens                          # verify tokens == draft block ids
        self.params = torch.zeros(8, dtype=torch.float32, device=dev)
        self.seed = torch.zeros(1, dtype=torch.int64, device=dev)
        self.codes = torch.zeros(15, V, dtype=torch.int32, device=dev)
        self.counts = torch.zeros(V, dtype=torch.int16, device=dev)
        self.state = torch.zeros(K.sampler_state_bytes() // 8 + 1, dtype=torch.int64, device=dev)
        self.stop_ids = torch.tensor(list(spec.stop_token_ids) or [-1], dtype=torch.int32, device=dev)
        import os
        self.sampler_one_launch = target.fused and os.environ.get("NAIVERT_SAMPLER_PERSISTENT", "1") == "1"
        self.sampler_sync = torch.zeros(2, dtype=torch.int64, device=dev)
        self.ring = HostRing(ring_size)
        self.draft = DraftRuntime(spec, draft_weights, target, capacity, self.seed, self.params, self.block_ids, pdl=pdl)
        self.capacity = capacity
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.prefill_graph: Optional[torch.cuda.CUDAGraph] = None
        self.prompt_dev = torch.zeros(capacity, dtype=torch.int32, device=dev)
        self.n_prompt = 0
        self.use_penalties = False
        self.kernels_per_round = 0
        # device chain: the round graph is instantiated for device launch and relaunches itself from its
        # last kernel; the host launches once per request and polls the ring
        self.device_chain = device_chain
        self.nudge_s = 0.5                                  # silence after which a paused chain is restarted
        self.native_graph: Optional[K.NativeGraph] = None
        self.chain_started = False
        self.host_launches = 0
        self._build_args()
        self.stream = torch.cuda.Stream(device=dev)

    def _build_args(self):
        s = K.SamplerArgs()
        s.zp, s.ldp = self.t.logits.data_ptr(), self.t.logits.shape[1]
        s.zq, s.ldq = self.draft.zq.data_ptr(), self.draft.zq.shape[1]
        s.vlocal, s.vbase, s.e = self.vlocal, self.vbase, self.codes.data_ptr()
        s.counts = None
        s.params, s.seed = self.params.data_ptr(), self.seed.data_ptr()
        s.ctrl, s.block_ids = self.t.ctrl.data_ptr(), self.block_ids.data_ptr()
        s.n_rows_p, s.n_rows_q = 8, 7
        s.st = self.state.data_ptr()
        s.x = self.fab.xchg_args()
        self.args_sampler = s
        t = K.TailArgs()
        t.ctrl, t.block_ids, t.epoch = self.t.ctrl.data_ptr(), self.block_ids.data_ptr(), self.fab.epoch.data_ptr()
        t.st, t.ring, t.ring_size = self.state.data_ptr(), self.ring.dev, self.ring.size
        t.cancel, t.stop_ids, t.n_stop = self.ring.cancel_dev, self.stop_ids.data_ptr(), len(self.spec.stop_token_ids)
        t.counts, t.vbase, t.vlocal = None, self.vbase, self.vlocal
        t.status, t.n_rows_q = self.fab.status.data_ptr(), 7
        t.host_consumed = self.ring.consumed_dev if self.device_chain else None     # pause consensus of the chain
        t.x = self.fab.xchg_args()
        self.args_tail = t

    # ------------------------------------------------------------------ sampling controls
    def set_sampling(self, sp: SamplingParams) -> None:
        sp.validate()
        penal = (sp.repetition_penalty != 1.0 or sp.frequency_penalty != 0.0 or sp.presence_penalty != 0.0)
        if penal != self.use_penalties:
            self.use_penalties = penal
            self.args_sampler.counts = self.counts.data_ptr() if penal else None
            self.args_tail.counts = self.counts.data_ptr() if penal else None
            self.graph = None                              # pointers are baked into the captured nodes
        forced = -1.0 if sp.forced_accept_p is None else float(sp.forced_accept_p)
        vals = [1.0 / sp.temperature, sp.clamped_top_p(), sp.repetition_penalty, sp.frequency_penalty,
                sp.presence_penalty, forced, 1.0 / sp.temperature, 0.0]
        self.params.copy_(torch.tensor(vals, dtype=torch.float32))
        self.seed.fill_(sp.seed)

    # ------------------------------------------------------------------ phases
    def phases(self) -> None:
        """Enqueue one round on the current stream."""
        self.draft.ingest()
        self.draft.block()
        self.draft.propose()
        self.t.step()
        self.sample()
        K.tail_commit(self.args_tail, pdl=self.pdl)

    def sample(self, domain: int = 1, one_launch: Optional[bool] = None) -> None:
        """Verify + resample on the logits in place: the single-launch sampler, or the nine-kernel chain where its
        grid cannot be resident at once (or when ``one_launch`` is False)."""
        want = self.sampler_one_launch if one_launch is None else one_launch
        if want and K.sampler_persistent(self.args_sampler, self.sampler_sync, domain=domain, pdl=self.pdl) == 0:
            return
        if one_launch is None:
            self.sampler_one_launch = False
        K.sampler_run(self.args_sampler, domain=domain, pdl=self.pdl)

    def prefill_phases(self) -> None:
        """One 8-row prompt replay step: target rows (no head) + draft ingest of their features."""
        K.prefill_cursor(self.prompt_dev, -1, self.t.rows, self.t.ctrl, self.t.tokens, pdl=self.pdl)
        self.t.step(head=False)
        self.draft.ingest()
        K.epoch_advance(self.fab.epoch, pdl=self.pdl)

    def _capture(self, fn) -> torch.cuda.CUDAGraph:
        torch.cuda.synchronize()
        with torch.cuda.stream(self.stream):
            fn()                                          # warm-up (loads modules, sets attributes)
        self.stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=self.stream):
            fn()
        return g

    # ------------------------------------------------------------------ request lifecycle
    def initialize(self, prompt: torch.Tensor, max_tokens: int, sp: SamplingParams, use_graphs: bool = True,
                   start_pos: int = 0) -> None:
        """Reset the session state, replay the prompt (all but its last token, which becomes
        the first anchor) and arm the control block.  ``prompt`` may live in pinned host memory.
        ``start_pos`` context rows are already valid in the caches (a restored prefix): replay
        starts there."""
        n = int(prompt.numel())
        if not request_fits(n, max_tokens, self.capacity, PAD_ROWS):
            raise RuntimeContractError(f"prompt {n} + decode {max_tokens} does not fit capacity {self.capacity}")
        self.set_sampling(sp)
        self.ring.clear()
        self.ring.cancel.value = 0
        self.prompt_dev[:n].copy_(prompt.to(torch.int32), non_blocking=True)
        self.n_prompt, self.n_prompt_ctx = n, n - 1
        ctrl = torch.zeros(16, dtype=torch.int32)
        if not 0 <= start_pos <= n - 1:
            raise RuntimeContractError(f"resume position {start_pos} outside the prompt context 0..{n - 1}")
        ctrl[CTRL_MAX_TOKENS], ctrl[CTRL_CAPACITY], ctrl[CTRL_CURSOR], ctrl[CTRL_PROMPT_CTX] = max_tokens, self.capacity, start_pos, n - 1
        self.t.ctrl.copy_(ctrl)
        self.counts.zero_()
        self.fab.status.zero_()
        steps = -(-(n - 1 - start_pos) // self.t.rows)
        if steps:
            if use_graphs:
                if self.prefill_graph is None:
                    self.prefill_graph = self._capture_prefill()
                with torch.cuda.stream(self.stream):
                    for _ in range(steps):
                        self.prefill_graph.replay()
            else:
                with torch.cuda.stream(self.stream):
                    for _ in range(steps):
                        self.prefill_phases()
        with torch.cuda.stream(self.stream):
            # arm: anchor = last prompt token at position n-1; the last replay chunk is re-ingested by round 0
            last_chunk = start_pos + max(0, (steps - 1) * self.t.rows)
            if steps == 0:
                # nothing was replayed: the feature rows are stale, so round 0 must not overwrite valid
                # draft context; point its (harmless) ingest beyond the context instead
                last_chunk = n - 1
            arm = torch.tensor([n - 1, min(self.t.rows, max(0, n - 1 - last_chunk)), last_chunk], dtype=torch.int32)
            self.t.ctrl[:3].copy_(arm.to(self.t.dev))
            self.block_ids[0:1].copy_(self.prompt_dev[n - 1:n])
            if self.use_penalties:
                self._count_prompt(n)
        self.stream.synchronize()
        self.fab.check()
        if use_graphs and self.graph is None:
            self._snapshot_and_capture()
        self.next_round = 0
        self.launched = 0
        self.use_graphs = use_graphs
        self.chain_started = False
        self.host_launches = 0
        self.ring.consumed.value = 0

    def _capture_prefill(self):
        saved = self.t.ctrl.clone()
        g = self._capture(self.prefill_phases)
        self.t.ctrl.copy_(saved)
        return g

    def _snapshot_and_capture(self):
        """Capture the round graph; the warm-up run inside capture mutates session state, so
        the control block, the block ids and the feature rows of the last replay chunk are restored
        (KV rows it wrote lie at or beyond the anchor and are rewritten by round 0)."""
        saved_ctrl, saved_ids, saved_feats = self.t.ctrl.clone(), self.block_ids.clone(), self.t.feats.clone()
        self.ring.cancel.value = 1                       # the warm-up round commits nothing
        before = K.LAUNCHES["count"]
        if self.device_chain:
            self.graph = self._capture_native()
        else:
            self.graph = self._capture(self.phases)
        self.kernels_per_round = (K.LAUNCHES["count"] - before) // 2     # warm-up + capture
        self.stream.synchronize()
        self.ring.cancel.value = 0
        self.ring.clear()
        self.t.ctrl.copy_(saved_ctrl)
        self.block_ids.copy_(saved_ids)
        self.t.feats.copy_(saved_feats)                  # round 0 re-ingests the last replay chunk's features
        self.fab.status.zero_()
        torch.cuda.synchronize()

    def _capture_native(self):
        """Capture through the runtime API, append the relaunch kernel, instantiate for device launch."""
        torch.cuda.synchronize()
        with torch.cuda.stream(self.stream):
            self.phases()                                   # warm-up (a cancelled round)
        self.stream.synchronize()
        g = K.NativeGraph()
        sid = self.stream.cuda_stream
        with torch.cuda.stream(self.stream):
            g.begin(sid)
            try:
                self.phases()
                K.relaunch(self.t.ctrl, 0, self.ring.size)      # pause decided by the tail (rank consensus)
            finally:
                g.end(sid)
        g.instantiate(True, sid)
        self.stream.synchronize()
        self.native_graph = g
        return g

    def _count_prompt(self, n: int):
        toks = self.prompt_dev[:n].long() - self.vbase
        toks = toks[(toks >= 0) & (toks < self.vlocal)]
        self.counts.zero_()
        self.counts.index_add_(0, toks, torch.ones_like(toks, dtype=torch.int16))

    def launch(self, n: int = 1, force: bool = False) -> None:
        """Enqueue ``n`` rounds.  With the device chain one host launch starts a self-relaunching chain;
        further calls are no-ops unless ``force`` (a stalled or finished chain is restarted by the host)."""
        if self.device_chain and self.use_graphs:
            if not self.chain_started or force:
                self.native_graph.launch(self.stream.cuda_stream)
                self.chain_started = True
                self.host_launches += 1
            return
        with torch.cuda.stream(self.stream):
            for _ in range(n):
                if self.use_graphs:
                    self.graph.replay()
                else:
                    self.phases()
        self.launched += n
        self.host_launches += n

    def poll(self) -> Optional[RoundRecord]:
        rec = self.ring.poll(self.next_round)
        if rec is not None:
            self.next_round += 1
            self.ring.consumed.value = self.next_round
        return rec

    def wait_round(self, timeout_s: float = 120.0) -> RoundRecord:
        t0 = time.monotonic()
        nudged = False
        while True:
            rec = self.poll()
            if rec is not None:
                return rec
            if self.device_chain and self.use_graphs and not nudged and time.monotonic() - t0 > self.nudge_s:
                self.launch(force=True)                      # the chain paused for backpressure: restart it
                nudged = True
            if time.monotonic() - t0 > timeout_s:
                raise RuntimeError(f"round {self.next_round} did not publish within {timeout_s}s")
            time.sleep(50e-6)

    def cancel(self) -> None:
        self.ring.cancel.value = 1

    def close(self) -> None:
        self.ring.close()
