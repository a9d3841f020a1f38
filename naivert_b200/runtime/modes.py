"""Decode modes as data: what each mode launches, which buffers it reads and writes, and the call-index plans.

A mode names the kernel entry points it needs (``ops.variants``; the engine requires them from the loaded library
before capturing anything), the token rows of a step, and its buffer table: for every pointer the kernels of the mode
receive, who owns the storage (``owned``: allocated by the runtime named in ``owner``; ``borrowed``: a view of another
runtime's tensor; ``null``: not used in this mode) and its size as expressions over the model specification.

Two index plans live here because every rank must derive the same numbers without talking:

* all-reduce call indices inside one step epoch - target layer ``L`` uses ``2L`` (attention output) and ``2L + 1``
  (MLP / MoE output), the draft block uses ``200 ..``; the mailbox tag is ``epoch * 1024 + call + 1`` and the slab is
  ``call % 4``, so calls that follow each other must differ modulo 4;
* small-exchange call indices (sampler, Markov head, EP counts, arg-max; tag ``epoch * 64 + call + 1``), same slab rule:
  a peer may already push call ``n + 1`` while this rank still polls call ``n``.

Reference counterpart: naivert/decode_modes.py (``DecodeModeSpec``, ``runtime_memory_abi``, ``mailbox_layer_tags``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

from ..models.spec import ModelSpec

MAILBOX_CALLS = 1024          # call indices per epoch of the all-reduce mailbox (csrc/gemm.cuh)
MAILBOX_SLABS = 4
XCHG_CALLS = 64               # call indices per epoch of the small exchange (csrc/fabric.cuh)
XCHG_SLABS = 4
DRAFT_CALL_BASE = 200


@dataclass(frozen=True)
class BufferRecord:
    name: str
    owner: str                # target | draft | round | session
    storage: str              # owned | borrowed | null
    rows: str                 # expression over the spec / mode ("rows", "16", "capacity", "0")
    row_bytes: str            # expression ("hidden * 2", "vocab_shard * 4", ...)


@dataclass(frozen=True)
class DecodeMode:
    mode_id: str
    rows: int                               # token rows per step (0: chunked)
    uses_draft: bool
    entries: Tuple[str, ...]                # extern "C" launchers (ops.variants)
    buffers: Tuple[BufferRecord, ...]

    @property
    def pointer_fields(self) -> Tuple[str, ...]:
        return tuple(b.name for b in self.buffers)


POINTER_FIELDS = ("control_state", "input_tokens", "input_hidden", "target_logits", "feature_taps", "kv_cache",
                  "indexer_cache", "block_ids", "draft_hidden", "draft_logits", "draft_cache", "sampler_state", "host_ring")
DRAFT_ONLY = frozenset({"block_ids", "draft_hidden", "draft_logits", "draft_cache", "sampler_state", "feature_taps"})


def buffer_table(rows: int, draft: bool, ring: bool) -> Tuple[BufferRecord, ...]:
    out: List[BufferRecord] = []
    for name in POINTER_FIELDS:
        if (name in DRAFT_ONLY and not draft) or (name == "host_ring" and not ring):
            out.append(BufferRecord(name, "-", "null", "0", "0"))
        elif name == "control_state":
            out.append(BufferRecord(name, "target", "owned", "1", "16 * 4"))
        elif name == "input_tokens":
            out.append(BufferRecord(name, "target", "owned", "16", "4"))
        elif name == "input_hidden":
            out.append(BufferRecord(name, "target", "owned", "16", "hidden * 2"))
        elif name == "target_logits":
            out.append(BufferRecord(name, "target", "owned", "16", "vocab_shard * 4"))
        elif name == "feature_taps":
            out.append(BufferRecord(name, "target", "owned", "16", "taps_local * hidden * 2"))
        elif name == "kv_cache":
            out.append(BufferRecord(name, "target", "owned", "capacity | window ring", "kv_heads_local * (head_dim + v_head_dim) * 2"))
        elif name == "indexer_cache":
            out.append(BufferRecord(name, "target", "owned", "capacity", "indexer_head_dim + 4"))
        elif name == "block_ids":
            out.append(BufferRecord(name, "round", "borrowed", "8", "4"))                 # a view of input_tokens
        elif name == "draft_hidden":
            out.append(BufferRecord(name, "draft", "owned", "16", "draft_hidden * 2"))
        elif name == "draft_logits":
            out.append(BufferRecord(name, "draft", "owned", "8", "vocab_shard * 4"))
        elif name == "draft_cache":
            out.append(BufferRecord(name, "draft", "owned", "capacity", "draft_kv_heads_local * draft_head_dim * 4"))
        elif name == "sampler_state":
            out.append(BufferRecord(name, "round", "owned", "1", "sampler_state_bytes"))
        elif name == "host_ring":
            out.append(BufferRecord(name, "round", "owned", "ring_size", "64"))           # mapped pinned host memory
    return tuple(out)


_STEP = ("nrt_step_prologue", "nrt_gemm_launch", "nrt_attn_decode", "nrt_index_sweep", "nrt_topk_rows", "nrt_router",
         "nrt_moe_layer")
_ROUND = _STEP + ("nrt_draft_block_input", "nrt_markov_chain", "nrt_markov_step", "nrt_sampler_persistent", "nrt_sampler_run",
                  "nrt_tail_commit")

MODES: Dict[str, DecodeMode] = {m.mode_id: m for m in (
    DecodeMode("greedy_step", 1, False, _STEP + ("nrt_argmax_rows",), buffer_table(1, False, False)),
    DecodeMode("verify8", 8, False, _STEP + ("nrt_argmax_rows",), buffer_table(8, False, False)),
    DecodeMode("speculative_round", 8, True, _ROUND, buffer_table(8, True, True)),
    DecodeMode("prefill_replay", 8, True, _ROUND, buffer_table(8, True, False)),
    DecodeMode("prefill_native", 0, True,
               ("nrt_wide_gemm_launch", "nrt_attn_post", "nrt_attn_group", "nrt_index_sweep", "nrt_topk_rows_grid", "nrt_router",
                "nrt_ep_count", "nrt_ep_dispatch", "nrt_ep_combine", "nrt_ag_push"), buffer_table(0, True, False)),
)}


def layer_call_tags(layer: int) -> Tuple[int, int]:
    """All-reduce call indices of target layer ``layer``: (attention output, MLP / MoE output)."""
    return 2 * int(layer), 2 * int(layer) + 1


def draft_call_tags(layer: int) -> Tuple[int, int]:
    """All-reduce call indices of draft layer ``layer`` (the block's input projection uses ``DRAFT_CALL_BASE``)."""
    return DRAFT_CALL_BASE + 1 + 2 * int(layer), DRAFT_CALL_BASE + 2 + 2 * int(layer)


def allreduce_call_plan(spec: ModelSpec) -> List[Tuple[str, int]]:
    """(name, call index) of every all-reduce of one round in launch order; raises if two collide, one falls outside
    the epoch's range, or two consecutive ones share a slab."""
    plan: List[Tuple[str, int]] = []
    for L in range(spec.layer_count):
        a, m = layer_call_tags(L)
        plan += [(f"target.{L}.attn", a), (f"target.{L}.mlp", m)]
    if spec.draft is not None:
        plan.append(("draft.input", DRAFT_CALL_BASE))
        for l in range(spec.draft.layer_count):
            a, m = draft_call_tags(l)
            plan += [(f"draft.{l}.attn", a), (f"draft.{l}.mlp", m)]
    _check_plan(plan, MAILBOX_CALLS, MAILBOX_SLABS, "all-reduce")
    return plan


# small exchanges of one round in launch order (csrc/sampler.cu, csrc/draft.cu); the EP counts (32 + call % 16) and
# the greedy arg-max (60) belong to other modes and never interleave with these
def exchange_call_plan(markov_steps: int = 7) -> List[Tuple[str, int]]:
    plan = [(f"markov.{s}", 16 + s) for s in range(markov_steps)]
    plan += [("sampler.maxima", 0), ("sampler.totals", 1)]
    for p in range(4):
        plan += [(f"sampler.nucleus{p}.bins_to_owner", 2 + 2 * p), (f"sampler.nucleus{p}.digit", 3 + 2 * p)]
    plan += [("sampler.accept", 10), ("sampler.rank_totals", 11), ("sampler.token", 12), ("tail.pause_consensus", 13)]
    _check_plan(plan, XCHG_CALLS, XCHG_SLABS, "exchange")
    return plan


def _check_plan(plan: List[Tuple[str, int]], calls: int, slabs: int, what: str) -> None:
    seen: Dict[int, str] = {}
    for i, (name, c) in enumerate(plan):
        if not 0 <= c < calls:
            raise ValueError(f"{what} call index {c} of {name} is outside one epoch (0..{calls - 1})")
        if c in seen:
            raise ValueError(f"{what} call index {c} is used by {seen[c]} and {name}")
        seen[c] = name
        if i and plan[i - 1][1] % slabs == c % slabs:
            raise ValueError(f"{what} calls {plan[i - 1][0]} and {name} follow each other in the same slab")


def request_fits(prompt_tokens: int, max_new_tokens: int, capacity: int, pad_rows: int = 16) -> bool:
    """True when every step of the request stays inside the caches: the prompt, the tokens to generate, and two padded
    steps of head room (a verify step writes ``pad_rows`` rows at the current position, and the round after the last
    committed token has already been launched when the stop is seen)."""
    return int(prompt_tokens) >= 1 and int(prompt_tokens) + int(max_new_tokens) + 2 * int(pad_rows) <= int(capacity)
