"""Tensor ABI of one rank: every weight and cache tensor the runtimes expect, as pure data.

``rank_tensor_abi(spec, rank, tp)`` expands a model specification into slots - id, domain (``parameter`` or
``cache``), index inside the domain, shape, element type, byte alignment and layout - without touching a tensor, so
shard sizes can be planned and a checkpoint's slices checked before any device memory is committed
(``parameter_bytes`` is what a rank uploads: ~40 GB per rank for the full model at 8 ranks).
``check_rank_weights`` walks a prepared weights dictionary (``models.weights.shard_weights`` /
``models.checkpoint.load_rank_weights_sliced`` / ``models.device_init``) and names the first slot whose tensor is
missing or has another shape or element type; the checkpoint loader calls it before the upload.

Layouts: ``row_major`` (as in the checkpoint; the 128-byte shared-memory swizzle is applied by the TMA unit on load, so
no tensor is stored pre-swizzled) and ``e4m3_block128`` (e4m3 payload ``.w`` plus one fp32 scale per 128 x 128 block
``.s``, listed as two slots).

Reference counterpart: naivert/tensor_abi.py (``TensorSlotAbi``, ``ModelTensorAbi``) and the slot tables of
naivert/models/naive_n0p5/model.py.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

from .spec import FULL_DSA, ModelSpec

ELEMENT_BYTES = {"bf16": 2, "f32": 4, "e4m3": 1, "u8": 1, "i32": 4}
_TORCH_NAMES = {"bf16": ("torch.bfloat16",), "f32": ("torch.float32",), "e4m3": ("torch.float8_e4m3fn", "torch.uint8"),
                "u8": ("torch.uint8",), "i32": ("torch.int32",)}
DOMAINS = ("parameter", "cache")
LAYOUTS = ("row_major", "e4m3_block128.payload", "e4m3_block128.scale")


@dataclass(frozen=True)
class TensorSlot:
    slot_id: str                      # path in the weights dictionary ("layers.3.gate.w") or cache name ("layers.3.k")
    domain: str
    index: int
    shape: Tuple[int, ...]
    dtype: str
    alignment: int                    # bytes; 16 for everything a TMA descriptor or a 128-bit load reads
    layout: str
    optional: bool = False            # may be None in the dictionary (a layer kind without sink bias)

    @property
    def nbytes(self) -> int:
        n = ELEMENT_BYTES[self.dtype]
        for d in self.shape:
            n *= d
        return n


@dataclass(frozen=True)
class RankTensorAbi:
    abi_id: str
    slots: Tuple[TensorSlot, ...]

    def __post_init__(self) -> None:
        ids = [s.slot_id for s in self.slots]
        if len(set(ids)) != len(ids):
            raise ValueError("tensor slot ids must be unique")
        for dom in DOMAINS:
            idx = sorted(s.index for s in self.slots if s.domain == dom)
            if idx != list(range(len(idx))):
                raise ValueError(f"{dom} slots do not cover their index range")
        for s in self.slots:
            if s.domain not in DOMAINS or s.layout not in LAYOUTS or s.dtype not in ELEMENT_BYTES:
                raise ValueError(f"slot {s.slot_id}: unknown domain, layout or element type")
            if s.alignment <= 0 or s.alignment & (s.alignment - 1):
                raise ValueError(f"slot {s.slot_id}: alignment must be a power of two")
            if any(d <= 0 for d in s.shape):
                raise ValueError(f"slot {s.slot_id}: empty dimension in {s.shape}")

    def domain(self, name: str) -> List[TensorSlot]:
        return [s for s in self.slots if s.domain == name]

    def slot(self, slot_id: str) -> TensorSlot:
        for s in self.slots:
            if s.slot_id == slot_id:
                return s
        raise KeyError(slot_id)

    @property
    def parameter_bytes(self) -> int:
        return sum(s.nbytes for s in self.domain("parameter"))

    @property
    def cache_bytes(self) -> int:
        return sum(s.nbytes for s in self.domain("cache"))


class _Builder:
    def __init__(self) -> None:
        self.slots: List[TensorSlot] = []
        self.count: Dict[str, int] = {d: 0 for d in DOMAINS}

    def add(self, slot_id: str, domain: str, shape, dtype: str, layout: str = "row_major", optional: bool = False) -> None:
        self.slots.append(TensorSlot(slot_id, domain, self.count[domain], tuple(int(d) for d in shape), dtype, 16, layout, optional))
        self.count[domain] += 1

    def linear(self, slot_id: str, rows: int, cols: int, fp8: bool, lead: Tuple[int, ...] = ()) -> None:
        """A linear weight [rows, cols] (optionally stacked over experts): block-scaled e4m3 or bf16."""
        if fp8:
            self.add(slot_id + ".w", "parameter", lead + (rows, cols), "e4m3", "e4m3_block128.payload")
            self.add(slot_id + ".s", "parameter", lead + (-(-rows // 128), -(-cols // 128)), "f32", "e4m3_block128.scale")
        else:
            self.add(slot_id + ".w", "parameter", lead + (rows, cols), "bf16")


def rank_tensor_abi(spec: ModelSpec, rank: int, tp: int, capacity: int = 0) -> RankTensorAbi:
    """Slots of the target model at rank ``rank`` of ``tp``.  ``capacity`` > 0 adds the KV / indexer cache slots of a context of that many
    positions (sliding-window layers keep ``sliding_window`` + a multiple-of-128 margin; their ring is listed at the window)."""
    if tp < 1 or not 0 <= rank < tp:
        raise ValueError("rank outside the tensor-parallel group")
    fp8 = spec.weight_dtype == "fp8"
    H, ix, rt = spec.hidden, spec.indexer, spec.routing
    b = _Builder()
    b.add("embed", "parameter", (spec.vocab, H), "bf16")
    b.add("norm", "parameter", (H,), "bf16")
    b.add("lm_head", "parameter", (spec.vocab_shard(tp), H), "bf16")
    for L, kind in enumerate(spec.layer_kinds):
        a = spec.attention[kind]
        p = f"layers.{L}."
        nh, kvs = a.local_heads(tp), a.kv_head_for_rank(rank, tp)
        b.add(p + "g_in", "parameter", (H,), "bf16")
        b.add(p + "g_post", "parameter", (H,), "bf16")
        b.add(p + "wq", "parameter", (nh * a.head_dim, H), "bf16")
        b.add(p + "wk", "parameter", (len(kvs) * a.head_dim, H), "bf16")
        b.add(p + "wv", "parameter", (len(kvs) * a.v_head_dim, H), "bf16")
        b.linear(p + "wo", H, nh * a.v_head_dim, fp8)
        if a.sink_bias:
            b.add(p + "sink", "parameter", (nh,), "bf16", optional=True)
        if kind == FULL_DSA:
            b.add(p + "iwq", "parameter", (ix.head_count * ix.head_dim, H), "bf16")
            b.add(p + "iwk", "parameter", (ix.head_dim, H), "bf16")
            b.add(p + "iww", "parameter", (ix.head_count, H), "bf16")
            b.add(p + "ik_w", "parameter", (ix.head_dim,), "bf16")
            b.add(p + "ik_b", "parameter", (ix.head_dim,), "bf16")
        if spec.is_dense(L):
            I = spec.dense_inter_local(tp)
            b.linear(p + "dense.gate", I, H, fp8)
            b.linear(p + "dense.up", I, H, fp8)
            b.linear(p + "dense.down", H, I, fp8)
        else:
            I = spec.expert_inter_local(tp)
            E = rt.expert_count + rt.shared_expert_count
            b.add(p + "router_w", "parameter", (rt.expert_count, H), "f32")
            b.add(p + "router_b", "parameter", (rt.expert_count,), "f32")
            b.linear(p + "gate", I, H, fp8, (E,))
            b.linear(p + "up", I, H, fp8, (E,))
            b.linear(p + "down", H, I, fp8, (E,))
        if capacity > 0:
            rows = capacity if kind == FULL_DSA else min(capacity, a.sliding_window or capacity)
            b.add(p + "k", "cache", (rows, len(kvs), a.head_dim), "bf16")
            b.add(p + "v", "cache", (rows, len(kvs), a.v_head_dim), "bf16")
            if kind == FULL_DSA:
                b.add(p + "ik", "cache", (capacity, ix.head_dim), "e4m3")
                b.add(p + "iks", "cache", (capacity,), "f32")
    return RankTensorAbi(f"{spec.name}.tp{tp}.rank{rank}.{'w8a8' if fp8 else 'bf16'}", tuple(b.slots))


def _lookup(weights: dict, slot_id: str):
    cur = weights
    for part in slot_id.split("."):
        if isinstance(cur, (list, tuple)):
            cur = cur[int(part)]
        elif isinstance(cur, dict):
            if part not in cur:
                return None, False
            cur = cur[part]
        else:
            return None, False
    return cur, True


def check_rank_weights(spec: ModelSpec, weights: dict, rank: int, tp: int, abi: Optional[RankTensorAbi] = None) -> RankTensorAbi:
    """Raise ``ValueError`` naming the first parameter slot that ``weights`` does not fill as declared."""
    abi = abi or rank_tensor_abi(spec, rank, tp)
    if len(weights.get("layers", ())) != spec.layer_count:
        raise ValueError(f"{abi.abi_id}: {len(weights.get('layers', ()))} layers in the weights, {spec.layer_count} in the model")
    strict_dtype = spec.weight_dtype in ("fp8", "bf16")          # fp32 oracle geometries keep their own element types
    for s in abi.domain("parameter"):
        t, found = _lookup(weights, s.slot_id)
        if t is None:
            if found and s.optional:
                continue
            raise ValueError(f"{abi.abi_id}: slot {s.slot_id} is missing")
        if tuple(t.shape) != s.shape:
            raise ValueError(f"{abi.abi_id}: slot {s.slot_id} has shape {tuple(t.shape)}, the model needs {s.shape}")
        if strict_dtype and str(t.dtype) not in _TORCH_NAMES[s.dtype]:
            raise ValueError(f"{abi.abi_id}: slot {s.slot_id} has element type {t.dtype}, the model needs {s.dtype}")
    return abi
