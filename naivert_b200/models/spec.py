"""Model description types.

One set of frozen dataclasses describes every geometry the engine can run: the
full Naive-N0.5-Flash target, its block-draft model, and reduced geometries for
CPU tests.  Tensor-parallel degree is a *runtime* parameter of every derived
quantity (``local_heads(tp)``, ``kv_head_for_rank(rank, tp)`` ...) instead of a
compile-time macro.

Parity: the reference keeps the same information in ``naivert/model.py``
(``AttentionLayout`` :425, ``SparseIndexerSpec`` :495, ``MoeRoutingSpec`` :512,
``HybridModelSpec`` :535) and ``naivert/models/naive_n0p5/model.py:28-93``.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Mapping, Optional, Tuple

FULL_DSA = "full_dsa"
SLIDING_WINDOW = "sliding_window"


@dataclass(frozen=True)
class AttentionLayout:
    """Per-kind attention geometry (query heads are TP-sharded, KV heads shared)."""

    kind: str
    head_count: int
    kv_head_count: int
    head_dim: int          # q/k width (rope + nope)
    v_head_dim: int
    rope_dim: int
    rope_theta: float
    value_scale: float = 1.0
    sliding_window: Optional[int] = None
    sink_bias: bool = False

    def local_heads(self, tp: int) -> int:
        if self.head_count % tp:
            raise ValueError(f"{self.head_count} query heads do not split over tp={tp}")
        return self.head_count // tp

    def local_kv_heads(self, tp: int) -> int:
        """KV heads a rank stores: whole heads when tp <= kv heads, else one shared head."""
        return max(1, self.kv_head_count // tp)

    def kv_head_for_rank(self, rank: int, tp: int) -> Tuple[int, ...]:
        """Global KV head ids cached by ``rank`` (ranks share a head when tp > kv heads)."""
        n = self.local_kv_heads(tp)
        if tp <= self.kv_head_count:
            return tuple(range(rank * n, rank * n + n))
        share = tp // self.kv_head_count
        return (rank // share,)

    @property
    def softmax_scale(self) -> float:
        return float(self.head_dim) ** -0.5


@dataclass(frozen=True)
class SparseIndexerSpec:
    """Lightning indexer: fp8 relu-weighted scoring that picks ``top_k`` cached keys."""

    head_count: int
    head_dim: int
    rope_dim: int
    top_k: int

    @property
    def weight_scale(self) -> float:
        return float(self.head_count) ** -0.5


@dataclass(frozen=True)
class MoeRoutingSpec:
    score_func: str = "sigmoid"       # "sigmoid" (with correction bias) or "softmax"
    expert_count: int = 256
    top_k: int = 8
    intermediate: int = 2048
    shared_expert_count: int = 0
    route_scale: float = 1.0
    normalize_top_k: bool = True
    group_count: int = 1
    limited_group_count: int = 1


@dataclass(frozen=True)
class DraftSpec:
    """Block-draft ("DSpark") geometry.  Reference: naivert/models/naive_n0p5/dspark.py:20-51."""

    layer_count: int = 5
    hidden: int = 4096
    head_count: int = 32
    kv_head_count: int = 4
    head_dim: int = 128
    intermediate: int = 4096
    markov_rank: int = 256
    block_size: int = 7           # proposals per round; +1 anchor row = 8 rows
    window: int = 1024
    rope_theta: float = 1.0e4
    mask_token_id: int = 151675
    target_layer_ids: Tuple[int, ...] = (1, 7, 14, 20, 26, 32, 39, 45)
    norm_eps: float = 1e-5

    @property
    def rows(self) -> int:
        return self.block_size + 1


@dataclass(frozen=True)
class ModelSpec:
    """Whole-model geometry.  ``weight_dtype`` selects the numerical recipe:

    * ``"fp8"``  - W8A8: 128x128 block-scaled e4m3 weights, e4m3 activations with one
      power-of-two scale per 128-wide K block, bf16 residual stream.
    * ``"fp32"`` - no rounding points at all (CPU reference configuration).
    """

    name: str
    hidden: int
    vocab: int
    layer_kinds: Tuple[str, ...]
    attention: Mapping[str, AttentionLayout]
    indexer: SparseIndexerSpec
    routing: MoeRoutingSpec
    dense_layer_count: int = 1
    dense_intermediate: int = 16384
    norm_eps: float = 1e-5
    weight_dtype: str = "fp8"
    stop_token_ids: Tuple[int, ...] = (151645,)
    think_end_token_id: int = 151668
    draft: Optional[DraftSpec] = None
    precision_id: str = "n0p5-w8a8-fp32-expert-completion-v1"

    @property
    def layer_count(self) -> int:
        return len(self.layer_kinds)

    def layout(self, layer: int) -> AttentionLayout:
        return self.attention[self.layer_kinds[layer]]

    def is_dense(self, layer: int) -> bool:
        return layer < self.dense_layer_count

    def dsa_layers(self) -> Tuple[int, ...]:
        return tuple(i for i, k in enumerate(self.layer_kinds) if k == FULL_DSA)

    def vocab_shard(self, tp: int) -> int:
        if self.vocab % tp:
            raise ValueError(f"vocab {self.vocab} does not split over tp={tp}")
        return self.vocab // tp

    def expert_inter_local(self, tp: int) -> int:
        if self.routing.intermediate % tp:
            raise ValueError("expert intermediate does not split over tp")
        return self.routing.intermediate // tp

    def dense_inter_local(self, tp: int) -> int:
        return self.dense_intermediate // tp

    def with_layers(self, n: int) -> "ModelSpec":
        """Same geometry truncated to the first ``n`` layers (used when weights do not fit)."""
        if not 1 <= n <= self.layer_count:
            raise ValueError(f"layer count {n} outside 1..{self.layer_count}")
        draft = self.draft
        if draft is not None:
            ids = tuple(i for i in draft.target_layer_ids if i < n)
            if len(ids) < len(draft.target_layer_ids):
                # spread the taps over the surviving layers (fewer taps when fewer layers remain)
                k = min(len(draft.target_layer_ids), n)
                ids = tuple((j * n) // k for j in range(k))
            draft = replace(draft, target_layer_ids=ids)
        return replace(self, name=f"{self.name}-L{n}", layer_kinds=self.layer_kinds[:n], draft=draft)

    def kv_bytes_per_token(self, tp: int) -> int:
        """Bytes of full-length (DSA) cache per token per rank, incl. the draft KV."""
        total = 0
        for layer, kind in enumerate(self.layer_kinds):
            if kind != FULL_DSA:
                continue
            a = self.attention[kind]
            total += a.local_kv_heads(tp) * (a.head_dim + a.v_head_dim) * 2
            total += self.indexer.head_dim + 4
        if self.draft is not None:
            d = self.draft
            total += d.layer_count * max(1, d.kv_head_count // tp) * d.head_dim * 2 * 2
        return total


@dataclass(frozen=True)
class SamplingParams:
    """Per-request sampling controls; defaults follow the reference HTTP surface
    (docs/messages_http.md:64-72): T=1, top-p 0.95, seed 1234, penalties 1/0/0."""

    temperature: float = 1.0
    top_p: float = 0.95
    seed: int = 1234
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    forced_accept_p: Optional[float] = None   # Bernoulli(p) per-position forced acceptance mask

    TOP_P_MAX = 1.0 - 2.0 ** -20

    def clamped_top_p(self) -> float:
        return min(self.top_p, self.TOP_P_MAX)

    def validate(self) -> None:
        if not (0.0 < self.temperature <= 5.0):
            raise ValueError("temperature must be in (0, 5]")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if not (0 <= self.seed < 2 ** 63):
            raise ValueError("seed must be in [0, 2^63)")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be > 0")
