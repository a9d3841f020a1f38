"""Naive-N0.5-Flash geometry (target + block draft) and reduced test geometries.

Parity: naivert/models/naive_n0p5/model.py:17-93 (hybrid pattern, attention layouts,
indexer, routing, sizes) and naivert/models/naive_n0p5/dspark.py:20-51 (draft).
"""
from __future__ import annotations

from .spec import (FULL_DSA, SLIDING_WINDOW, AttentionLayout, DraftSpec, ModelSpec,
                   MoeRoutingSpec, SparseIndexerSpec)

# full attention (+ DSA indexer) every sixth layer starting at 0 (with layer 5 the first repeat)
_FULL_LAYERS = (0, 5, 11, 17, 23, 29, 35, 41, 47)
LAYER_KINDS = tuple(FULL_DSA if i in _FULL_LAYERS else SLIDING_WINDOW for i in range(48))

NAIVE_N0P5 = ModelSpec(
    name="naive-n0.5",
    hidden=4096,
    vocab=152576,
    layer_kinds=LAYER_KINDS,
    attention={
        FULL_DSA: AttentionLayout(kind=FULL_DSA, head_count=64, kv_head_count=4, head_dim=192,
                                  v_head_dim=128, rope_dim=64, rope_theta=1.0e7, value_scale=0.707),
        SLIDING_WINDOW: AttentionLayout(kind=SLIDING_WINDOW, head_count=64, kv_head_count=8,
                                        head_dim=192, v_head_dim=128, rope_dim=64, rope_theta=1.0e4,
                                        value_scale=0.707, sliding_window=128, sink_bias=True),
    },
    indexer=SparseIndexerSpec(head_count=16, head_dim=128, rope_dim=64, top_k=2048),
    routing=MoeRoutingSpec(score_func="sigmoid", expert_count=256, top_k=8, intermediate=2048,
                           shared_expert_count=0, route_scale=1.0, normalize_top_k=True),
    dense_layer_count=1,
    dense_intermediate=16384,
    norm_eps=1e-5,
    weight_dtype="fp8",
    stop_token_ids=(151645,),
    think_end_token_id=151668,
    draft=DraftSpec(),
)


def tiny_spec(weight_dtype: str = "fp32") -> ModelSpec:
    """The CPU-reference geometry: 2 layers, hidden 256, 4 heads of 64, lightning indexer
    with 4 heads of 32 picking top-64, 8 routed experts top-2 plus one shared expert
    (FFN 128), softmax router, vocab 1024."""
    return ModelSpec(
        name=f"tiny-{weight_dtype}",
        hidden=256,
        vocab=1024,
        layer_kinds=(FULL_DSA, SLIDING_WINDOW),
        attention={
            FULL_DSA: AttentionLayout(kind=FULL_DSA, head_count=4, kv_head_count=2, head_dim=64,
                                      v_head_dim=64, rope_dim=32, rope_theta=1.0e4, value_scale=0.707),
            SLIDING_WINDOW: AttentionLayout(kind=SLIDING_WINDOW, head_count=4, kv_head_count=2,
                                            head_dim=64, v_head_dim=64, rope_dim=32, rope_theta=1.0e4,
                                            value_scale=0.707, sliding_window=128, sink_bias=True),
        },
        indexer=SparseIndexerSpec(head_count=4, head_dim=32, rope_dim=16, top_k=64),
        routing=MoeRoutingSpec(score_func="softmax", expert_count=8, top_k=2, intermediate=128,
                               shared_expert_count=1, route_scale=1.0, normalize_top_k=True),
        dense_layer_count=0,
        dense_intermediate=512,
        norm_eps=1e-5,
        weight_dtype=weight_dtype,
        stop_token_ids=(1023,),
        think_end_token_id=1022,
        draft=DraftSpec(layer_count=2, hidden=256, head_count=4, kv_head_count=2, head_dim=64,
                        intermediate=256, markov_rank=32, block_size=7, window=64,
                        mask_token_id=1021, target_layer_ids=(0, 1)),
    )


def small_w8a8_spec(layers: int = 4) -> ModelSpec:
    """A W8A8 geometry with every tile dimension a multiple of 128 but tiny weights:
    used by GPU kernel tests and the smoke run (same kernels as the full model)."""
    kinds = tuple(FULL_DSA if i % 3 == 0 else SLIDING_WINDOW for i in range(layers))
    return ModelSpec(
        name=f"small-w8a8-L{layers}",
        hidden=1024,
        vocab=8192,
        layer_kinds=kinds,
        attention={
            FULL_DSA: AttentionLayout(kind=FULL_DSA, head_count=8, kv_head_count=4, head_dim=192,
                                      v_head_dim=128, rope_dim=64, rope_theta=1.0e7, value_scale=0.707),
            SLIDING_WINDOW: AttentionLayout(kind=SLIDING_WINDOW, head_count=8, kv_head_count=8,
                                            head_dim=192, v_head_dim=128, rope_dim=64, rope_theta=1.0e4,
                                            value_scale=0.707, sliding_window=128, sink_bias=True),
        },
        indexer=SparseIndexerSpec(head_count=16, head_dim=128, rope_dim=64, top_k=256),
        routing=MoeRoutingSpec(score_func="sigmoid", expert_count=32, top_k=8, intermediate=1024,
                               shared_expert_count=0, route_scale=1.0, normalize_top_k=True),
        dense_layer_count=1,
        dense_intermediate=2048,
        norm_eps=1e-5,
        weight_dtype="fp8",
        stop_token_ids=(8191,),
        think_end_token_id=8190,
        draft=DraftSpec(layer_count=2, hidden=1024, head_count=8, kv_head_count=4, head_dim=128,
                        intermediate=1024, markov_rank=128, block_size=7, window=1024,
                        mask_token_id=8189, target_layer_ids=tuple(range(layers))),
    )
