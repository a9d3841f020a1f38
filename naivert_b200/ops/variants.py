"""Kernel variant records: which entry points of the native library a runtime needs, and their argument ABI.

Every launcher of ``libnaivert_b200.so`` is named here once: its variant id (``<op>.<form>.sm100a.abi<N>``), the
``extern "C"`` symbol, the argument struct it reads (mirrored in ``ops/kernels.py``) and the symbol that reports the
struct's size as compiled.  ``library_variant`` reads the actual record back from the loaded library;
``require_variant`` fails closed unless the two are the same record, so a runtime built against one ABI never drives a
library built from other sources.  ``STEP_VARIANTS`` / ``PREFILL_VARIANTS`` are what the decode round and the native
prefill ask for before they capture anything.

``abi<N>`` is the revision of the argument struct's layout: bump it in the table when a field is added, moved or
re-typed (the struct-size check catches most of these by itself; the revision also covers same-size edits).

Reference counterpart: naivert/kernel_variant.py (``KernelVariantSpec``, ``require_kernel_variant``) and
naivert/models/naive_n0p5/kernel_specs.py (the accepted variants of the model).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, replace
from typing import Dict, Iterable, List, Optional

ARCH = "sm100a"


@dataclass(frozen=True)
class KernelVariant:
    variant_id: str
    entry: str                              # extern "C" launcher
    args_struct: Optional[str] = None       # ctypes class in ops.kernels (None: scalar arguments only)
    size_symbol: Optional[str] = None       # extern "C" int f(): sizeof the struct as compiled
    abi_version: int = 1
    args_bytes: Optional[int] = None        # filled from the ctypes mirror (expected) or the library (actual)
    max_rows: Optional[int] = None          # widest token batch the launcher accepts (None: unbounded)

    def __post_init__(self) -> None:
        vid = str(self.variant_id).strip()
        if not vid or not vid.endswith(f".{ARCH}.abi{self.abi_version}"):
            raise ValueError(f"variant id {self.variant_id!r} must end in .{ARCH}.abi{self.abi_version}")
        if self.abi_version <= 0:
            raise ValueError("ABI revision must be positive")
        if (self.args_struct is None) != (self.size_symbol is None):
            raise ValueError(f"{vid}: argument struct and size symbol come together")
        if self.args_bytes is not None and self.args_bytes <= 0:
            raise ValueError(f"{vid}: argument bytes must be positive")


def _v(op: str, entry: str, struct: Optional[str] = None, size: Optional[str] = None, abi: int = 1,
       max_rows: Optional[int] = None) -> KernelVariant:
    return KernelVariant(f"{op}.{ARCH}.abi{abi}", entry, struct, size, abi, None, max_rows)


_TABLE: List[KernelVariant] = [
    _v("skinny_gemm.fused_epilogues", "nrt_gemm_launch", "GemmArgs", "nrt_gemm_args_size", abi=4, max_rows=16),
    _v("chunk_gemm.persistent", "nrt_wide_gemm_launch", "GemmArgs", "nrt_gemm_args_size", abi=4),
    _v("attn_post.rope_kv_append", "nrt_attn_post", "AttnPostArgs", "nrt_attn_post_args_size", abi=2),
    _v("attn_decode.tensor_core", "nrt_attn_decode", "AttnArgs", "nrt_attn_decode_args_size", abi=3),
    _v("attn_rows.scalar", "nrt_attn_rows", "AttnArgs", "nrt_attn_args_size", abi=3),
    _v("attn_group.chunk", "nrt_attn_group", "AttnArgs", "nrt_attn_group_args_size", abi=3),
    _v("index_sweep.tcgen05", "nrt_index_sweep", "SweepArgs", "nrt_sweep_args_size"),
    _v("index_logits.simple", "nrt_index_logits_simple", "IndexArgs", "nrt_index_args_size"),
    _v("topk_rows.radix", "nrt_topk_rows", "IndexArgs", "nrt_index_args_size"),
    _v("topk_rows.grid", "nrt_topk_rows_grid", "IndexArgs", "nrt_index_args_size"),
    _v("router.select", "nrt_router", "RouterArgs", "nrt_router_args_size", abi=2),
    _v("moe_layer.fused", "nrt_moe_layer", "MoeArgs", "nrt_moe_args_size", abi=3, max_rows=8),
    _v("step_prologue.embed_norm", "nrt_step_prologue", "PrologueArgs", "nrt_prologue_args_size", max_rows=16),
    _v("argmax_rows.exchange", "nrt_argmax_rows", "ArgmaxArgs", "nrt_argmax_args_size"),
    _v("sampler.staged", "nrt_sampler_run", "SamplerArgs", "nrt_sampler_args_size", abi=2),
    _v("sampler.persistent", "nrt_sampler_persistent", "SamplerArgs", "nrt_sampler_args_size", abi=2),
    _v("tail_commit.ring", "nrt_tail_commit", "TailArgs", "nrt_tail_args_size", abi=2),
    _v("markov.step", "nrt_markov_step", "MarkovArgs", "nrt_markov_args_size"),
    _v("markov.chain", "nrt_markov_chain", "MarkovArgs", "nrt_markov_args_size"),
    _v("ag_push.peer_store", "nrt_ag_push", "AgPushArgs", "nrt_ag_push_args_size"),
    _v("ep.count", "nrt_ep_count", "EpArgs", "nrt_ep_args_size"),
    _v("ep.dispatch", "nrt_ep_dispatch", "EpArgs", "nrt_ep_args_size"),
    _v("ep.combine", "nrt_ep_combine", "EpCombineArgs", "nrt_ep_combine_args_size"),
    _v("graph.relaunch", "nrt_relaunch"),
    _v("draft.block_input", "nrt_draft_block_input"),
    _v("router.route_noalloc", "nrt_router_route_noalloc", max_rows=16),
]


def _expected(v: KernelVariant) -> KernelVariant:
    if v.args_struct is None:
        return v
    from . import kernels as K
    return replace(v, args_bytes=C.sizeof(getattr(K, v.args_struct)))


def variants() -> Dict[str, KernelVariant]:
    """Variant id -> the record this package was written against (argument bytes from the ctypes mirrors)."""
    return {v.variant_id: _expected(v) for v in _TABLE}


def by_entry(entry: str) -> KernelVariant:
    for v in _TABLE:
        if v.entry == entry:
            return _expected(v)
    raise KeyError(entry)


# what the speculative round and the native prefill launch
STEP_VARIANTS = ("nrt_gemm_launch", "nrt_attn_decode", "nrt_index_sweep", "nrt_topk_rows", "nrt_moe_layer", "nrt_router",
                 "nrt_step_prologue", "nrt_sampler_persistent", "nrt_sampler_run", "nrt_tail_commit", "nrt_markov_chain",
                 "nrt_markov_step", "nrt_draft_block_input", "nrt_argmax_rows")
PREFILL_VARIANTS = ("nrt_wide_gemm_launch", "nrt_attn_post", "nrt_attn_group", "nrt_index_sweep", "nrt_topk_rows_grid",
                    "nrt_router", "nrt_ep_count", "nrt_ep_dispatch", "nrt_ep_combine", "nrt_ag_push")


def library_variant(lib, expected: KernelVariant) -> KernelVariant:
    """The record the loaded library actually provides for ``expected``'s entry point.  A missing launcher or size symbol
    raises; the argument bytes are what the library's compiler laid out."""
    if not hasattr(lib, expected.entry):
        raise ValueError(f"kernel variant {expected.variant_id!r}: the library exports no {expected.entry}")
    actual_bytes = None
    if expected.size_symbol is not None:
        if not hasattr(lib, expected.size_symbol):
            raise ValueError(f"kernel variant {expected.variant_id!r}: the library exports no {expected.size_symbol}")
        actual_bytes = int(getattr(lib, expected.size_symbol)())        # ctypes' default result type is int
    return replace(expected, args_bytes=actual_bytes)


def require_variant(expected: KernelVariant, actual: KernelVariant) -> KernelVariant:
    """Fail closed unless the caller's record and the library's record are the same."""
    if not isinstance(expected, KernelVariant) or expected != actual:
        got = getattr(actual, "args_bytes", None)
        raise ValueError(f"kernel variant {getattr(expected, 'variant_id', expected)!r} differs from the library's "
                         f"(argument bytes {getattr(expected, 'args_bytes', None)} expected, {got} built)")
    return actual


def require_entries(lib, entries: Iterable[str]) -> List[KernelVariant]:
    """``require_variant`` for every launcher a runtime is about to use."""
    out = []
    for e in entries:
        exp = by_entry(e)
        out.append(require_variant(exp, library_variant(lib, exp)))
    return out


def check_library(lib=None) -> List[str]:
    """Problems of the whole table against the loaded library (empty: every variant is present with the expected ABI)."""
    if lib is None:
        from . import kernels as K
        lib = K.lib()
    problems = []
    for v in variants().values():
        try:
            require_variant(v, library_variant(lib, v))
        except ValueError as e:
            problems.append(str(e))
    return problems
