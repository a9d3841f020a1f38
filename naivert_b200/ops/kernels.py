"""ctypes bindings of the sm_100a kernel library.

Every wrapper takes torch CUDA tensors (already allocated: nothing here allocates on the
launch path, so the calls are graph-capturable) and launches on the current stream.  The
argument structures mirror the C structs field by field; their sizes are checked against the
library at import so a layout drift fails loudly instead of corrupting a launch.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from .build import load_library

VP, I32, F32, U64 = C.c_void_p, C.c_int, C.c_float, C.c_ulonglong

K_TOK = 16
K_MAX_PEERS = 8
K_ROW_PAIRS = 8
K_MAILBOX_SLABS = 4

# GEMM variants: fp8 | dual<<1 | epi<<2 | group<<5 | bsrc<<7
EPI_STORE_F32, EPI_STORE_BF16, EPI_SILU_QUANT, EPI_ALLREDUCE, EPI_SILU_BF16, EPI_RETURN, EPI_QKV_POST = 0, 1, 2, 3, 4, 5, 6
B_TMA, B_NORM = 0, 1
GROUP_NONE, GROUP_ITEM, GROUP_LOOP = 0, 1, 2


def gemm_variant(fp8: bool, dual: bool, epi: int, group: int, bsrc: int = 0) -> int:
    return int(fp8) | (int(dual) << 1) | (epi << 2) | (group << 5) | (bsrc << 7)


class FabricArgs(C.Structure):
    _fields_ = [("mailbox", VP * K_MAX_PEERS), ("epoch", VP), ("status", VP), ("tp", I32), ("rank", I32),
                ("call_idx", I32), ("features", I32), ("timeout_ns", U64), ("mode", I32), ("ag_call", I32),
                ("ag_flags", VP)]


class AttnPostArgs(C.Structure):
    _fields_ = [("qkv", VP), ("ld", I32), ("rows", I32), ("pos0", VP),
                ("heads", I32), ("kv_heads", I32), ("head_dim", I32), ("v_dim", I32), ("rope_dim", I32),
                ("value_scale", F32), ("rope", VP), ("q_out", VP), ("k_cache", VP), ("v_cache", VP), ("ring", I32),
                ("q_norm", VP), ("k_norm", VP), ("norm_eps", F32),
                ("idx_heads", I32), ("idx_dim", I32), ("idx_rope", I32), ("idx_rope_tab", VP),
                ("ik_w", VP), ("ik_b", VP), ("ln_eps", F32), ("idx_weight_scale", F32),
                ("iq8", VP), ("ihw", VP), ("ik_cache", VP), ("ik_scale", VP),
                ("col_q", I32), ("col_k", I32), ("col_v", I32), ("col_iq", I32), ("col_ik", I32), ("col_iw", I32),
                ("iq_scale", VP), ("group_cols", I32), ("norm_group_stride", I32), ("k_group_stride", C.c_longlong),
                ("v_group_stride", C.c_longlong)]


class GemmArgs(C.Structure):
    _fields_ = [("n_total", I32), ("k_total", I32), ("rows", I32), ("a_group", I32),
                ("n_active", VP), ("active_ids", VP), ("probs", VP), ("max_slots", I32), ("n_experts", I32),
                ("w_scale0", VP), ("w_scale1", VP), ("a_scale", VP),
                ("out_f32", VP), ("out_bf16", VP), ("ld_out", I32), ("out_scale", F32),
                ("out_q", VP), ("out_qscale", VP), ("resid", VP), ("out_copy", VP), ("ld_copy", I32),
                ("fab", FabricArgs), ("status", VP),
                ("row_offsets", VP), ("ep_meta", VP), ("ep_combine", VP * K_MAX_PEERS), ("ep_top_k", I32),
                ("ep_dispatch_call", I32), ("ep_return_call", I32),
                ("nx", VP), ("ngamma", VP), ("nssq", VP), ("neps", F32), ("ssq_out", VP), ("post", AttnPostArgs),
                ("stamps", VP), ("publish_delay_ns", C.c_uint), ("pf_ptr", VP), ("pf_bytes", U64)]


class AttnArgs(C.Structure):
    _fields_ = [("q", VP), ("k_cache", VP), ("v_cache", VP), ("pos0", VP),
                ("rows", I32), ("heads", I32), ("kv_heads", I32), ("head_dim", I32), ("v_dim", I32),
                ("scale", F32), ("mode", I32), ("window", I32), ("ring", I32), ("sink", VP), ("sel", VP),
                ("top_k", I32), ("k_blk", VP), ("v_blk", VP), ("o_bf16", VP), ("o8", VP), ("o_scale", VP),
                ("part", VP), ("tickets", VP), ("stamps", VP)]


class IndexArgs(C.Structure):
    _fields_ = [("iq8", VP), ("ihw", VP), ("ik", VP), ("iks", VP), ("pos0", VP),
                ("rows", I32), ("heads", I32), ("dim", I32), ("top_k", I32), ("logits", VP), ("ld", I32), ("iq_scale", VP)]


class RouterArgs(C.Structure):
    _fields_ = [("xn", VP), ("x", VP), ("gamma", VP), ("eps", F32), ("ssq", VP), ("xs", VP),
                ("w", VP), ("bias", VP), ("hidden", I32), ("experts", I32), ("rows", I32),
                ("top_k", I32), ("sigmoid", I32), ("normalize", I32), ("route_scale", F32),
                ("scores", VP), ("ticket", VP), ("n_active", VP), ("active_ids", VP), ("probs", VP),
                ("topk_ids", VP), ("topk_p", VP), ("max_slots", I32), ("x8", VP), ("stamps", VP)]


class MoeArgs(C.Structure):
    _fields_ = [("r", RouterArgs), ("inter", I32), ("gate_s", VP), ("up_s", VP), ("down_s", VP), ("y8", VP), ("ys", VP),
                ("sync", VP), ("slot_flags", VP), ("part", VP), ("part_flags", VP), ("ar", GemmArgs)]


_lib = None

BOUNDS_SITES = {1: "attention key id beyond the query position", 2: "expert id", 3: "token id", 4: "Markov previous-token id"}


def bounds_violations() -> list:
    """(translation unit, site description, offending index) of the first out-of-range index each translation unit of
    the checking flavour recorded since the last call (the words are cleared).  The regular library reports none."""
    from .build import BOUNDS_UNITS
    L = lib()
    out = []
    for unit in BOUNDS_UNITS:
        f = getattr(L, "nrt_bounds_" + unit)
        f.restype = C.c_ulonglong
        v = int(f())
        if v == (1 << 64) - 1:
            raise RuntimeError(f"the bounds word of {unit} could not be read")
        if v:
            out.append((unit, BOUNDS_SITES.get((v >> 32) & 0x7FFFFFFF, "unknown site"), int(C.c_int32(v & 0xFFFFFFFF).value)))
    return out


def lib():
    global _lib
    if _lib is None:
        _lib = load_library()
        _lib.nrt_attn_decode_part_floats.restype = C.c_longlong
        for name, st in (("nrt_gemm_args_size", GemmArgs), ("nrt_attn_post_args_size", AttnPostArgs),
                         ("nrt_attn_args_size", AttnArgs), ("nrt_index_args_size", IndexArgs),
                         ("nrt_router_args_size", RouterArgs)):
            got = getattr(_lib, name)()
            if got != C.sizeof(st):
                raise RuntimeError(f"{st.__name__}: library has {got} bytes, bindings {C.sizeof(st)}")
    return _lib


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


LAUNCHES = {"count": 0}          # kernels launched through this module (sampler chain counts as 9)


def check(code: int, what: str) -> None:
    LAUNCHES["count"] += 9 if what == "sampler" else 1
    if code != 0:
        raise RuntimeError(f"{what} failed with CUDA/driver error {code}")


# ----------------------------------------------------------------------------- tensor maps
class TensorMap:
    """A 128-byte CUtensorMap kept alive with the tensor it describes."""

    def __init__(self, t: torch.Tensor, dims: Sequence[int], strides_bytes: Sequence[int], box: Sequence[int],
                 dtype_code: int, swizzle: int = 3):
        self.tensor = t
        self.buf = (C.c_ubyte * 128)()
        rank = len(dims)
        d = (C.c_uint64 * 5)(*dims)
        s = (C.c_uint64 * 5)(*strides_bytes)
        b = (C.c_uint32 * 5)(*box)
        check(lib().nrt_tmap_encode(C.byref(self.buf), dtype_code, rank, d, s, b, swizzle, VP(t.data_ptr())),
              "cuTensorMapEncodeTiled")


def weight_tmap(w: torch.Tensor) -> TensorMap:
    """[N, K] or [E, N, K] weights (e4m3 bytes or bf16) -> 3-D map with 128-row x 128-byte boxes."""
    if w.dim() == 2:
        w = w.unsqueeze(0)
    assert w.is_contiguous()
    e, n, k = w.shape
    es = w.element_size()
    code = 0 if es == 1 else 1
    return TensorMap(w, (k, n, e), (k * es, n * k * es), (128 // es, 128, 1), code)


def act_tmap(x: torch.Tensor, box_rows: int = K_TOK) -> TensorMap:
    """[rows (multiple of ``box_rows``), K] activations -> 2-D map with ``box_rows`` x 128-byte boxes
    (16 rows for the step engine, 64 for the chunk GEMM)."""
    assert x.dim() == 2 and x.stride(1) == 1 and x.shape[0] % box_rows == 0
    r, k = x.shape
    es = x.element_size()
    assert (x.stride(0) * es) % 16 == 0 and x.data_ptr() % 16 == 0
    return TensorMap(x, (k, r), (x.stride(0) * es,), (128 // es, box_rows), 0 if es == 1 else 1)


_SPLIT_MIN_KB = int(__import__("os").environ.get("NAIVERT_SPLIT_MIN_KB", "1"))


def pick_split(n_tiles: int, k_blocks: int, max_ctas: int = 160, max_split: int = 4) -> int:
    """CTAs per output tile (one cluster): the largest of (8,) 4, 2, 1 that divides the K blocks, leaves
    every CTA at least ``NAIVERT_SPLIT_MIN_KB`` K blocks and keeps the grid within about one wave of
    the 148 SMs."""
    for s in (8, 4, 2):
        if s > max_split:
            continue
        if k_blocks % s == 0 and n_tiles * s <= max_ctas and k_blocks // s >= _SPLIT_MIN_KB:
            return s
    return 1


def norm_split(n_tiles: int, k_total: int, fp8: bool, dual: bool, max_split: int = 8) -> int:
    """``pick_split`` for the projections that build their normalised token operand in shared memory: the CTA's whole
    K slice of the operand sits beside the weight ring, so a small grid may not keep K unsplit.  The split is raised
    (even past one wave of CTAs) until ring + operand + epilogue staging + split partials fit the 227 KiB of an SM."""
    kb_total = k_total // (128 if fp8 else 64)
    tile_a = 128 * 128                                    # bytes of one weight stage per matrix (128 rows x 128 B)
    ring = (4 if dual else 8) * (2 if dual else 1) * tile_a
    def fits(split: int) -> bool:
        kb = kb_total // split
        operand = kb * 2048 + (((kb * 16 * 4 + 1023) // 1024) * 1024 if fp8 else 0)
        part = (2 if dual else 1) * (split - 1) * 8 * 128 * 4 if split > 1 else 0
        return ring + operand + 1024 + 1024 + 16 * 128 * 4 + part <= 227 * 1024
    s = pick_split(n_tiles, kb_total, max_split=max_split)
    while not fits(s) and s < 8 and kb_total % (2 * s) == 0:
        s *= 2
    return s


# ----------------------------------------------------------------------------- launches
def gemm(variant: int, a0: TensorMap, a1: Optional[TensorMap], b: Optional[TensorMap], args: GemmArgs, grid_x: int,
         grid_y: int = 1, pdl: bool = True) -> None:
    check(lib().nrt_gemm_launch(variant, C.byref(a0.buf), C.byref(a1.buf) if a1 is not None else None,
                                C.byref(b.buf) if b is not None else None, C.byref(args), grid_x, grid_y, VP(_stream()),
                                int(pdl)), "gemm launch")


WIDE_TOK = 64


def wide_gemm(variant: int, a0: TensorMap, a1: Optional[TensorMap], b: TensorMap, args: GemmArgs, n_tiles: int,
              items: int, pdl: bool = False, items_fastest: bool = False) -> None:
    """Chunk GEMM (64 token rows per item, item mode only); ``b`` must be a 64-row-box token map.
    ``items_fastest``: consecutive CTAs share a weight tile (one large weight matrix) instead of a token tile."""
    check(lib().nrt_wide_gemm_launch(variant, C.byref(a0.buf), C.byref(a1.buf) if a1 is not None else None,
                                     C.byref(b.buf), C.byref(args), n_tiles, items, int(items_fastest), VP(_stream()),
                                     int(pdl)), "wide gemm launch")


def embed_rows(tokens, table, x, rows, pdl=True):
    check(lib().nrt_embed_rows(VP(ptr(tokens)), VP(ptr(table)), VP(ptr(x)), table.shape[1], rows, table.shape[0],
                               VP(_stream()), int(pdl)), "embed_rows")


class PrologueArgs(C.Structure):
    _fields_ = [("tokens", VP), ("table", VP), ("mask", VP), ("x", VP), ("ssq", VP),
                ("hidden", I32), ("rows", I32), ("vocab", I32), ("mode", I32), ("n_tabs", I32),
                ("tab_pos0", VP * 4), ("tab_dim", I32 * 4), ("tab_theta", C.c_double * 4), ("tab_out", VP * 4)]


def step_prologue(args: PrologueArgs, pdl=True):
    """Input rows (embedding gather or draft block), their per-tile sums of squares, and the step's RoPE tables."""
    L = lib()
    if L.nrt_prologue_args_size() != C.sizeof(PrologueArgs):
        raise RuntimeError("PrologueArgs layout drift")
    check(L.nrt_step_prologue(C.byref(args), VP(_stream()), int(pdl)), "step_prologue")


def rope_table(pos0, rows, dim, theta, out, pdl=True):
    check(lib().nrt_rope_table(VP(ptr(pos0)), rows, dim, C.c_double(theta), VP(ptr(out)), VP(_stream()), int(pdl)),
          "rope_table")


def prep_norm(x, gamma, rows, eps, xn=None, x8=None, xs=None, pdl=True):
    check(lib().nrt_prep_norm(VP(ptr(x)), VP(ptr(gamma)), x.shape[1], rows, C.c_float(eps), VP(ptr(xn)), VP(ptr(x8)),
                              VP(ptr(xs)), VP(_stream()), int(pdl)), "prep_norm")


def attn_post(args: AttnPostArgs, pdl=True):
    check(lib().nrt_attn_post(C.byref(args), VP(_stream()), int(pdl)), "attn_post")


def attn_rows(args: AttnArgs, splits: int = 1, pdl=True):
    check(lib().nrt_attn_rows(C.byref(args), splits, VP(_stream()), int(pdl)), "attn_rows")


def attn_decode_ok(args: AttnArgs) -> bool:
    """Geometry served by the tensor-core decode attention (else use ``attn_rows``)."""
    return (args.v_dim == 128 and args.head_dim in (128, 192) and args.kv_heads >= 1 and args.heads % args.kv_heads == 0
            and args.heads // args.kv_heads <= 16)


def attn_decode_part_floats(rows: int, kv_heads: int, splits: int) -> int:
    return int(lib().nrt_attn_decode_part_floats(rows, kv_heads, splits))


def attn_decode(args: AttnArgs, splits: int = 1, pdl=True):
    """Row attention of the step on tensor cores: the query heads of a KV head share every gathered key."""
    L = lib()
    if L.nrt_attn_decode_args_size() != C.sizeof(AttnArgs):
        raise RuntimeError("AttnArgs layout drift")
    check(L.nrt_attn_decode(C.byref(args), splits, VP(_stream()), int(pdl)), "attn_decode")


def attn_group(args: AttnArgs, pdl=True):
    """Row attention with the query heads of each KV head handled by one CTA (prefill chunks)."""
    L = lib()
    if L.nrt_attn_group_args_size() != C.sizeof(AttnArgs):
        raise RuntimeError("AttnArgs layout drift")
    check(L.nrt_attn_group(C.byref(args), VP(_stream()), int(pdl)), "attn_group")


class SweepArgs(C.Structure):
    _fields_ = [("ihw", VP), ("iks", VP), ("pos0", VP), ("rows", I32), ("heads", I32), ("top_k", I32),
                ("logits", VP), ("ld", I32), ("status", VP), ("group0", I32), ("ngroups", I32), ("iq_scale", VP)]


def sweep_maps(ik_cache: torch.Tensor, iq8: torch.Tensor):
    """Tensor maps of the tcgen05 indexer sweep: key cache [cap, 128] e4m3 bytes, queries [256, 128]."""
    assert ik_cache.shape[1] == 128 and iq8.shape[1] == 128 and iq8.shape[0] % 256 == 0
    km = TensorMap(ik_cache, (128, ik_cache.shape[0]), (128,), (128, 128), 0)
    qm = TensorMap(iq8, (128, iq8.shape[0]), (128,), (128, 256), 0)
    return km, qm


def index_sweep(km: TensorMap, qm: TensorMap, args: SweepArgs, blocks: int, pdl=True):
    L = lib()
    if L.nrt_sweep_args_size() != C.sizeof(SweepArgs):
        raise RuntimeError("SweepArgs layout drift")
    check(L.nrt_index_sweep(C.byref(km.buf), C.byref(qm.buf), C.byref(args), blocks, VP(_stream()), int(pdl)), "index_sweep")


def index_logits_simple(args: IndexArgs, blocks: int, pdl=True):
    check(lib().nrt_index_logits_simple(C.byref(args), blocks, VP(_stream()), int(pdl)), "index_logits")


def topk_rows(logits, pos0, rows, top_k, sel, pdl=True):
    check(lib().nrt_topk_rows(VP(ptr(logits)), logits.shape[1], VP(ptr(pos0)), rows, top_k, VP(ptr(sel)),
                              VP(_stream()), int(pdl)), "topk_rows")


def moe_layer(gate: TensorMap, up: TensorMap, down: TensorMap, x8: TensorMap, y8: TensorMap, args: "MoeArgs", pdl=True) -> int:
    """Router + grouped gate/up + grouped down + all-reduce of one MoE block in a single launch.  Returns the
    library's code without raising for -3 / -9 (geometry or occupancy does not fit: use the separate kernels)."""
    L = lib()
    if L.nrt_moe_args_size() != C.sizeof(MoeArgs):
        raise RuntimeError("MoeArgs layout drift")
    code = L.nrt_moe_layer(C.byref(gate.buf), C.byref(up.buf), C.byref(down.buf), C.byref(x8.buf), C.byref(y8.buf),
                           C.byref(args), VP(_stream()), int(pdl))
    if code in (-3, -9):
        return code
    check(code, "moe_layer")
    return 0


def moe_scratch_sizes(hidden: int):
    """(slot flag words, partial floats) of the fused MoE kernel's hand-off buffers."""
    L = lib()
    L.nrt_moe_part_floats.restype = C.c_longlong
    return int(L.nrt_moe_slot_flag_words()), int(L.nrt_moe_part_floats(hidden))


def router(args: RouterArgs, pdl=True):
    check(lib().nrt_router(C.byref(args), VP(_stream()), int(pdl)), "router")


# ----------------------------------------------------------------------------- fabric / sampler / draft / tail
class XchgArgs(C.Structure):
    _fields_ = [("box", VP * K_MAX_PEERS), ("epoch", VP), ("status", VP), ("tp", I32), ("rank", I32),
                ("timeout_ns", U64)]


class ArgmaxArgs(C.Structure):
    _fields_ = [("logits", VP), ("ld", I32), ("rows", I32), ("vlocal", I32), ("vbase", I32), ("tokens", VP), ("keys", VP),
                ("ticket", VP), ("call", I32), ("x", XchgArgs)]


def argmax_rows(args: ArgmaxArgs, pdl=True):
    """Greedy arg-max over the vocabulary shards of all ranks (lowest id on ties)."""
    L = aux_lib()
    if L.nrt_argmax_args_size() != C.sizeof(ArgmaxArgs):
        raise RuntimeError("ArgmaxArgs layout drift")
    check(L.nrt_argmax_rows(C.byref(args), VP(_stream()), int(pdl)), "argmax_rows")


class SamplerArgs(C.Structure):
    _fields_ = [("zp", VP), ("ldp", I32), ("zq", VP), ("ldq", I32), ("vlocal", I32), ("vbase", I32), ("e", VP),
                ("counts", VP), ("params", VP), ("seed", VP), ("ctrl", VP), ("block_ids", VP),
                ("n_rows_p", I32), ("n_rows_q", I32), ("st", VP), ("x", XchgArgs), ("stamps", VP)]


class TailArgs(C.Structure):
    _fields_ = [("ctrl", VP), ("block_ids", VP), ("epoch", VP), ("st", VP), ("ring", VP), ("ring_size", I32),
                ("cancel", VP), ("stop_ids", VP), ("n_stop", I32), ("counts", VP), ("vbase", I32), ("vlocal", I32),
                ("status", VP), ("n_rows_q", I32), ("host_consumed", VP), ("x", XchgArgs)]


class MarkovArgs(C.Structure):
    _fields_ = [("logits", VP), ("ld", I32), ("w1", VP), ("w2", VP), ("rank_dim", I32), ("vlocal", I32),
                ("vbase", I32), ("vocab", I32), ("block_ids", VP), ("zq", VP), ("params", VP), ("seed", VP),
                ("ctrl", VP), ("best", VP), ("ticket", VP), ("x", XchgArgs)]


class RingRecord(C.Structure):
    _fields_ = [("generation", C.c_uint), ("count", I32), ("tokens", I32 * 8), ("pos0", I32), ("stop_reason", I32),
                ("t_end_ns", U64), ("accepted", I32), ("pad", I32 * 1)]


_checked_aux = False


def aux_lib():
    """Library handle with the sampler/draft/tail struct sizes verified."""
    global _checked_aux
    L = lib()
    if not _checked_aux:
        for name, st in (("nrt_sampler_args_size", SamplerArgs), ("nrt_tail_args_size", TailArgs),
                         ("nrt_markov_args_size", MarkovArgs), ("nrt_ring_record_size", RingRecord)):
            got = getattr(L, name)()
            if got != C.sizeof(st):
                raise RuntimeError(f"{st.__name__}: library has {got} bytes, bindings {C.sizeof(st)}")
        L.nrt_philox_uniform.restype = C.c_float
        _checked_aux = True
    return L


def sampler_state_bytes() -> int:
    return aux_lib().nrt_sampler_state_size()


def sampler_run(args: SamplerArgs, domain: int = 1, pdl=True):
    check(aux_lib().nrt_sampler_run(C.byref(args), domain, VP(_stream()), int(pdl)), "sampler")


def sampler_persistent(args: SamplerArgs, sync, domain: int = 1, pdl=True) -> int:
    """The whole sampler in one launch; -3 / -9 are returned (not raised) when that form does not fit."""
    code = aux_lib().nrt_sampler_persistent(C.byref(args), domain, VP(ptr(sync)), VP(_stream()), int(pdl))
    if code in (-3, -9):
        return code
    LAUNCHES["count"] += 1
    if code != 0:
        raise RuntimeError(f"sampler failed with CUDA/driver error {code}")
    return 0


def tail_commit(args: TailArgs, pdl=True):
    check(aux_lib().nrt_tail_commit(C.byref(args), VP(_stream()), int(pdl)), "tail_commit")


def epoch_advance(epoch, pdl=True):
    check(aux_lib().nrt_epoch_advance(VP(ptr(epoch)), VP(_stream()), int(pdl)), "epoch_advance")


def draft_block_input(block_ids, embed, mask, x, rows, pdl=True):
    check(aux_lib().nrt_draft_block_input(VP(ptr(block_ids)), VP(ptr(embed)), VP(ptr(mask)), VP(ptr(x)), x.shape[1],
                                          rows, embed.shape[0], VP(_stream()), int(pdl)), "draft_block_input")


def markov_step(args: MarkovArgs, step: int, pdl=True):
    check(aux_lib().nrt_markov_step(C.byref(args), step, VP(_stream()), int(pdl)), "markov_step")


def markov_chain(args: MarkovArgs, steps: int, sync, pdl=True) -> int:
    """All ``steps`` proposals in one launch; returns -3 / -9 without raising when the launch form does not fit."""
    code = aux_lib().nrt_markov_chain(C.byref(args), steps, VP(ptr(sync)), VP(_stream()), int(pdl))
    if code in (-3, -9):
        return code
    check(code, "markov_chain")
    return 0


def philox_uniform(seed: int, domain: int, a: int, b: int) -> float:
    return float(aux_lib().nrt_philox_uniform(C.c_ulonglong(seed), C.c_uint(domain), C.c_uint(a), C.c_uint(b)))


def prefill_cursor(prompt, n_prompt, rows, ctrl, tokens, pdl=True):
    check(aux_lib().nrt_prefill_cursor(VP(ptr(prompt)), n_prompt, rows, VP(ptr(ctrl)), VP(ptr(tokens)), VP(_stream()),
                                       int(pdl)), "prefill_cursor")


def host_alloc_mapped(nbytes: int):
    """Mapped pinned host memory: (host address, device alias)."""
    h, d = C.c_void_p(), C.c_void_p()
    check(lib().nrt_host_alloc_mapped(C.byref(h), C.byref(d), C.c_size_t(nbytes)), "cudaHostAlloc")
    return h.value, d.value


def host_free(addr: int):
    lib().nrt_host_free(C.c_void_p(addr))


class AgPushArgs(C.Structure):
    _fields_ = [("src", VP), ("src_stride", I32), ("slice_bytes", I32), ("row_bytes", I32), ("gather", VP * K_MAX_PEERS),
                ("flags", VP * K_MAX_PEERS), ("epoch", VP), ("tp", I32), ("rank", I32), ("call", I32)]


def ag_push(args: AgPushArgs, pdl=True):
    L = lib()
    if L.nrt_ag_push_args_size() != C.sizeof(AgPushArgs):
        raise RuntimeError("AgPushArgs layout drift")
    check(L.nrt_ag_push(C.byref(args), VP(_stream()), int(pdl)), "ag_push")


def l2_flush(buf: torch.Tensor):
    check(lib().nrt_l2_flush(VP(buf.data_ptr()), C.c_size_t(buf.numel() * buf.element_size()), VP(_stream())), "l2_flush")


class EpArgs(C.Structure):
    _fields_ = [("topk_ids", VP), ("topk_p", VP), ("tokens", I32), ("top_k", I32), ("experts", I32), ("experts_local", I32),
                ("hidden", I32), ("slot_of", VP), ("n_items", VP), ("item_expert", VP), ("item_row", VP), ("seg_rows", VP),
                ("max_items", I32), ("cap_rows", I32), ("x", VP), ("gamma", VP), ("eps", F32),
                ("recv8", VP * K_MAX_PEERS), ("recvs", VP * K_MAX_PEERS), ("meta", VP * K_MAX_PEERS), ("flags", VP * K_MAX_PEERS),
                ("ticket", VP), ("call", I32), ("item_rows", I32), ("x_args", XchgArgs)]


class EpCombineArgs(C.Structure):
    _fields_ = [("slots", VP), ("topk_p", VP), ("resid", VP), ("out", VP), ("epoch", VP), ("status", VP),
                ("tokens", I32), ("top_k", I32), ("hidden", I32), ("call", I32), ("timeout_ns", U64)]


def _ep_lib():
    L = lib()
    if L.nrt_ep_args_size() != C.sizeof(EpArgs) or L.nrt_ep_combine_args_size() != C.sizeof(EpCombineArgs):
        raise RuntimeError("EP argument layout drift")
    return L


def ep_count(args: EpArgs, pdl=True):
    check(_ep_lib().nrt_ep_count(C.byref(args), VP(_stream()), int(pdl)), "ep_count")


def ep_dispatch(args: EpArgs, pdl=True):
    check(_ep_lib().nrt_ep_dispatch(C.byref(args), VP(_stream()), int(pdl)), "ep_dispatch")


def ep_combine(args: EpCombineArgs, pdl=True):
    check(_ep_lib().nrt_ep_combine(C.byref(args), VP(_stream()), int(pdl)), "ep_combine")


# ----------------------------------------------------------------------------- native CUDA graphs
class NativeGraph:
    """A captured CUDA graph instantiated through the runtime API (optionally for device-side launch)."""

    def __init__(self):
        self.graph, self.exec = C.c_void_p(), C.c_void_p()
        self.counts = (C.c_int * 4)()

    def begin(self, stream: int) -> None:
        check_nc(lib().nrt_graph_begin(VP(stream)), "cudaStreamBeginCapture")

    def end(self, stream: int) -> None:
        check_nc(lib().nrt_graph_end(VP(stream), C.byref(self.graph)), "cudaStreamEndCapture")
        lib().nrt_graph_inspect(self.graph, self.counts)

    def instantiate(self, device_launch: bool, stream: int) -> None:
        check_nc(lib().nrt_graph_instantiate(self.graph, int(device_launch), C.byref(self.exec)), "cudaGraphInstantiate")
        if device_launch:
            check_nc(lib().nrt_graph_upload(self.exec, VP(stream)), "cudaGraphUpload")

    def launch(self, stream: int) -> None:
        check_nc(lib().nrt_graph_launch(self.exec, VP(stream)), "cudaGraphLaunch")

    @property
    def info(self) -> dict:
        return {"nodes": self.counts[0], "kernel_nodes": self.counts[1], "edges": self.counts[2],
                "programmatic_edges": self.counts[3]}

    def destroy(self) -> None:
        lib().nrt_graph_destroy(self.graph, self.exec)
        self.graph, self.exec = C.c_void_p(), C.c_void_p()


def check_nc(code: int, what: str) -> None:
    """Like ``check`` but does not count a kernel launch."""
    if code != 0:
        raise RuntimeError(f"{what} failed with CUDA error {code}")


def relaunch(ctrl, consumed_dev_ptr: int, ring_size: int):
    check(lib().nrt_relaunch(VP(ptr(ctrl)), VP(consumed_dev_ptr), ring_size, VP(_stream())), "relaunch")


def topk_grid_state_bytes() -> int:
    return lib().nrt_topk_grid_state_bytes()


def topk_rows_grid(logits, pos0, rows, top_k, sel, state, ctas: int = 16, pdl=True):
    """Exact top-k with ``ctas`` CTAs per row (six launches); for long contexts."""
    LAUNCHES["count"] += 5
    check(lib().nrt_topk_rows_grid(VP(ptr(logits)), logits.shape[1], VP(ptr(pos0)), rows, top_k, VP(ptr(sel)), VP(ptr(state)),
                                   ctas, VP(_stream()), int(pdl)), "topk_rows_grid")
