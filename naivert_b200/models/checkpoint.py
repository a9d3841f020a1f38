"""Safetensors checkpoints in the reference layout: header-only validation, identity
digests, sharded index, random-init writer, and the TP-sliced loader.

Layout (reference naivert/checkpoint.py:33,152,271 and
naivert/models/naive_n0p5/checkpoint_fp8.py:74-94): the target is a directory with
``config.json``, ``model.safetensors.index.json`` (``weight_map`` name -> shard file) and
``model-XXXXX-of-YYYYY.safetensors`` shards; the draft is a single ``model.safetensors``
plus ``config.json`` carrying ``dflash_config``.  Allowed dtypes: BF16, F32, F8_E4M3.

Identity: the reference pins SHA-256 digests of config, index and tensor metadata of the
released checkpoint.  Here the same digests are *computed and reported*
(``CheckpointIdentity``) and may be pinned by the caller (``expect=``), so random-init
checkpoints written by ``write_target_checkpoint`` load through the same checks.
"""
from __future__ import annotations

import hashlib
import json
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Mapping, Optional, Tuple

import torch

from .spec import FULL_DSA, SLIDING_WINDOW, ModelSpec
from .weights import (StateDict, init_draft_state_dict, init_state_dict, prepare_draft_weights,
                      prepare_weights, shard_draft_weights, shard_weights)

ALLOWED_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F8_E4M3": torch.float8_e4m3fn}
_DTYPE_NAMES = {v: k for k, v in ALLOWED_DTYPES.items()}
INDEX_NAME = "model.safetensors.index.json"


class CheckpointError(ValueError):
    pass


# --------------------------------------------------------------------------- header-only reader
def read_header(path: str) -> Dict[str, dict]:
    """Parse the JSON header of one safetensors file without touching tensor bytes."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise CheckpointError(f"{path}: truncated header length")
        (n,) = struct.unpack("<Q", raw)
        if n > size - 8 or n > 512 << 20:
            raise CheckpointError(f"{path}: header length {n} exceeds file size")
        header = json.loads(f.read(n))
    header.pop("__metadata__", None)
    end = 0
    spans = []
    for name, meta in header.items():
        if meta["dtype"] not in ALLOWED_DTYPES:
            raise CheckpointError(f"{path}: tensor {name} has unsupported dtype {meta['dtype']}")
        lo, hi = meta["data_offsets"]
        numel = 1
        for d in meta["shape"]:
            numel *= d
        if hi - lo != numel * torch.empty((), dtype=ALLOWED_DTYPES[meta["dtype"]]).element_size():
            raise CheckpointError(f"{path}: tensor {name} byte range does not match its shape")
        end = max(end, hi)
        spans.append((lo, hi, name))
    if 8 + n + end > size:
        raise CheckpointError(f"{path}: tensor data runs past end of file")
    # payload intervals tile [0, end) without gaps or overlaps (the format writes tensors back to back)
    at = 0
    for lo, hi, name in sorted(spans):
        if lo != at:
            raise CheckpointError(f"{path}: tensor {name} starts at byte {lo}, expected {at} (overlapping or non-contiguous payload)")
        at = hi
    return header


@dataclass(frozen=True)
class CheckpointIdentity:
    config_sha256: str
    index_sha256: str
    metadata_sha256: str
    tensor_count: int
    dtype_counts: Mapping[str, int]

    def require(self, expect: Optional["CheckpointIdentity"]) -> None:
        if expect is not None and (self.config_sha256, self.index_sha256, self.metadata_sha256) != (
                expect.config_sha256, expect.index_sha256, expect.metadata_sha256):
            raise CheckpointError("checkpoint identity does not match the pinned digests")


def _sha(b: bytes) -> str:
    return hashlib.sha256(b).hexdigest()


class LocalCheckpoint:
    """A checkpoint directory resolved to its files, headers and identity."""

    def __init__(self, root: str):
        self.root = root
        cfg = os.path.join(root, "config.json")
        if not os.path.isfile(cfg):
            raise CheckpointError(f"{root}: missing config.json")
        self.config_bytes = open(cfg, "rb").read()
        self.config = json.loads(self.config_bytes)
        idx = os.path.join(root, INDEX_NAME)
        if os.path.isfile(idx):
            self.index_bytes = open(idx, "rb").read()
            self.weight_map: Dict[str, str] = json.loads(self.index_bytes)["weight_map"]
        else:
            single = os.path.join(root, "model.safetensors")
            if not os.path.isfile(single):
                raise CheckpointError(f"{root}: neither {INDEX_NAME} nor model.safetensors")
            self.index_bytes = b""
            self.weight_map = {k: "model.safetensors" for k in read_header(single)}
        self.headers = {f: read_header(os.path.join(root, f)) for f in sorted(set(self.weight_map.values()))}
        for name, f in self.weight_map.items():
            if name not in self.headers[f]:
                raise CheckpointError(f"index maps {name} to {f}, which does not contain it")

    def identity(self) -> CheckpointIdentity:
        meta = {n: (self.headers[f][n]["dtype"], self.headers[f][n]["shape"], f, self.headers[f][n]["data_offsets"])
                for n, f in self.weight_map.items()}
        counts: Dict[str, int] = {}
        for dt, *_ in meta.values():
            counts[dt] = counts.get(dt, 0) + 1
        return CheckpointIdentity(_sha(self.config_bytes), _sha(self.index_bytes),
                                  _sha(json.dumps(meta, sort_keys=True).encode()), len(meta), counts)

    def load_tensors(self, names: Optional[Iterable[str]] = None, device="cpu") -> StateDict:
        from safetensors import safe_open
        want = set(self.weight_map) if names is None else set(names)
        missing = want - set(self.weight_map)
        if missing:
            raise CheckpointError(f"tensors not in checkpoint: {sorted(missing)[:4]} ...")
        out: StateDict = {}
        by_file: Dict[str, list] = {}
        for n in want:
            by_file.setdefault(self.weight_map[n], []).append(n)
        for f, ns in by_file.items():
            with safe_open(os.path.join(self.root, f), framework="pt", device=str(device)) as sf:
                for n in ns:
                    out[n] = sf.get_tensor(n)
        return out


def resolve_checkpoint(name_or_path: str, roots_env: str = "NAIVERT_MODEL_ROOTS") -> str:
    """Directory, or a short name under one of the ``roots_env`` directories; a directory
    holding ``step_*`` children resolves to the newest one (examples/serve_sessions.py:27-54)."""
    cands = [name_or_path] + [os.path.join(r, name_or_path) for r in os.environ.get(roots_env, "").split(":") if r]
    for c in cands:
        if os.path.isdir(c):
            steps = sorted((d for d in os.listdir(c) if d.startswith("step_") and os.path.isdir(os.path.join(c, d))),
                           key=lambda d: int(d.split("_")[1]) if d.split("_")[1].isdigit() else -1)
            return os.path.join(c, steps[-1]) if steps and not os.path.isfile(os.path.join(c, "config.json")) else c
    raise CheckpointError(f"checkpoint {name_or_path!r} not found (searched {cands})")


def list_weights(model_roots_env: str = "NAIVERT_MODEL_ROOTS", draft_roots_env: str = "NAIVERT_DRAFT_ROOTS") -> str:
    """The checkpoints found under the root directories, as the short names ``resolve_checkpoint`` accepts: targets
    are directories (or their newest ``step_*`` child) with ``config.json`` and a shard index, drafts directories with
    ``config.json`` and a single ``model.safetensors`` (``--list-weights`` of examples/serve_sessions.py:57-72)."""
    def roots(env):
        return [r for r in os.environ.get(env, "").split(":") if r and os.path.isdir(r)]

    lines = ["targets (--target):"]
    for base in roots(model_roots_env):
        for name in sorted(os.listdir(base)):
            try:
                d = resolve_checkpoint(os.path.join(base, name))
            except CheckpointError:
                continue
            if os.path.isfile(os.path.join(d, "config.json")) and os.path.isfile(os.path.join(d, INDEX_NAME)):
                lines.append(f"  {name:48s} {d}")
    lines.append("drafts (--draft):")
    for base in roots(draft_roots_env):
        for name in sorted(os.listdir(base)):
            d = os.path.join(base, name)
            if os.path.isfile(os.path.join(d, "config.json")) and os.path.isfile(os.path.join(d, "model.safetensors")):
                lines.append(f"  {name:48s} {d}")
    return "\n".join(lines)


# --------------------------------------------------------------------------- config.json
def target_config(spec: ModelSpec) -> dict:
    dsa, swa = spec.attention[FULL_DSA], spec.attention[SLIDING_WINDOW]
    rt, ix = spec.routing, spec.indexer
    return {
        "model_type": "naive_n0p5", "hidden_size": spec.hidden, "vocab_size": spec.vocab,
        "num_hidden_layers": spec.layer_count,
        "hybrid_layer_pattern": [0 if k == FULL_DSA else 1 for k in spec.layer_kinds],
        "num_attention_heads": dsa.head_count, "num_key_value_heads": dsa.kv_head_count,
        "swa_num_key_value_heads": swa.kv_head_count, "head_dim": dsa.head_dim, "v_head_dim": dsa.v_head_dim,
        "rope_dim": dsa.rope_dim, "rope_theta": dsa.rope_theta, "swa_rope_theta": swa.rope_theta,
        "sliding_window": swa.sliding_window, "value_scale": dsa.value_scale,
        "index_n_heads": ix.head_count, "index_head_dim": ix.head_dim, "index_rope_dim": ix.rope_dim,
        "index_topk": ix.top_k, "n_routed_experts": rt.expert_count, "num_experts_per_tok": rt.top_k,
        "moe_intermediate_size": rt.intermediate, "n_shared_experts": rt.shared_expert_count,
        "scoring_func": rt.score_func, "routed_scaling_factor": rt.route_scale, "norm_topk_prob": rt.normalize_top_k,
        "first_k_dense_replace": spec.dense_layer_count, "intermediate_size": spec.dense_intermediate,
        "rms_norm_eps": spec.norm_eps, "eos_token_id": list(spec.stop_token_ids),
        "quantization_config": {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [128, 128],
                                "ignored_layers": ["self_attn", "mlp.gate", "lm_head", "embed_tokens"]}
        if spec.weight_dtype == "fp8" else None,
    }


def draft_config(spec: ModelSpec) -> dict:
    d = spec.draft
    return {
        "hidden_size": d.hidden, "intermediate_size": d.intermediate, "num_hidden_layers": d.layer_count,
        "num_attention_heads": d.head_count, "num_key_value_heads": d.kv_head_count, "head_dim": d.head_dim,
        "vocab_size": spec.vocab, "markov_rank": d.markov_rank, "block_size": d.block_size,
        "rms_norm_eps": d.norm_eps, "sliding_window": d.window, "use_sliding_window": True,
        "layer_types": ["sliding_attention"] * d.layer_count, "hidden_act": "silu",
        "markov_head_type": "vanilla",
        "dflash_config": {"target_layer_ids": list(d.target_layer_ids), "mask_token_id": d.mask_token_id,
                          "use_mask_embedding": True},
        "rope_parameters": {"rope_theta": d.rope_theta, "rope_type": "default"},
    }


def validate_draft_config(spec: ModelSpec, cfg: dict) -> None:
    """Refuse a draft checkpoint with different math (naivert/models/naive_n0p5/dspark.py:29-58)."""
    want = draft_config(spec)
    for key in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                "num_key_value_heads", "head_dim", "vocab_size", "markov_rank", "block_size",
                "sliding_window"):
        if cfg.get(key) != want[key]:
            raise CheckpointError(f"unsupported draft {key}: {cfg.get(key)!r} (expected {want[key]!r})")
    flash = cfg.get("dflash_config", {})
    if tuple(flash.get("target_layer_ids", ())) != tuple(spec.draft.target_layer_ids) \
            or flash.get("mask_token_id") != spec.draft.mask_token_id:
        raise CheckpointError("unsupported draft feature-tap / mask-token contract")


# --------------------------------------------------------------------------- writer
def _save_shards(root: str, sd: StateDict, shard_bytes: int) -> Dict[str, str]:
    from safetensors.torch import save_file
    groups, cur, size = [], {}, 0
    for name in sorted(sd):
        t = sd[name]
        nbytes = t.numel() * t.element_size()
        if cur and size + nbytes > shard_bytes:
            groups.append(cur)
            cur, size = {}, 0
        cur[name] = t.contiguous()
        size += nbytes
    if cur:
        groups.append(cur)
    weight_map = {}
    for i, g in enumerate(groups):
        fname = f"model-{i + 1:05d}-of-{len(groups):05d}.safetensors"
        save_file(g, os.path.join(root, fname))
        for n in g:
            weight_map[n] = fname
    return weight_map


def write_target_checkpoint(root: str, spec: ModelSpec, seed: int = 0, shard_bytes: int = 2 << 30,
                            state_dict: Optional[StateDict] = None) -> CheckpointIdentity:
    os.makedirs(root, exist_ok=True)
    sd = state_dict if state_dict is not None else init_state_dict(spec, seed)
    for n, t in sd.items():
        if t.dtype not in _DTYPE_NAMES:
            raise CheckpointError(f"{n}: dtype {t.dtype} is not storable in this layout")
    with open(os.path.join(root, "config.json"), "w") as f:
        json.dump(target_config(spec), f, indent=1, sort_keys=True)
    wm = _save_shards(root, sd, shard_bytes)
    total = sum(t.numel() * t.element_size() for t in sd.values())
    with open(os.path.join(root, INDEX_NAME), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": wm}, f, indent=1, sort_keys=True)
    return LocalCheckpoint(root).identity()


def write_draft_checkpoint(root: str, spec: ModelSpec, seed: int = 1,
                           state_dict: Optional[StateDict] = None) -> CheckpointIdentity:
    from safetensors.torch import save_file
    os.makedirs(root, exist_ok=True)
    sd = state_dict if state_dict is not None else init_draft_state_dict(spec, seed)
    with open(os.path.join(root, "config.json"), "w") as f:
        json.dump(draft_config(spec), f, indent=1, sort_keys=True)
    save_file({k: v.contiguous() for k, v in sd.items()}, os.path.join(root, "model.safetensors"))
    return LocalCheckpoint(root).identity()


# --------------------------------------------------------------------------- loader
def expected_target_names(spec: ModelSpec) -> Dict[str, str]:
    """name -> dtype string of every tensor the target layout must contain."""
    fp8 = spec.weight_dtype == "fp8"
    w = "BF16" if fp8 else "F32"
    out = {"model.embed_tokens.weight": w, "model.norm.weight": w, "lm_head.weight": w}
    rt = spec.routing
    for L, kind in enumerate(spec.layer_kinds):
        p = f"model.layers.{L}."
        for n in ("input_layernorm", "post_attention_layernorm"):
            out[p + n + ".weight"] = w
        for n in ("q", "k", "v", "o"):
            out[p + f"self_attn.{n}_proj.weight"] = w
        if spec.attention[kind].sink_bias:
            out[p + "self_attn.attention_sink_bias"] = w
        if kind == FULL_DSA:
            for n in ("wq.weight", "wk.weight", "weights_proj.weight", "k_norm.weight", "k_norm.bias"):
                out[p + "self_attn.indexer." + n] = w
        if spec.is_dense(L):
            for n in ("gate", "up", "down"):
                out[p + f"mlp.{n}_proj.weight"] = w
        else:
            out[p + "mlp.gate.weight"] = "F32"
            if rt.score_func == "sigmoid":
                out[p + "mlp.gate.e_score_correction_bias"] = "F32"
            groups = [("experts", rt.expert_count), ("shared_experts", rt.shared_expert_count)]
            for gname, cnt in groups:
                for e in range(cnt):
                    for n in ("gate", "up", "down"):
                        out[p + f"mlp.{gname}.{e}.{n}_proj.weight"] = "F8_E4M3" if fp8 else "F32"
                        if fp8:
                            out[p + f"mlp.{gname}.{e}.{n}_proj.weight_scale_inv"] = "F32"
    return out


def validate_target_layout(spec: ModelSpec, ckpt: LocalCheckpoint) -> None:
    want = expected_target_names(spec)
    have = {n: ckpt.headers[f][n]["dtype"] for n, f in ckpt.weight_map.items()}
    missing = sorted(set(want) - set(have))
    if missing:
        raise CheckpointError(f"checkpoint lacks {len(missing)} tensors, e.g. {missing[:3]}")
    wrong = [n for n, dt in want.items() if have[n] != dt]
    if wrong:
        raise CheckpointError(f"dtype mismatch for {wrong[:3]}")
    pat = ckpt.config.get("hybrid_layer_pattern")
    if pat is not None and list(pat) != [0 if k == FULL_DSA else 1 for k in spec.layer_kinds]:
        raise CheckpointError("hybrid_layer_pattern does not match the model geometry")


class SliceReader:
    """Reads rows / columns of checkpoint tensors straight from the shards (``safe_open(...).get_slice``): a rank
    touches only the bytes it owns.  Shard handles stay open for the lifetime of the reader.
    Parity: the sliced reads of naivert/models/naive_n0p5/checkpoint_fp8.py:149-224."""

    def __init__(self, ckpt: "LocalCheckpoint"):
        self.ckpt, self._open = ckpt, {}
        self.bytes_read = 0

    def _slice(self, name: str):
        from safetensors import safe_open
        f = self.ckpt.weight_map[name]
        if f not in self._open:
            self._open[f] = safe_open(os.path.join(self.ckpt.root, f), framework="pt", device="cpu").__enter__()
        return self._open[f].get_slice(name)

    def _count(self, t: torch.Tensor) -> torch.Tensor:
        self.bytes_read += t.numel() * t.element_size()
        return t

    def has(self, name: str) -> bool:
        return name in self.ckpt.weight_map

    def full(self, name: str) -> torch.Tensor:
        return self._count(self._slice(name)[:])

    def rows(self, name: str, lo: int, hi: int) -> torch.Tensor:
        return self._count(self._slice(name)[lo:hi])

    def cols(self, name: str, lo: int, hi: int) -> torch.Tensor:
        return self._count(self._slice(name)[:, lo:hi])

    def close(self) -> None:
        for h in self._open.values():
            h.__exit__(None, None, None)
        self._open = {}


def load_rank_weights_sliced(spec: ModelSpec, ckpt: "LocalCheckpoint", rank: int, tp: int, reader: Optional[SliceReader] = None) -> dict:
    """The weights rank ``rank`` of ``tp`` owns, read slice by slice: equal to
    ``shard_weights(spec, prepare_weights(spec, full_state_dict), rank, tp)`` without ever holding the full
    checkpoint (about 300 GB at full size) in host memory.  q / k rows are re-ordered for adjacent-pair RoPE per
    head, so a slice of whole heads is transformed exactly like the full matrix; the 128 x 128 e4m3 blocks of
    o_proj / dense weights are cut on block boundaries, so quantising a slice equals slicing the quantised matrix."""
    from .weights import _q8, interleave_rope
    own = reader is None
    rd = reader or SliceReader(ckpt)
    fp8 = spec.weight_dtype == "fp8"
    ix, rt = spec.indexer, spec.routing
    V = spec.vocab_shard(tp)
    try:
        out = {"embed": rd.full("model.embed_tokens.weight"), "norm": rd.full("model.norm.weight"),
               "lm_head": rd.rows("lm_head.weight", rank * V, (rank + 1) * V).contiguous(), "layers": []}
        for L, kind in enumerate(spec.layer_kinds):
            a = spec.attention[kind]
            p = f"model.layers.{L}."
            nh = a.local_heads(tp)
            kvs = a.kv_head_for_rank(rank, tp)
            r = {"kind": kind, "g_in": rd.full(p + "input_layernorm.weight"), "g_post": rd.full(p + "post_attention_layernorm.weight")}
            r["wq"] = interleave_rope(rd.rows(p + "self_attn.q_proj.weight", rank * nh * a.head_dim, (rank + 1) * nh * a.head_dim),
                                      nh, a.head_dim, a.rope_dim)
            r["wk"] = torch.cat([interleave_rope(rd.rows(p + "self_attn.k_proj.weight", h * a.head_dim, (h + 1) * a.head_dim),
                                                 1, a.head_dim, a.rope_dim) for h in kvs]).contiguous()
            r["wv"] = torch.cat([rd.rows(p + "self_attn.v_proj.weight", h * a.v_head_dim, (h + 1) * a.v_head_dim)
                                 for h in kvs]).contiguous()
            r["wo"] = _q8(rd.cols(p + "self_attn.o_proj.weight", rank * nh * a.v_head_dim, (rank + 1) * nh * a.v_head_dim).contiguous(), fp8)
            sink = p + "self_attn.attention_sink_bias"
            r["sink"] = rd.rows(sink, rank * nh, (rank + 1) * nh).contiguous() if rd.has(sink) else None
            if kind == FULL_DSA:
                q = p + "self_attn.indexer."
                r["iwq"] = interleave_rope(rd.full(q + "wq.weight"), ix.head_count, ix.head_dim, ix.rope_dim)
                r["iwk"] = interleave_rope(rd.full(q + "wk.weight"), 1, ix.head_dim, ix.rope_dim)
                r["iww"] = rd.full(q + "weights_proj.weight")
                r["ik_w"] = interleave_rope(rd.full(q + "k_norm.weight"), 1, ix.head_dim, ix.rope_dim)
                r["ik_b"] = interleave_rope(rd.full(q + "k_norm.bias"), 1, ix.head_dim, ix.rope_dim)
            if spec.is_dense(L):
                I = spec.dense_inter_local(tp)
                r["dense"] = {"gate": _q8(rd.rows(p + "mlp.gate_proj.weight", rank * I, (rank + 1) * I).contiguous(), fp8),
                              "up": _q8(rd.rows(p + "mlp.up_proj.weight", rank * I, (rank + 1) * I).contiguous(), fp8),
                              "down": _q8(rd.cols(p + "mlp.down_proj.weight", rank * I, (rank + 1) * I).contiguous(), fp8)}
            else:
                I = spec.expert_inter_local(tp)
                r["router_w"] = rd.full(p + "mlp.gate.weight").float()
                bias = p + "mlp.gate.e_score_correction_bias"
                r["router_b"] = rd.full(bias).float() if rd.has(bias) else torch.zeros(rt.expert_count)
                names = [p + f"mlp.experts.{e}." for e in range(rt.expert_count)]
                names += [p + f"mlp.shared_experts.{e}." for e in range(rt.shared_expert_count)]
                if fp8 and (I % 128 or (rank * I) % 128):
                    raise CheckpointError(f"expert slice of {I} channels is not aligned to the 128-wide scale blocks")
                b0, b1 = rank * I // 128, -(-(rank + 1) * I // 128)
                for name in ("gate", "up", "down"):
                    ws, ss = [], []
                    for q in names:
                        t = q + f"{name}_proj.weight"
                        if name == "down":
                            ws.append(rd.cols(t, rank * I, (rank + 1) * I).contiguous())
                            if fp8:
                                ss.append(rd.cols(t + "_scale_inv", b0, b1).contiguous())
                        else:
                            ws.append(rd.rows(t, rank * I, (rank + 1) * I).contiguous())
                            if fp8:
                                ss.append(rd.rows(t + "_scale_inv", b0, b1).contiguous())
                    r[name] = {"w": torch.stack(ws), "s": torch.stack(ss) if fp8 else None}
            out["layers"].append(r)
        return out
    finally:
        if own:
            rd.close()


def load_rank_weights(spec: ModelSpec, root: str, rank: int, tp: int, device="cpu",
                      expect: Optional[CheckpointIdentity] = None) -> Tuple[dict, CheckpointIdentity]:
    """Validate a target checkpoint and read the slices one rank owns (nothing else is read from the shards)."""
    ckpt = LocalCheckpoint(root)
    ident = ckpt.identity()
    ident.require(expect)
    validate_target_layout(spec, ckpt)
    w = load_rank_weights_sliced(spec, ckpt, rank, tp)
    from .tensor_abi import check_rank_weights
    check_rank_weights(spec, w, rank, tp)                       # every slot present with the shape the kernels expect
    return _to_device(w, device), ident


def load_draft_rank_weights(spec: ModelSpec, root: str, rank: int, tp: int, device="cpu"):
    ckpt = LocalCheckpoint(root)
    validate_draft_config(spec, ckpt.config)
    sd = ckpt.load_tensors(device="cpu")
    return _to_device(shard_draft_weights(spec, prepare_draft_weights(spec, sd), rank, tp), device), ckpt.identity()


def _to_device(obj, device):
    if isinstance(obj, torch.Tensor):
        return obj.to(device)
    if isinstance(obj, dict):
        return {k: _to_device(v, device) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_device(v, device) for v in obj)
    return obj
