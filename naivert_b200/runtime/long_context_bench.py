"""Long-context decode with a parked synthetic session prefix.

    python -m naivert_b200.runtime.long_context_bench --context 1048576 [--shape-tp 8] [--decode 2048]
    python -m torch.distributed.run --nproc-per-node 8 ... -m naivert_b200.runtime.long_context_bench --context 1048576

A ``context``-token session prefix is synthesised directly in the KV caches (uniform random ids; random
bf16 keys/values, random e4m3 indexer keys - replaying a million tokens is not what this measures), parked
under a session key, and then reused by two requests that each append the same 256-token suffix and decode
``decode`` tokens at the forced Bernoulli(0.7) acceptance.  Reports per-round device latency, KV bytes per
GPU, the restore time, and whether the two reuse runs produced identical tokens.
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist

from ..models.registry import resolve_model
from ..models.spec import FULL_DSA, SamplingParams
from .engine import Engine
from .session_engine import SessionEngine


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--context", type=int, default=1048576)
    ap.add_argument("--suffix", type=int, default=256)
    ap.add_argument("--decode", type=int, default=2048)
    ap.add_argument("--model", default="naive-n0.5")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--shape-tp", type=int, default=0)
    a = ap.parse_args()
    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    spec = resolve_model(a.model)
    if a.layers:
        spec = spec.with_layers(a.layers)
    capacity = -(-(a.context + a.suffix + a.decode + 256) // 128) * 128
    eng = Engine.build(spec, rank=rank, tp=world, group=group, capacity=capacity, seed=0, device=dev, shape_tp=a.shape_tp)
    eng.round.stop_ids.fill_(-1)
    g = torch.Generator(device=dev).manual_seed(123)          # same synthetic prefix on every rank (replicated parts)
    n = a.context
    for d in eng.target.layers:
        if d["kind"] == FULL_DSA:
            d["k"][:n] = torch.randn(n, *d["k"].shape[1:], device=dev, generator=g).bfloat16()
            d["v"][:n] = torch.randn(n, *d["v"].shape[1:], device=dev, generator=g).bfloat16()
            d["ik"][:n] = (torch.randn(n, d["ik"].shape[1], device=dev, generator=g) * 60).clamp_(-448, 448).to(
                torch.float8_e4m3fn).view(torch.uint8)
            d["iks"][:n] = torch.rand(n, device=dev, generator=g) * 0.01 + 0.005
        else:
            d["k"].copy_(torch.randn(d["k"].shape, device=dev, generator=g).bfloat16())
            d["v"].copy_(torch.randn(d["v"].shape, device=dev, generator=g).bfloat16())
    for L in eng.round.draft.layers:
        lo = max(0, n - 2048)                                  # the draft only ever looks 1024 positions back
        L["k"][lo:n] = torch.randn(n - lo, *L["k"].shape[1:], device=dev, generator=g).bfloat16()
        L["v"][lo:n] = torch.randn(n - lo, *L["v"].shape[1:], device=dev, generator=g).bfloat16()
    gc = torch.Generator().manual_seed(5)
    prefix = torch.randint(0, spec.vocab, (n,), generator=gc).tolist()
    suffix = torch.randint(0, spec.vocab, (a.suffix,), generator=gc).tolist()
    se = SessionEngine(eng, store_gb=64.0)
    t0 = time.perf_counter()
    se.store.save("long", prefix, n)
    torch.cuda.synchronize()
    park_s = time.perf_counter() - t0
    sp = SamplingParams(temperature=0.4, top_p=0.95, seed=1234, forced_accept_p=0.7)
    runs = []
    for _ in range(2):
        t1 = time.perf_counter()
        s = se.open_session(prefix + suffix, a.decode, "long", sp)
        open_s = time.perf_counter() - t1
        out = []
        while not s.done:
            out += s.step(300)
        ns = list(s.round_ns)
        # do not park the grown sequence: both runs must resume from the same synthetic prefix
        s.closed = True
        eng.round.launch(1)
        eng.round.stream.synchronize()
        eng.fabric.check()
        per_round_ms = (ns[-1] - ns[0]) * 1e-6 / max(1, len(ns) - 1)
        runs.append({"tokens": out, "cached": s.cached_tokens, "open_s": round(open_s, 3), "rounds": len(ns),
                     "ms_per_round": round(per_round_ms, 3), "restore_ms": s.prefill_info["restore_ms"]})
        se.active = None
    same = runs[0]["tokens"] == runs[1]["tokens"]
    if world > 1:
        flags = [None] * world
        dist.all_gather_object(flags, same)
        same = all(flags)
    if rank == 0:
        print(json.dumps({"context": n, "suffix": a.suffix, "decode": a.decode, "tp": a.shape_tp or world, "layers": spec.layer_count,
                          "diagnostic_shape_tp": a.shape_tp or None, "kv_bytes_per_gpu": eng.kv_bytes(),
                          "parked_bytes_per_gpu": se.store.bytes(), "park_s": round(park_s, 3),
                          "reuse_runs_identical": same, "cached_tokens": [r["cached"] for r in runs],
                          "ms_per_round": [r["ms_per_round"] for r in runs], "rounds": [r["rounds"] for r in runs],
                          "open_s": [r["open_s"] for r in runs], "restore_ms": [r["restore_ms"] for r in runs],
                          "tokens_per_s": [round(len(r["tokens"]) / (r["rounds"] * r["ms_per_round"] * 1e-3), 1) for r in runs]}),
              flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
