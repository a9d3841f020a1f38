"""Chunked native prefill throughput on the full-size geometry.

    python -m naivert_b200.prefill.prefill_bench --tokens 131072 [--chunk 4096] [--layers 16] [--moe ep|tp]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m naivert_b200.prefill.prefill_bench --tokens 131072

Random-init weights drawn on the device (expert-parallel copies of the experts are drawn independently of
the tensor-parallel slices: a benchmark model), uniform random prompt in pinned host memory.  One untimed
warm-up pass over two chunk sizes, then the whole prompt is ingested once: CUDA events around the run on the
launching stream, maximum over the ranks.  A second pass with per-stage events gives the breakdown (not the
headline number).  Prints one JSON line from rank 0.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..models.registry import resolve_model
from ..runtime.engine import Engine


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=131072)
    ap.add_argument("--chunk", type=int, default=4096)
    ap.add_argument("--model", default="naive-n0.5")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--moe", choices=("ep", "tp"), default="ep")
    ap.add_argument("--breakdown-tokens", type=int, default=0, help="rows of the per-stage pass (default: two chunks at the end)")
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
    capacity = -(-(a.tokens + 512) // 128) * 128
    ep_w = None
    if world > 1 and a.moe == "ep":
        from ..models.device_init import init_expert_rank_weights_device
        ep_w = init_expert_rank_weights_device(spec, rank, world, seed=0, device=dev)
    eng = Engine.build(spec, rank=rank, tp=world, group=group, capacity=capacity, seed=0, device=dev,
                       prefill_chunk=a.chunk, ep_weights=ep_w)
    del ep_w
    pf = eng.prefill
    g = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, spec.vocab - 16, (a.tokens + 1,), generator=g, dtype=torch.int32).pin_memory()
    stream = eng.round.stream
    with torch.cuda.stream(stream):
        pf.warm_chunks([pf.quantum, a.chunk])
        pos = pf.run(prompt, 0, a.tokens)
        ms = pf.executor_ms()
        pf.check()
        # per-stage pass over the last rows (the caches before them are valid from the timed pass)
        n_bd = a.breakdown_tokens or min(a.tokens, 2 * a.chunk)
        pf.profile = True
        pf.run(prompt, a.tokens - n_bd, a.tokens)
        stages = pf.stage_ms()
        pf.profile = False
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    tot = sum(stages.values()) or 1.0
    out = {"metric": "chunked native prefill tokens/s", "value": round(pos / (ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": world,
           "tokens": pos, "ms": round(ms, 2), "chunk": a.chunk, "layers": spec.layer_count,
           "moe": "ep" if pf.ep else ("local" if world == 1 else "tp"), "dtype": "fp8 weights/activations, bf16 residual",
           "data": "synthetic: device-drawn random weights, uniform random prompt (pinned host)",
           "breakdown_rows": n_bd, "stage_ms": stages, "stage_share": {k: round(v / tot, 3) for k, v in stages.items()},
           "kv_bytes_per_gpu": eng.kv_bytes(), "status": int(eng.fabric.status[0])}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
