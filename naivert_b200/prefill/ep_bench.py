"""Expert-parallel all-to-all microbenchmark (one process per GPU, torchrun).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m naivert_b200.prefill.ep_bench [--tokens 4096] [--hidden 4096] [--inter 2048] [--experts 256] [--top-k 8]

``tokens`` prompt rows are row-sharded over the ranks, expert ids are drawn uniformly from the seed.
Times (device, CUDA events, max over ranks, median): the whole fused layer (count + dispatch + grouped
gate/up + grouped down with fused return + combine) and its parts; the baseline moves the same payloads
with NCCL ``all_to_all_single`` (bf16 rows out, bf16 rows back) around a torch quantise.  The NVLink
roofline is bytes leaving one GPU / 770 GB/s: e4m3 rows + scales out, bf16 rows back, for the (tp-1)/tp
share of pairs whose expert lives on another rank.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..parallel.fabric import Fabric
from .ep_moe import EPMoE

NVLINK_GBS = 770.0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--iters", type=int, default=12)
    ap.add_argument("--item-rows", type=int, default=64, help="64: chunk GEMM engine, 16: step engine tiles")
    a = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    fab = Fabric(rank, world, a.hidden, group=dist.group.WORLD if world > 1 else None, device=dev)
    T, H, I, E, Kk = a.tokens // world, a.hidden, a.inter, a.experts, a.top_k
    El = E // world
    g = torch.Generator(device=dev).manual_seed(11 + rank)

    def q8(*shape):
        w = (torch.randn(*shape, device=dev, generator=g) * 96).clamp_(-448, 448).to(torch.float8_e4m3fn)
        s = torch.full((shape[0], shape[1] // 128, shape[2] // 128), 0.02 / 96, device=dev)
        return {"w": w, "s": s}

    moe = EPMoE(fab, H, I, E, Kk, T, q8(El, I, H), q8(El, I, H), q8(El, H, I), item_rows=a.item_rows)
    x = torch.randn(T, H, device=dev, generator=g).bfloat16()
    gamma = torch.ones(H, device=dev, dtype=torch.bfloat16)
    ids = torch.stack([torch.randperm(E, device=dev, generator=g)[:Kk] for _ in range(T)]).int().contiguous()
    probs = torch.full((T, Kk), 1.0 / Kk, device=dev)
    out = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn):
        ts = []
        for _ in range(a.iters):
            K.l2_flush(flush)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(400000)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) * 1e3], device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts.append(float(t))
        return statistics.median(ts[2:])

    fused = timed(lambda: moe.run(x, gamma, ids, probs, x, out))
    fab.check()

    # parts: count + dispatch only (then let the epoch move so tags stay unique)
    def disp_only():
        ea = moe._ep_args(x, gamma, ids, probs, T)
        K.ep_count(ea, pdl=False)
        K.ep_dispatch(ea, pdl=False)
        K.epoch_advance(fab.epoch, pdl=False)

    dispatch_us = timed(disp_only)

    # NCCL baseline of the traffic only: bf16 rows out (expert-sorted), bf16 rows back
    base = None
    if world > 1:
        order = torch.argsort((ids // El).flatten(), stable=True)
        send_counts = torch.bincount((ids // El).flatten(), minlength=world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        rows_out = x.repeat_interleave(Kk, 0)[order].contiguous()
        recv = torch.empty(sum(rc), H, dtype=torch.bfloat16, device=dev)
        back = torch.empty_like(rows_out)

        def nccl():
            dist.all_to_all_single(recv, rows_out, rc, sc)
            dist.all_to_all_single(back, recv, sc, rc)

        base = timed(nccl)
    remote = (world - 1) / world
    nv_bytes = T * Kk * remote * (H + H // 128 * 4 + 16) + T * Kk * remote * H * 4      # e4m3 out; tagged bf16 words back
    roof = nv_bytes / (NVLINK_GBS * 1e9) * 1e6
    flops = 2.0 * T * Kk * 3 * H * I
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")))
    except OSError:
        pass
    bf16_peak = float(peaks.get("bf16_tflops", 1590.0))
    gemm_us = flops / (bf16_peak * 1e12) * 1e6            # expert math at the measured cuBLAS bf16 rate (no e4m3 figure is measured)
    hbm_us = El * 3.0 * H * I / (float(peaks.get("hbm_gbs", 6650.0)) * 1e9) * 1e6   # every local expert's e4m3 weights once
    target = max(roof, gemm_us, hbm_us)
    res = {"tp": world, "tokens": a.tokens, "item_rows": a.item_rows, "gemm_term_us_at_measured_bf16_peak": round(gemm_us, 1),
           "hbm_weight_term_us_at_measured_copy_rate": round(hbm_us, 1),
           "roofline_target_us": round(target, 1), "fraction_of_roofline": round(target / max(fused, 1e-9), 4), "hidden": H, "inter": I, "experts": E, "top_k": Kk,
           "fused_layer_us": round(fused, 1), "count_dispatch_us": round(dispatch_us, 1),
           "nccl_all_to_all_both_ways_us": None if base is None else round(base, 1),
           "nvlink_roofline_us": round(roof, 1), "dispatch_combine_fraction_of_roofline": round(roof / max(fused, 1e-9), 4),
           "expert_gemm_tflops_per_gpu": round(flops / (fused * 1e-6) / 1e12, 1), "items": int(moe.n_items),
           "rows_received": int(moe.seg_rows.sum())}
    if rank == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
