"""Where a speculative round spends its time: kernel timeline of whole rounds plus in-kernel phase stamps.

    python -m naivert_b200.runtime.step_profile --layers 48 --shape-tp 8 --stamp-layer 20 --out timeline.txt

builds the engine on one GPU with one rank's share of a ``--shape-tp``-way model (the per-rank shapes of the
multi-GPU deployment, no peers), opens a request with a ``--prompt``-token context, replays the captured round graph
and reports

* per kernel name: launches per round, mean device duration and mean gap to the previous kernel, from the CUPTI
  activity records of the replayed graph (``torch.profiler``, not a kernel profiler: the kernels run at full speed);
* with ``--stamp-layer L``: the ``%globaltimer`` stamps the projection / router / fused MoE kernels of layer ``L``
  write at their phase boundaries (kernel entry, barriers ready, upstream grid done, operand built, first weight
  stage landed, last MMA issued, accumulators read, partials merged, epilogue done), relative to the first stamp -
  that is the absolute in-round timeline of one layer, launch gaps included.

``--rounds 0`` skips the timeline (the process then only builds, captures and replays: the small-case driver for a
kernel profiler, e.g. ``ncu -k regex:moe_layer_kernel -c 3 python -m naivert_b200.runtime.step_profile --layers 4
--prompt 1024 --rounds 0``).

Reference counterpart: the per-kernel timing harness tests/gpu/naive_n0p5_e2e/bench_verify_kernels.py and
the wait-metrics dumps of naivert/entry/expert_down_runtime_domain.hpp.
"""
from __future__ import annotations

import argparse
import collections
import os
import sys
from typing import Dict, List

import torch

STAMP_NAMES = {
    "attn": ["entry", "upstream done", "first chunk landed", "chunks done", "merge begins (last CTA)", "done"],
    "gemm": ["entry", "barriers+tmem", "upstream done", "operand built", "first stage", "last mma", "acc read",
             "partials merged", "peer words pushed", "peer words arrived", "(polls)", "epilogue done"],
    "router": {0: "entry", 12: "upstream done", 13: "row scales", 14: "dot products", 1: "scores published",
               2: "selection begins", 10: "choices made", 15: "lists built", 3: "end"},
    "moe": {0: "entry", 12: "upstream done", 13: "row scales", 14: "dot products", 1: "scores published", 2: "arrival passed",
            10: "choices made", 15: "lists built", 3: "lists ready", 4: "first gate/up stage", 5: "last gate/up mma",
            7: "gate/up epilogue done", 6: "last down mma", 8: "down accumulators read", 9: "ranges merged", 11: "done"},
}


def _short(name: str) -> str:
    return name.replace("(anonymous namespace)::", "").replace("void ", "").replace("nrt::", "").split("(")[0][:70]


def attach_stamps(eng, layer: int) -> Dict[str, torch.Tensor]:
    """Point the stamp words of layer ``layer``'s projection / router / MoE kernels at fresh buffers.  Call before the
    round graph is captured (the pointers are kernel arguments)."""
    bufs: Dict[str, torch.Tensor] = {}
    d = eng.target.layers[layer]
    for key in ("args_qkv", "args_attn", "args_o", "args_router", "args_moe", "args_gu", "args_down"):
        if key not in d:
            continue
        b = torch.zeros(300 * 16, dtype=torch.int64, device=eng.target.x.device)
        bufs[key] = b
        if key == "args_moe":
            d[key].ar.stamps = b.data_ptr()
        else:
            d[key].stamps = b.data_ptr()
    return bufs


def attach_sampler_stamps(eng) -> torch.Tensor:
    buf = torch.zeros(32, dtype=torch.int64, device=eng.target.x.device)
    eng.round.args_sampler.stamps = buf.data_ptr()
    return buf


def report_sampler_stamps(buf: torch.Tensor) -> List[str]:
    t = buf.cpu().tolist()
    if t[30] <= 0:
        return []
    names = ["maxima", "codes", "nucleus pass 0", "nucleus pass 1", "nucleus pass 2", "nucleus pass 3 + accept", "tile masses / draw"]
    lines = ["sampler (single launch): us after kernel entry - last CTA of the phase arrived / phase released"]
    for ph, nm in enumerate(names):
        lines.append(f"   {nm:26s} {(t[2 * ph] - t[30]) / 1e3:8.2f} / {(t[2 * ph + 1] - t[30]) / 1e3:8.2f}")
    return lines


def report_stamps(bufs: Dict[str, torch.Tensor], layer: int) -> List[str]:
    import numpy as np
    if any(b.is_cuda for b in bufs.values()):
        torch.cuda.synchronize()
    lines: List[str] = []
    T = {k: b.view(300, 16).cpu().numpy() for k, b in bufs.items()}
    t0 = min(t[:, 0][t[:, 0] > 0].min() for t in T.values() if (t[:, 0] > 0).any())
    for k, t in T.items():
        t = t[t[:, 0] > 0]
        if len(t) == 0:
            continue
        names = STAMP_NAMES["router"] if k == "args_router" else STAMP_NAMES["moe"] if k == "args_moe" else None
        if k == "args_attn":
            t8 = bufs[k][:300 * 16].view(600, 8).cpu().numpy()
            t8 = t8[t8[:, 0] > 0]
            lines.append(f"layer {layer} attn: {len(t8)} CTAs; us after the layer's first stamp (median over CTAs / last CTA)")
            for i, label in enumerate(["entry", "upstream done", "first chunk landed", "chunks done", "merge begins (last CTA)", "done"]):
                col = t8[:, i]
                col = col[col > t0]
                if len(col):
                    lines.append(f"   {label:26s} {(np.median(col) - t0) / 1e3:8.2f} / {(col.max() - t0) / 1e3:8.2f}   ({len(col)} CTAs)")
            continue
        lines.append(f"layer {layer} {k[5:]}: {len(t)} CTAs; us after the layer's first stamp (median over CTAs / last CTA)")
        order = sorted(range(16), key=lambda i: np.median(t[:, i][t[:, i] > t0]) if (t[:, i] > t0).any() else 1e30)
        for i in order:
            if names is None and i == 10:           # a count, not a time
                if t[:, 10].max() > 0:
                    lines.append(f"   {'mailbox sweeps (max)':26s} {int(t[:, 10].max()):8d}")
                continue
            col = t[:, i]
            col = col[col > t0]                     # stamps of earlier replays (a CTA that was not last this time) lie before t0
            if len(col) == 0:
                continue
            label = names.get(i, str(i)) if names else STAMP_NAMES["gemm"][i] if i < 12 else {12: "row scales ready", 14: "operand stored"}.get(i, str(i))
            lines.append(f"   {label:26s} {(np.median(col) - t0) / 1e3:8.2f} / {(col.max() - t0) / 1e3:8.2f}   ({len(col)} CTAs)")
    return lines


def main(argv: List[str] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="naive-n0.5")
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--shape-tp", type=int, default=8, help="per-rank shapes of this tensor-parallel degree (single-rank fabric)")
    ap.add_argument("--prompt", type=int, default=8192)
    ap.add_argument("--rounds", type=int, default=4, help="rounds under the activity trace (0: none)")
    ap.add_argument("--warm", type=int, default=10)
    ap.add_argument("--stamp-layer", type=int, default=-1)
    ap.add_argument("--pdl", dest="pdl", action="store_true", default=None)
    ap.add_argument("--no-pdl", dest="pdl", action="store_false")
    ap.add_argument("--out", default=None, help="write the report to this file as well")
    a = ap.parse_args(argv)

    from ..models.registry import resolve_model
    from ..models.spec import SamplingParams
    from .engine import Engine

    spec = resolve_model(a.model)
    if a.layers < spec.layer_count:
        spec = spec.with_layers(a.layers)
    dev = torch.device("cuda", 0)
    eng = Engine.build(spec, rank=0, tp=1, group=None, capacity=a.prompt + 1024, seed=0, device=dev, pdl=a.pdl, shape_tp=a.shape_tp)
    eng.round.stop_ids.fill_(-1)
    bufs = attach_stamps(eng, a.stamp_layer) if a.stamp_layer >= 0 else {}
    samp_stamps = attach_sampler_stamps(eng) if a.stamp_layer >= 0 else None
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, spec.vocab, (a.prompt,), generator=g, dtype=torch.int32)
    sp = SamplingParams(temperature=0.4, top_p=0.95, seed=1234, forced_accept_p=0.7)
    eng.open(prompt, 8 * (a.warm + max(a.rounds, 1)) + 64, sp)
    r = eng.round
    r.launch(a.warm)
    for _ in range(a.warm):
        r.wait_round(120)
    torch.cuda.synchronize()
    lines: List[str] = [f"model {spec.name} shape_tp {a.shape_tp} prompt {a.prompt} pdl {r.pdl} kernels/round {r.kernels_per_round}"]
    if a.rounds > 0:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            r.launch(a.rounds)
            for _ in range(a.rounds):
                r.wait_round(120)
            torch.cuda.synchronize()
        ks = sorted(((e.time_range.start, e.time_range.end, e.name) for e in prof.events()
                     if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda t: t[0])
        agg: Dict[str, list] = collections.OrderedDict()
        prev_end = None
        for st, en, name in ks:
            v = agg.setdefault(_short(name), [0, 0.0, 0.0])
            v[0] += 1
            v[1] += en - st
            if prev_end is not None:
                v[2] += max(0.0, st - prev_end)
            prev_end = max(en, prev_end or en)
        span = ks[-1][1] - ks[0][0]
        busy, gaps = sum(v[1] for v in agg.values()), sum(v[2] for v in agg.values())
        lines.append(f"rounds {a.rounds} us/round {span / a.rounds:.1f} sum of kernel durations/round {busy / a.rounds:.1f} "
                     f"gaps/round {gaps / a.rounds:.1f}")
        for k, v in sorted(agg.items(), key=lambda kv: -(kv[1][1] + kv[1][2])):
            lines.append(f"{k:70s} n/round {v[0] / a.rounds:6.1f} us {v[1] / v[0]:7.2f} gap before {v[2] / v[0]:5.2f} "
                         f"us/round {(v[1] + v[2]) / a.rounds:8.1f}")
    if bufs:
        lines += report_stamps(bufs, a.stamp_layer)
    if samp_stamps is not None:
        lines += report_sampler_stamps(samp_stamps)
    eng.close()
    text = "\n".join(lines)
    print(text)
    if a.out:
        os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
        with open(a.out, "w") as f:
            f.write(text + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
