"""Worker of the chunked native prefill test (plain process at world 1, torchrun beyond).

One engine ingests the same prompt twice: by eight-row replay and by the chunked native prefill
(tensor-parallel attention; expert-parallel MoE when WORLD_SIZE > 1), then decodes.  The caches both
paths leave behind are compared: bitwise where the arithmetic is the same (single rank, layers before
the first MoE output), by relative error elsewhere.  Prints one JSON line from rank 0.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).abs().mean() / b.abs().mean().clamp_min(1e-9)).item()


def main():
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    else:
        # single rank: take the K split and the key split out of the replay so that both paths add in the same order
        os.environ["NAIVERT_SPLIT_MIN_KB"] = "100000"
    from naivert_b200.models.naive_n0p5 import small_w8a8_spec
    from naivert_b200.models.spec import FULL_DSA, SamplingParams
    from naivert_b200.models.weights import (init_draft_state_dict, init_state_dict, prepare_draft_weights, prepare_weights,
                                             shard_draft_weights, shard_expert_weights, shard_weights)
    from naivert_b200.runtime.engine import Engine

    spec = small_w8a8_spec(4)
    w = prepare_weights(spec, init_state_dict(spec, seed=0, device=dev))
    dw = prepare_draft_weights(spec, init_draft_state_dict(spec, seed=1, device=dev))
    eng = Engine.build(spec, rank=rank, tp=world, group=dist.group.WORLD if world > 1 else None, capacity=2048, device=dev,
                       weights=shard_weights(spec, w, rank, world), draft_weights=shard_draft_weights(spec, dw, rank, world),
                       prefill_chunk=256,
                       ep_weights=shard_expert_weights(spec, w, rank, world) if (world > 1 and os.environ.get("PREFILL_MOE", "ep") == "ep") else None)
    if world == 1:
        eng.target.attn_splits = 1
    g = torch.Generator().manual_seed(3)
    n = 700
    prompt = torch.randint(0, spec.vocab - 16, (n,), generator=g)
    sp = SamplingParams(top_p=1e-6, seed=9, forced_accept_p=0.0)            # greedy
    t, dr = eng.target, eng.round.draft

    def caches():
        out = []
        for d in t.layers:
            out += [d["k"], d["v"]] + ([d["ik"], d["iks"]] if d["kind"] == FULL_DSA else [])
        for L in dr.layers:
            out += [L["k"], L["v"]]
        return out

    def snapshot(upto):
        snap = {}
        for i, d in enumerate(t.layers):
            if d["kind"] == FULL_DSA:
                snap[f"L{i}.k"], snap[f"L{i}.v"] = d["k"][:upto].clone(), d["v"][:upto].clone()
                snap[f"L{i}.ik"], snap[f"L{i}.iks"] = d["ik"][:upto].clone(), d["iks"][:upto].clone()
            else:
                win = spec.attention[d["kind"]].sliding_window
                slots = torch.arange(upto - win, upto, device=dev) % d["ring"]
                snap[f"L{i}.k"], snap[f"L{i}.v"] = d["k"][slots].clone(), d["v"][slots].clone()
        for i, L in enumerate(dr.layers):
            snap[f"D{i}.k"], snap[f"D{i}.v"] = L["k"][:upto].clone(), L["v"][:upto].clone()
        return snap

    def run(native):
        for c in caches():
            c.zero_()
        torch.cuda.synchronize()
        if native:
            eng.open(prompt, 24, sp)
        else:
            eng.round.initialize(prompt, 24, sp, start_pos=0)
        torch.cuda.synchronize()
        snap = snapshot(n - 1)
        toks = []
        for rec in eng.stream_rounds():
            toks.extend(rec.tokens)
        return snap, toks

    ref, ref_toks = run(False)
    got, got_toks = run(True)
    info = dict(eng.last_prefill)
    got2, got2_toks = run(True)
    errs = {k: rel(got[k], ref[k]) for k in ref}
    out = {"world": world, "prefill": info, "moe": "ep" if eng.prefill.ep else ("local" if world == 1 else "tp"), "errs": {k: round(v, 5) for k, v in errs.items()},
           "bitwise": sorted(k for k in ref if torch.equal(got[k], ref[k])),
           "repeat_identical": all(torch.equal(got[k], got2[k]) for k in got) and got_toks == got2_toks,
           "repeat_diff": sorted(k for k in got if not torch.equal(got[k], got2[k])) + ([] if got_toks == got2_toks else ["tokens"]),
           "worst": max(errs.values()), "tokens_ref": ref_toks[:12], "tokens_native": got_toks[:12],
           "status": int(eng.fabric.status[0])}
    agree = 0
    for a, b in zip(ref_toks, got_toks):
        if a != b:
            break
        agree += 1
    out["token_prefix_agreement"] = agree
    if world > 1:
        allr = [None] * world
        dist.all_gather_object(allr, {"worst": out["worst"], "tokens": got_toks})
        out["worst"] = max(r["worst"] for r in allr)
        out["lockstep"] = all(r["tokens"] == allr[0]["tokens"] for r in allr)
    if rank == 0:
        print("RESULT " + json.dumps(out), flush=True)
    eng.fabric.check()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
