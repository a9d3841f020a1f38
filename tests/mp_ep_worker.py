"""Worker of the expert-parallel all-to-all test (torchrun, one process per GPU; also runs at world 1)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from naivert_b200.ops.quant import quantize_act_pow2, quantize_fp8_block, w8a8_linear_ref
    from naivert_b200.parallel.fabric import Fabric
    from naivert_b200.prefill.ep_moe import EPMoE, ep_layout_reference
    H, I, E, Kk, T = 1024, 512, 16, 4, 96
    El = E // world
    g = torch.Generator(device=dev).manual_seed(5)          # same on every rank: the full model
    gate = torch.randn(E, I, H, device=dev, generator=g) * 0.05
    up = torch.randn(E, I, H, device=dev, generator=g) * 0.05
    down = torch.randn(E, H, I, device=dev, generator=g) * 0.05
    gamma = (1 + 0.05 * torch.randn(H, device=dev, generator=g)).bfloat16()
    g8, gs = quantize_fp8_block(gate); u8, us = quantize_fp8_block(up); d8, ds = quantize_fp8_block(down)
    x_all = torch.randn(world, T, H, device=dev, generator=g).bfloat16()
    scores = torch.rand(world, T, E, device=dev, generator=g)
    scores[:, :, 3] += 0.5                                   # skewed routing: expert 3 is popular
    p_all, ids_all = torch.topk(scores, Kk, dim=-1)
    p_all = (p_all / p_all.sum(-1, keepdim=True)).float()
    sl = slice(rank * El, (rank + 1) * El)
    fab = Fabric(rank, world, H, group=dist.group.WORLD if world > 1 else None, device=dev)
    moe = EPMoE(fab, H, I, E, Kk, T, {"w": g8[sl], "s": gs[sl]}, {"w": u8[sl], "s": us[sl]}, {"w": d8[sl], "s": ds[sl]})
    # the same layer on the 64-column chunk engine (segments padded to 64 rows)
    moe64 = EPMoE(fab, H, I, E, Kk, T, {"w": g8[sl], "s": gs[sl]}, {"w": u8[sl], "s": us[sl]}, {"w": d8[sl], "s": ds[sl]},
                  item_rows=64)
    x, ids, probs = x_all[rank].contiguous(), ids_all[rank].int().contiguous(), p_all[rank].contiguous()
    out = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
    outs = []
    for it in range(2):                                      # twice: buffers and tags are reused across layers
        out.zero_()
        moe.run(x, gamma, ids, probs, x, out)
        torch.cuda.synchronize()
        outs.append(out.clone())
    out.zero_()
    moe64.run(x, gamma, ids, probs, x, out)
    torch.cuda.synchronize()
    out64 = out.clone()
    fab.check()
    # device layout (segments, work list, destination rows) against its host restatement
    lay = ep_layout_reference([ids_all[s].int().cpu() for s in range(world)], E, 16)
    n_it = int(moe.n_items)
    layout_ok = (moe.seg_rows.tolist() == lay["seg_rows"][rank]
                 and list(zip(moe.item_expert[:n_it].tolist(), moe.item_row[:n_it].tolist())) == lay["items"][rank]
                 and moe.slot_of.tolist() == lay["slot"][rank].flatten().tolist())
    # torch reference of this rank's tokens
    xf = x.float()
    xn = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma.float()).bfloat16().float()
    ref = x.float().clone()
    for k in range(Kk):
        for e in ids[:, k].unique().tolist():
            rows = (ids[:, k] == e).nonzero().flatten()
            gg = w8a8_linear_ref(xn[rows], g8[e], gs[e]); uu = w8a8_linear_ref(xn[rows], u8[e], us[e])
            y = torch.nn.functional.silu(gg) * uu
            dd = w8a8_linear_ref(y, d8[e], ds[e]).bfloat16().float()
            ref[rows] += probs[rows, k, None] * dd
    ref = ref.bfloat16().float()
    err = ((outs[1].float() - ref).abs().max() / ref.abs().max()).item()
    err0 = ((outs[0].float() - ref).abs().max() / ref.abs().max()).item()
    dd = (outs[0].float() - outs[1].float()).abs()
    res = {"world": world, "max_rel_err": err, "first_err": err0, "diff_rows": dd.amax(-1).nonzero().flatten().tolist()[:12],
           "diff_max": dd.max().item(), "repeat_identical": bool(torch.equal(outs[0], outs[1])),
           "items": int(moe.n_items), "rows": int(moe.seg_rows.sum()), "status": int(fab.status[0]),
           "layout_ok": bool(layout_ok), "wide_identical": bool(torch.equal(out64, outs[1])), "wide_items": int(moe64.n_items),
           "wide_err": ((out64.float() - ref).abs().max() / ref.abs().max()).item()}
    if world > 1:
        allr = [None] * world
        dist.all_gather_object(allr, res)
        res["worst_err"] = max(max(r["max_rel_err"], r["wide_err"]) for r in allr)
        res["wide_identical"] = all(r["wide_identical"] for r in allr)
        res["layout_ok"] = all(r["layout_ok"] for r in allr)
        res["total_rows"] = sum(r["rows"] for r in allr)
    if rank == 0:
        print("RESULT " + json.dumps(res), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
