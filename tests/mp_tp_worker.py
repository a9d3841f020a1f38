"""Worker of the multi-GPU tensor-parallel test (one process per GPU, launched by torchrun).

Checks, at tp = WORLD_SIZE on the small W8A8 geometry sharded from one logical checkpoint:
one verify step against the torch oracle evaluated with the same tp (rank-partial rounding),
lockstep (identical tokens on every rank), run-to-run bitwise determinism, speculative ==
greedy, and a clean fabric status.  Prints one JSON line from rank 0.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from naivert_b200.models.naive_n0p5 import small_w8a8_spec
    from naivert_b200.models.reference import ReferenceModel
    from naivert_b200.models.spec import SamplingParams
    from naivert_b200.models.weights import (init_draft_state_dict, init_state_dict, prepare_draft_weights,
                                             prepare_weights, shard_draft_weights, shard_weights)
    from naivert_b200.runtime.engine import Engine

    spec = small_w8a8_spec(4)
    w = prepare_weights(spec, init_state_dict(spec, seed=0, device=dev))
    dw = prepare_draft_weights(spec, init_draft_state_dict(spec, seed=1, device=dev))
    eng = Engine.build(spec, rank=rank, tp=world, group=dist.group.WORLD, capacity=1024, device=dev,
                       weights=shard_weights(spec, w, rank, world), draft_weights=shard_draft_weights(spec, dw, rank, world))
    out = {"world": world}

    # ---- one verify step vs the oracle with the same rank-partial rounding
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, spec.vocab, (16,), generator=g)
    ref = ReferenceModel(spec, w, tp=world, capacity=64, device=dev)
    t = eng.target
    from naivert_b200.ops import kernels as K
    errs = []
    for i in range(2):
        t.set_inputs(toks[i * 8:(i + 1) * 8], i * 8)
        t.step()
        K.epoch_advance(eng.fabric.epoch, pdl=False)
        torch.cuda.synchronize()
        want = ref.step(toks[i * 8:(i + 1) * 8].to(dev), i * 8)
        V = spec.vocab // world
        got = t.logits[:8].float()
        wl = want[:, rank * V:(rank + 1) * V]
        errs.append(((got - wl).abs().mean() / wl.abs().mean()).item())
    eng.fabric.check()
    out["verify_mean_rel"] = max(errs)
    # tensor-parallel arg-max of the last step's logits vs the gathered full-vocabulary logits
    tok = t.greedy_argmax()
    K.epoch_advance(eng.fabric.epoch, pdl=False)
    torch.cuda.synchronize()
    full = [torch.zeros_like(t.logits[:8]) for _ in range(world)]
    dist.all_gather(full, t.logits[:8].contiguous())
    out["argmax_ok"] = tok[:8].tolist() == torch.cat(full, dim=1).argmax(-1).tolist()
    # residual stream must be bitwise identical on all ranks (same partials, same order)
    xs = [torch.zeros_like(t.x) for _ in range(world)]
    dist.all_gather(xs, t.x)
    out["residual_identical"] = all(torch.equal(xs[0], x) for x in xs)

    # ---- generation: lockstep, determinism, speculative == greedy
    prompt = torch.randint(0, spec.vocab - 16, (45,), generator=g)
    sp = SamplingParams(temperature=0.4, seed=5, forced_accept_p=0.7)
    a = eng.generate(prompt, 64, sp)
    b = eng.generate(prompt, 64, sp)
    out["deterministic"] = a.tokens == b.tokens
    gathered = [None] * world
    dist.all_gather_object(gathered, a.tokens)
    out["lockstep"] = all(x == gathered[0] for x in gathered)
    greedy = eng.generate(prompt, 32, SamplingParams(top_p=1e-6, seed=9, forced_accept_p=0.0))
    specd = eng.generate(prompt, 32, SamplingParams(top_p=1e-6, seed=9))
    out["spec_equals_greedy"] = greedy.tokens == specd.tokens
    real = eng.generate(prompt, 64, SamplingParams(temperature=0.8, seed=11))
    out["real_sampling_tokens"] = len(real.tokens)
    out["acceptance"] = real.acceptance
    eng.fabric.check()
    out["status"] = int(eng.fabric.status[0])
    if rank == 0:
        print("RESULT " + json.dumps(out), flush=True)
    eng.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
