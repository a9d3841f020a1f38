"""Tensor-parallel self-check on a small W8A8 geometry: the same kernels and code paths as the full model at
dimensions where the torch oracle is cheap.  One call per rank (collective); used by the multi-GPU test worker
and by the benchmark, which prints the result beside its timing so a scaling run also carries a correctness
record for its TP degree.

Checks: one verify step against the oracle evaluated with the same rank-partial rounding, tensor-parallel
arg-max, bitwise-identical residual streams on all ranks, run-to-run determinism, lockstep (identical tokens on
every rank), speculative == greedy, and a clean fabric status.

Parity: the reference's verify / round gates (tests/gpu/naive_n0p5_e2e/run_naive_n0p5_verify.py:513-613,
tests/gpu/naive_n0p5_draft/round/run.py) compare the same quantities on its 8-GPU box.
"""
from __future__ import annotations

import torch


def _sampler_check(eng, spec, rank: int, world: int, device) -> bool:
    """The sharded sampler on identical full-vocabulary logits (every rank draws the same tensors and keeps its
    vocabulary slice) against the integer oracle, which knows nothing about shards: equal results for every TP
    degree means the sampler is invariant under the sharding."""
    from ..models.spec import SamplingParams
    from ..ops import kernels as K
    from ..ops import sampling_ref as S
    r = eng.round
    V, vl = spec.vocab, spec.vocab // world
    g = torch.Generator(device=device).manual_seed(3)
    ok = True
    for trial, (top_p, forced, temp) in enumerate([(0.95, None, 1.0), (0.5, None, 0.4), (0.95, 0.7, 0.4)]):
        zp = torch.randn(8, V, device=device, generator=g) * 3
        zq = zp[:7] + torch.randn(7, V, device=device, generator=g)
        r.t.logits[:8].copy_(zp[:, rank * vl:(rank + 1) * vl])
        r.draft.zq[:7].copy_(zq[:, rank * vl:(rank + 1) * vl])
        ids = [11] + [int(torch.multinomial(torch.softmax(zq[j] / temp, -1), 1, generator=g)) for j in range(7)]
        r.block_ids[:8].copy_(torch.tensor(ids, dtype=torch.int32))
        sp = SamplingParams(temperature=temp, top_p=top_p, seed=77 + trial, forced_accept_p=forced)
        r.set_sampling(sp)
        r.t.ctrl[8] = trial
        r.sample()
        K.epoch_advance(eng.fabric.epoch, pdl=False)
        torch.cuda.synchronize()
        st = r.state.view(torch.int32)
        tail = (K.sampler_state_bytes() - 10 * 4) // 4
        accepted, extra = int(st[tail + 0]), int(st[tail + 1])
        m, tok, _, _ = S.verify_oracle(zp, zq, ids, 1.0 / temp, sp.clamped_top_p(), sp.seed, trial, forced=forced)
        ok = ok and accepted == m and extra == tok
    r.t.ctrl[8] = 0
    return ok


def tp_selfcheck(rank: int, world: int, group, device, layers: int = 4, generate: bool = True) -> dict:
    import torch.distributed as dist
    from ..models.naive_n0p5 import small_w8a8_spec
    from ..models.reference import ReferenceModel
    from ..models.spec import SamplingParams
    from ..models.weights import (init_draft_state_dict, init_state_dict, prepare_draft_weights, prepare_weights,
                                  shard_draft_weights, shard_weights)
    from ..ops import kernels as K
    from .engine import Engine

    spec = small_w8a8_spec(max(layers, world))              # one draft feature tap per layer: their count must split over the ranks
    w = prepare_weights(spec, init_state_dict(spec, seed=0, device=device))
    dw = prepare_draft_weights(spec, init_draft_state_dict(spec, seed=1, device=device))
    eng = Engine.build(spec, rank=rank, tp=world, group=group, capacity=1024, device=device,
                       weights=shard_weights(spec, w, rank, world), draft_weights=shard_draft_weights(spec, dw, rank, world))
    out = {"world": world, "geometry": spec.name}
    try:
        g = torch.Generator().manual_seed(0)
        toks = torch.randint(0, spec.vocab, (16,), generator=g)
        ref = ReferenceModel(spec, w, tp=world, capacity=64, device=device)
        t = eng.target
        errs = []
        for i in range(2):
            t.set_inputs(toks[i * 8:(i + 1) * 8], i * 8)
            t.step()
            K.epoch_advance(eng.fabric.epoch, pdl=False)
            torch.cuda.synchronize()
            want = ref.step(toks[i * 8:(i + 1) * 8].to(device), i * 8)
            V = spec.vocab // world
            got = t.logits[:8].float()
            wl = want[:, rank * V:(rank + 1) * V]
            errs.append(((got - wl).abs().mean() / wl.abs().mean()).item())
        eng.fabric.check()
        out["oracle_mean_rel"] = round(max(errs), 5)
        tok = t.greedy_argmax()
        K.epoch_advance(eng.fabric.epoch, pdl=False)
        torch.cuda.synchronize()
        if world > 1:
            full = [torch.zeros_like(t.logits[:8]) for _ in range(world)]
            dist.all_gather(full, t.logits[:8].contiguous(), group=group)
            out["argmax_ok"] = tok[:8].tolist() == torch.cat(full, dim=1).argmax(-1).tolist()
            xs = [torch.zeros_like(t.x) for _ in range(world)]
            dist.all_gather(xs, t.x, group=group)
            out["residual_identical"] = all(torch.equal(xs[0], x) for x in xs)
        else:
            out["argmax_ok"] = tok[:8].tolist() == t.logits[:8].argmax(-1).tolist()
            out["residual_identical"] = True
        out["sampler_matches_oracle"] = _sampler_check(eng, spec, rank, world, device)
        if generate:
            prompt = torch.randint(0, spec.vocab - 16, (45,), generator=g)
            sp = SamplingParams(temperature=0.4, seed=5, forced_accept_p=0.7)
            a = eng.generate(prompt, 64, sp)
            b = eng.generate(prompt, 64, sp)
            out["deterministic"] = a.tokens == b.tokens
            if world > 1:
                gathered = [None] * world
                dist.all_gather_object(gathered, a.tokens, group=group)
                out["lockstep"] = all(x == gathered[0] for x in gathered)
            else:
                out["lockstep"] = True
            greedy = eng.generate(prompt, 32, SamplingParams(top_p=1e-6, seed=9, forced_accept_p=0.0))
            specd = eng.generate(prompt, 32, SamplingParams(top_p=1e-6, seed=9))
            out["spec_equals_greedy"] = greedy.tokens == specd.tokens
            real = eng.generate(prompt, 64, SamplingParams(temperature=0.8, seed=11))
            out["real_sampling_tokens"] = len(real.tokens)
            out["acceptance"] = round(real.acceptance, 4)
        eng.fabric.check()
        out["status"] = int(eng.fabric.status[0])
    finally:
        eng.close()
    return out
