"""Worker of the tensor-parallel device-chain test (one process per GPU, launched by torchrun).

Every rank runs the self-relaunching round graph with a short record ring.  The last rank's host lags on
purpose, so its tail asks for a pause; the pause is a consensus over the ranks, hence every chain stops in the
same round and every host restarts it.  Checks: tokens equal those of host-launched rounds, identical on all
ranks, the chain was restarted at least once on every rank, clean fabric status.
"""
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from naivert_b200.models.naive_n0p5 import small_w8a8_spec
    from naivert_b200.models.spec import SamplingParams
    from naivert_b200.models.weights import (init_draft_state_dict, init_state_dict, prepare_draft_weights, prepare_weights,
                                             shard_draft_weights, shard_weights)
    from naivert_b200.runtime.engine import Engine

    spec = small_w8a8_spec(2)
    w = prepare_weights(spec, init_state_dict(spec, seed=0, device=dev))
    dw = prepare_draft_weights(spec, init_draft_state_dict(spec, seed=1, device=dev))
    kw = dict(rank=rank, tp=world, group=dist.group.WORLD, capacity=1024, device=dev,
              weights=shard_weights(spec, w, rank, world), draft_weights=shard_draft_weights(spec, dw, rank, world))
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, spec.vocab - 16, (41,), generator=g)
    sp = SamplingParams(temperature=0.6, seed=3)
    host = Engine.build(spec, **kw)
    want = host.generate(prompt, 200, sp).tokens
    host.close()
    dist.barrier()
    chain = Engine.build(spec, device_chain=True, ring_size=32, **kw)
    chain.round.nudge_s = 0.2
    out = {"world": world}
    try:
        chain.open(prompt, 200, sp)
        r = chain.round
        r.launch(1)
        got = []
        first = True
        while True:
            if first and rank == world - 1:
                time.sleep(1.0)                     # this host lags: its chain must pause, and so must the others
            first = False
            rec = r.wait_round(60.0)
            got.extend(rec.tokens)
            if rec.stop_reason is not None:
                break
        r.stream.synchronize()
        chain.fabric.check()
        gathered = [None] * world
        dist.all_gather_object(gathered, (got, r.host_launches), group=dist.group.WORLD)
        out["tokens_match_host_rounds"] = got == want
        out["lockstep"] = all(x[0] == gathered[0][0] for x in gathered)
        out["host_launches"] = [x[1] for x in gathered]
        out["status"] = int(chain.fabric.status[0])
    finally:
        chain.close()
    if rank == 0:
        print("RESULT " + json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
