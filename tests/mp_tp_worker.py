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
    from naivert_b200.runtime.selfcheck import tp_selfcheck
    out = tp_selfcheck(rank, world, dist.group.WORLD, dev)
    out["verify_mean_rel"] = out["oracle_mean_rel"]
    if rank == 0:
        print("RESULT " + json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
