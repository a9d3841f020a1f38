"""Child process of the index-checking test: loads the checking flavour of the kernel library (NAIVERT_BOUNDS_CHECK=1 is
set by the parent), decodes with a small model and prints what the bounds words recorded."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    from naivert_b200.models.naive_n0p5 import small_w8a8_spec
    from naivert_b200.models.spec import SamplingParams
    from naivert_b200.models.weights import (init_draft_state_dict, init_state_dict, prepare_draft_weights, prepare_weights,
                                             shard_draft_weights, shard_weights)
    from naivert_b200.ops import kernels as K
    from naivert_b200.runtime.engine import Engine
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    spec = small_w8a8_spec(4)
    w = prepare_weights(spec, init_state_dict(spec, seed=0, device="cpu"))
    dw = prepare_draft_weights(spec, init_draft_state_dict(spec, seed=1, device="cpu"))
    eng = Engine.build(spec, capacity=1024, device=dev, weights=shard_weights(spec, w, 0, 1),
                       draft_weights=shard_draft_weights(spec, dw, 0, 1))
    out = {"library": K.lib()._name.rsplit("/", 1)[-1]}
    eng.round.stop_ids.fill_(-1)                                            # no early stop: all 48 tokens are decoded
    try:
        g = torch.Generator().manual_seed(0)
        prompt = torch.randint(0, spec.vocab, (300,), generator=g)          # beyond the indexer's top-k: selected keys are used
        res = eng.generate(prompt, 48, SamplingParams(temperature=0.7, seed=3), use_graphs=False)
        eng.fabric.check()
        out["tokens"] = len(res.tokens)
        out["clean_run"] = K.bounds_violations()
        # a token id beyond the vocabulary: every build clamps it before the gather (no out-of-range access happens),
        # the checking build also records it
        bad = torch.tensor([3, spec.vocab + 5], dtype=torch.int32, device=dev)
        x = torch.zeros(16, spec.hidden, dtype=torch.bfloat16, device=dev)
        K.embed_rows(bad, eng.target.embed, x, 2, pdl=False)
        torch.cuda.synchronize()
        out["after_bad_token"] = K.bounds_violations()
        out["cleared"] = K.bounds_violations()
        out["row_is_last_table_row"] = bool(torch.equal(x[1], eng.target.embed[spec.vocab - 1]))
    finally:
        eng.close()
    print("BOUNDS " + json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
