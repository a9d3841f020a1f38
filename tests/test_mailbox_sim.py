"""Fabric protocol on CPU threads: bit-exact all-reduce over several generations, a late peer, a
withheld publish that must time out with a status code (never hang), and failure propagation."""
import numpy as np

from naivert_b200.parallel.mailbox_sim import SITE_MAILBOX, SimFabric, all_reduce, run_ranks, _bf16_round


def _data(tp, rows, feats, seed):
    rng = np.random.default_rng(seed)
    parts = [rng.standard_normal((rows, feats)).astype(np.float32) for _ in range(tp)]
    resid = _bf16_round(rng.standard_normal((rows, feats)).astype(np.float32))
    return parts, resid


def test_all_reduce_bit_exact_over_generations_and_slabs():
    tp, rows, feats = 8, 8, 64
    fab = SimFabric(tp, feats)
    for gen in range(6):                                   # walks all four slabs and two epochs
        parts, resid = _data(tp, rows, feats, gen)
        if gen == 3:
            fab.epoch[:] += 1
        outs = run_ranks(tp, lambda r: all_reduce(fab, r, parts[r], resid, call=gen % 5))
        want = resid.copy()
        for s in range(tp):
            want = want + _bf16_round(parts[s])
        want = _bf16_round(want)
        for o in outs:
            assert o is not None and np.array_equal(o.view(np.uint32), want.view(np.uint32))
    assert not fab.status.any()


def test_late_peer_still_arrives():
    tp = 4
    fab = SimFabric(tp, 32)
    parts, resid = _data(tp, 3, 32, 1)
    outs = run_ranks(tp, lambda r: all_reduce(fab, r, parts[r], resid, 0, timeout_s=2.0, delay_s=0.2 if r == 2 else 0.0))
    assert all(o is not None for o in outs) and not fab.status.any()


def test_withheld_publish_times_out_with_site_code():
    tp = 4
    fab = SimFabric(tp, 32)
    parts, resid = _data(tp, 8, 32, 2)
    outs = run_ranks(tp, lambda r: all_reduce(fab, r, parts[r], resid, 0, timeout_s=0.2, publish=(r != 1)))
    assert outs[1] is not None                              # the silent rank received everything
    for r in (0, 2, 3):
        assert outs[r] is None and fab.status[r] == (SITE_MAILBOX | 1)
    # after a failure every later wait returns immediately instead of spinning
    import time
    t0 = time.monotonic()
    again = all_reduce(fab, 0, parts[0], resid, 1, timeout_s=5.0)
    assert again is None and time.monotonic() - t0 < 0.5


def test_stale_generation_is_never_mistaken():
    tp = 2
    fab = SimFabric(tp, 16)
    parts, resid = _data(tp, 2, 16, 3)
    run_ranks(tp, lambda r: all_reduce(fab, r, parts[r], resid, 0))
    fab.epoch[:] += 1                                       # same call index, next epoch: old words must not match
    outs = run_ranks(tp, lambda r: all_reduce(fab, r, parts[r], resid, 0, timeout_s=0.2, publish=(r == 0)))
    assert outs[0] is None and outs[1] is not None
