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


def test_small_exchange_round_follows_the_call_plan_under_skew():
    """One round's small exchanges (Markov steps, sampler maxima / totals, four nucleus passes as reduce-scatter to the
    owning rank + digit broadcast, accept, draw, tail) run by eight skewed ranks in the order and with the call indices
    of ``runtime.modes.exchange_call_plan``: every rank ends with the same, correct values and nothing times out."""
    import time
    from naivert_b200.parallel.mailbox_sim import SimExchange, xchg_reduce, xchg_reduce_scatter
    from naivert_b200.runtime.modes import exchange_call_plan
    tp, groups, gsize = 8, 15, 32
    x = SimExchange(tp)
    plan = exchange_call_plan()
    rng = np.random.default_rng(0)
    hist = rng.integers(0, 1 << 40, size=(4, tp, groups * gsize), dtype=np.uint64)
    small = rng.integers(0, 1 << 30, size=(len(plan), tp, 16), dtype=np.uint64)
    want_hist = hist.sum(1, dtype=np.uint64)

    def rank_body(r):
        lrng = np.random.default_rng(100 + r)
        seen = []
        for i, (name, call) in enumerate(plan):
            if lrng.random() < 0.3:
                time.sleep(float(lrng.random()) * 2e-3)                   # skew between ranks, different every call
            if "bins_to_owner" in name:
                p = int(name[len("sampler.nucleus")])
                out = xchg_reduce_scatter(x, r, hist[p, r], groups, gsize, (1 << groups) - 1, call)
                assert out is not None, name
                for g in range(groups):
                    sl = slice(g * gsize, (g + 1) * gsize)
                    want = want_hist[p, sl] if g % tp == r else hist[p, r, sl]
                    assert np.array_equal(out[sl], want), (name, g)
            else:
                out = xchg_reduce(x, r, small[i, r], call, op="max" if name.startswith("markov") else "sum")
                assert out is not None, name
                seen.append(out)
        return seen

    outs = run_ranks(tp, rank_body)
    assert not x.status.any()
    for r in range(1, tp):
        for a, b in zip(outs[0], outs[r]):
            assert np.array_equal(a, b)


def test_consecutive_calls_in_one_slab_can_lose_words():
    """Why the plan keeps consecutive calls in different slabs: a fast rank that has finished call n (a reduce-scatter it
    owns nothing of) pushes call n + 1 over the words a slow owner has not read yet."""
    import time
    from naivert_b200.parallel.mailbox_sim import SITE_RENDEZVOUS, SimExchange, xchg_reduce, xchg_reduce_scatter
    tp, gsize = 2, 8
    x = SimExchange(tp)
    vals = [np.arange(gsize, dtype=np.uint64) + 10 * r for r in range(tp)]

    def body(r):
        if r == 0:                                   # owner of group 0, late
            time.sleep(0.2)
            return xchg_reduce_scatter(x, 0, vals[0], 1, gsize, 1, call=2, timeout_s=0.3)
        xchg_reduce_scatter(x, 1, vals[1], 1, gsize, 1, call=2)          # pushes to rank 0, owns nothing, returns
        return xchg_reduce(x, 1, vals[1], call=6, timeout_s=0.3)         # same slab (6 % 4 == 2), same value indices
    outs = run_ranks(tp, body)
    assert outs[0] is None and x.status[0] == (SITE_RENDEZVOUS | 2)      # the owner never sees call 2's words
    # with the next call in another slab nothing is lost
    x = SimExchange(tp)

    def body_ok(r):
        if r == 0:
            time.sleep(0.2)
            a = xchg_reduce_scatter(x, 0, vals[0], 1, gsize, 1, call=2, timeout_s=1.0)
            b = xchg_reduce(x, 0, vals[0], call=3, timeout_s=1.0)
            return a, b
        a = xchg_reduce_scatter(x, 1, vals[1], 1, gsize, 1, call=2)
        b = xchg_reduce(x, 1, vals[1], call=3, timeout_s=1.0)
        return a, b
    outs = run_ranks(tp, body_ok)
    assert np.array_equal(outs[0][0], vals[0] + vals[1]) and np.array_equal(outs[0][1], outs[1][1]) and not x.status.any()
