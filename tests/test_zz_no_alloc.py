"""The allocation-free routing entry point (``nrt_router_route_noalloc``) against the regular
router entry point.

Some callers cannot allocate device memory where they need a routing decision (hosts that own all
device memory through their own pools, latency-critical paths that must not hit cudaMalloc's
device-wide synchronisation).  For them the library keeps the router's scratch - score matrix and
arrival counter - in a fixed device array of its own; this test calls that entry through its exported
C symbol twice in a row, with different inputs, and requires the same routing as the regular entry
point that is given caller-allocated scratch.  It is collected last so that a failure here cannot hide
the result of any other test."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular(K, xn, w, bias, rows, top_k, experts, max_slots):
    dev = xn.device
    out = dict(n_active=torch.zeros(1, dtype=torch.int32, device=dev), active_ids=torch.full((max_slots,), -1, dtype=torch.int32, device=dev),
               probs=torch.zeros(max_slots, 16, device=dev), topk_ids=torch.zeros(16, top_k, dtype=torch.int32, device=dev),
               topk_p=torch.zeros(16, top_k, device=dev))
    scores = torch.zeros(16, experts, device=dev)
    ticket = torch.zeros(1, dtype=torch.int32, device=dev)
    a = K.RouterArgs()
    a.xn, a.w, a.bias = xn.data_ptr(), w.data_ptr(), bias.data_ptr()
    a.hidden, a.experts, a.rows, a.top_k = xn.shape[1], experts, rows, top_k
    a.sigmoid, a.normalize, a.route_scale = 1, 1, 1.0
    a.scores, a.ticket = scores.data_ptr(), ticket.data_ptr()
    a.n_active, a.active_ids, a.probs = out["n_active"].data_ptr(), out["active_ids"].data_ptr(), out["probs"].data_ptr()
    a.topk_ids, a.topk_p, a.max_slots = out["topk_ids"].data_ptr(), out["topk_p"].data_ptr(), max_slots
    K.router(a, pdl=False)
    torch.cuda.synchronize()
    return out


def _noalloc(lib, xn, w, bias, rows, top_k, experts, max_slots):
    dev = xn.device
    out = dict(n_active=torch.zeros(1, dtype=torch.int32, device=dev), active_ids=torch.full((max_slots,), -1, dtype=torch.int32, device=dev),
               probs=torch.zeros(max_slots, 16, device=dev), topk_ids=torch.zeros(16, top_k, dtype=torch.int32, device=dev),
               topk_p=torch.zeros(16, top_k, device=dev))
    fn = lib.nrt_router_route_noalloc
    fn.restype = C.c_int
    vp = C.c_void_p
    rc = fn(vp(xn.data_ptr()), vp(w.data_ptr()), vp(bias.data_ptr()), C.c_int(xn.shape[1]), C.c_int(experts), C.c_int(rows),
            C.c_int(top_k), C.c_int(1), C.c_int(1), C.c_float(1.0), vp(out["n_active"].data_ptr()), vp(out["active_ids"].data_ptr()),
            vp(out["probs"].data_ptr()), vp(out["topk_ids"].data_ptr()), vp(out["topk_p"].data_ptr()), C.c_int(max_slots),
            vp(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, rc
    torch.cuda.synchronize()
    return out


def test_no_alloc_router_matches_regular_entry_twice():
    from naivert_b200.ops import kernels as K
    lib = K.lib()
    g = torch.Generator(device="cuda").manual_seed(11)
    hidden, experts, top_k, max_slots = 1024, 64, 8, 64
    for call, rows in enumerate((8, 5)):                    # two calls in a row, different inputs and row counts
        xn = torch.randn(16, hidden, device="cuda", generator=g).bfloat16()
        w = torch.randn(experts, hidden, device="cuda", generator=g) * 0.03
        bias = torch.randn(experts, device="cuda", generator=g) * 0.05
        want = _regular(K, xn, w, bias, rows, top_k, experts, max_slots)
        got = _noalloc(lib, xn, w, bias, rows, top_k, experts, max_slots)
        assert int(got["n_active"]) == int(want["n_active"]) > 0, call
        n = int(want["n_active"])
        assert torch.equal(got["active_ids"][:n], want["active_ids"][:n])
        assert torch.equal(got["topk_ids"][:rows], want["topk_ids"][:rows])
        assert torch.allclose(got["topk_p"][:rows], want["topk_p"][:rows], rtol=1e-6, atol=1e-7)
        assert torch.allclose(got["probs"][:n], want["probs"][:n], rtol=1e-6, atol=1e-7)


def test_no_alloc_router_rejects_oversize():
    from naivert_b200.ops import kernels as K
    lib = K.lib()
    fn = lib.nrt_router_route_noalloc
    fn.restype = C.c_int
    t = torch.zeros(64, device="cuda")
    vp = C.c_void_p
    args = lambda experts, rows: (vp(t.data_ptr()), vp(t.data_ptr()), vp(None), C.c_int(1024), C.c_int(experts), C.c_int(rows), C.c_int(8),
                                  C.c_int(1), C.c_int(1), C.c_float(1.0), vp(t.data_ptr()), vp(t.data_ptr()), vp(t.data_ptr()),
                                  vp(t.data_ptr()), vp(t.data_ptr()), C.c_int(64), vp(None))
    assert fn(*args(1024, 8)) == -10            # experts beyond the compiled-in scratch
    assert fn(*args(64, 17)) == -10             # rows beyond the maximum
    torch.cuda.synchronize()
