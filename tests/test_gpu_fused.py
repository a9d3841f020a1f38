"""Fused forms of the step kernels against plain torch fp32 references of the same ops (single GPU):
RMSNorm folded into the GEMM's operand build, q/k/v post-processing in the projection epilogue, the
per-tile sums of squares left by the all-reduce epilogue, the router with the norm applied on the fly,
and the whole fused step against the step built from separate kernels."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _K():
    from naivert_b200.ops import kernels as K
    K.lib()
    return K


def _ssq(x):
    """[16, H] bf16 -> [H/128, 16] fp32 sums of squares per 128-feature tile."""
    r, h = x.shape
    return x.float().pow(2).view(r, h // 128, 128).sum(-1).t().contiguous()


def _rmsnorm_ref(x, gamma, eps):
    xf = x.float()
    rs = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * rs * gamma.float()).bfloat16()


@pytest.mark.parametrize("rows,n,k,split", [(8, 512, 1024, 1), (8, 256, 4096, 4), (3, 384, 2048, 2)])
def test_norm_operand_bf16_matches_torch(rows, n, k, split):
    K = _K()
    g = torch.Generator(device="cuda").manual_seed(11)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).bfloat16()
    x = torch.zeros(16, k, device="cuda", dtype=torch.bfloat16)
    x[:rows] = (torch.randn(rows, k, device="cuda", generator=g) * 3).bfloat16()
    gamma = (1 + 0.1 * torch.randn(k, device="cuda", generator=g)).bfloat16()
    ssq = _ssq(x)
    out = torch.zeros(rows, n, device="cuda")
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    a = K.GemmArgs()
    a.n_total, a.k_total, a.rows = n, k, rows
    a.out_f32, a.ld_out, a.out_scale = out.data_ptr(), n, 1.0
    a.nx, a.ngamma, a.nssq, a.neps = x.data_ptr(), gamma.data_ptr(), ssq.data_ptr(), 1e-5
    a.status = st.data_ptr()
    K.gemm(K.gemm_variant(False, False, K.EPI_STORE_F32, K.GROUP_NONE, K.B_NORM), K.weight_tmap(w), None, None, a,
           n // 128, split, pdl=False)
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    ref = _rmsnorm_ref(x[:rows], gamma, 1e-5).float() @ w.float().T
    assert (out - ref).abs().max().item() <= 4e-3 * ref.abs().max().item()


def test_norm_operand_fp8_gate_up_matches_torch():
    """RMSNorm + e4m3 packet built inside the dual gate/up GEMM: silu(gate) * up, re-quantised."""
    K = _K()
    from naivert_b200.ops.quant import quantize_act_pow2, quantize_fp8_block, w8a8_linear_ref
    g = torch.Generator(device="cuda").manual_seed(12)
    rows, n, k = 8, 256, 2048
    g8, gs = quantize_fp8_block(torch.randn(n, k, device="cuda", generator=g) * 0.05)
    u8, us = quantize_fp8_block(torch.randn(n, k, device="cuda", generator=g) * 0.05)
    x = torch.zeros(16, k, device="cuda", dtype=torch.bfloat16)
    x[:rows] = (torch.randn(rows, k, device="cuda", generator=g) * 2).bfloat16()
    gamma = (1 + 0.1 * torch.randn(k, device="cuda", generator=g)).bfloat16()
    ssq = _ssq(x)
    y8 = torch.zeros(16, n, dtype=torch.uint8, device="cuda")
    ys = torch.ones(16, n // 128, device="cuda")
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    a = K.GemmArgs()
    a.n_total, a.k_total, a.rows = n, k, rows
    a.w_scale0, a.w_scale1 = gs.data_ptr(), us.data_ptr()
    a.out_q, a.out_qscale = y8.data_ptr(), ys.data_ptr()
    a.nx, a.ngamma, a.nssq, a.neps = x.data_ptr(), gamma.data_ptr(), ssq.data_ptr(), 1e-5
    a.status = st.data_ptr()
    K.gemm(K.gemm_variant(True, True, K.EPI_SILU_QUANT, K.GROUP_NONE, K.B_NORM), K.weight_tmap(g8.view(torch.uint8)),
           K.weight_tmap(u8.view(torch.uint8)), None, a, n // 128, 1, pdl=False)
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    xn = _rmsnorm_ref(x[:rows], gamma, 1e-5).float()
    ref = torch.nn.functional.silu(w8a8_linear_ref(xn, g8, gs)) * w8a8_linear_ref(xn, u8, us)
    got = y8[:rows].view(torch.float8_e4m3fn).float().view(rows, n // 128, 128) * ys[:rows].unsqueeze(-1)
    got = got.view(rows, n)
    # e4m3 keeps 3 mantissa bits: half an ulp is 1/16 of the value, plus the block scale's granularity
    tol = ref.abs().view(rows, n // 128, 128).amax(-1, keepdim=True).expand(rows, n // 128, 128).reshape(rows, n) / 16
    assert ((got - ref).abs() <= tol + 1e-6).float().mean().item() > 0.995


def test_allreduce_epilogue_leaves_sums_of_squares():
    K = _K()
    from naivert_b200.ops.quant import quantize_act_pow2, quantize_fp8_block
    g = torch.Generator(device="cuda").manual_seed(13)
    rows, n, k = 8, 1024, 512
    w8, ws = quantize_fp8_block(torch.randn(n, k, device="cuda", generator=g) * 0.05)
    xq, xsc = quantize_act_pow2(torch.randn(rows, k, device="cuda", generator=g).bfloat16().float())
    x8 = torch.zeros(16, k, dtype=torch.uint8, device="cuda")
    xs = torch.ones(16, k // 128, device="cuda")
    x8[:rows], xs[:rows] = xq.view(torch.uint8), xsc
    resid = torch.randn(rows, n, device="cuda", generator=g).bfloat16()
    out = torch.zeros(rows, n, device="cuda", dtype=torch.bfloat16)
    ssq = torch.full((n // 128, 16), -1.0, device="cuda")
    st, epoch = torch.zeros(4, dtype=torch.int32, device="cuda"), torch.ones(1, dtype=torch.int32, device="cuda")
    a = K.GemmArgs()
    a.n_total, a.k_total, a.rows = n, k, rows
    a.w_scale0, a.a_scale = ws.data_ptr(), xs.data_ptr()
    a.out_bf16, a.ld_out, a.resid, a.ssq_out = out.data_ptr(), n, resid.data_ptr(), ssq.data_ptr()
    a.fab.epoch, a.fab.status, a.fab.tp, a.fab.features, a.fab.timeout_ns = epoch.data_ptr(), st.data_ptr(), 1, n, 10 ** 9
    a.fab.ag_call = -1
    a.status = st.data_ptr()
    for split in (1, 4):
        ssq.fill_(-1.0)
        K.gemm(K.gemm_variant(True, False, K.EPI_ALLREDUCE, K.GROUP_NONE), K.weight_tmap(w8.view(torch.uint8)), None,
               K.act_tmap(x8), a, n // 128, split, pdl=False)
        torch.cuda.synchronize()
        assert int(st[0]) == 0
        want = out.float().pow(2).view(rows, n // 128, 128).sum(-1).t()
        assert torch.allclose(ssq[:, :rows], want, rtol=1e-5, atol=1e-6), split
        assert (ssq[:, rows:] == 0).all()


def test_router_inline_norm_matches_torch():
    """scores = rmsnorm(x) @ W^T in fp32, sigmoid + bias for the choice, top-k with lowest-index ties,
    probabilities normalised over the chosen experts: at the full model's routing dimensions."""
    K = _K()
    g = torch.Generator(device="cuda").manual_seed(14)
    H, E, rows, top_k = 4096, 256, 8, 8
    x = torch.zeros(16, H, device="cuda", dtype=torch.bfloat16)
    x[:rows] = (torch.randn(rows, H, device="cuda", generator=g) * 2).bfloat16()
    gamma = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).bfloat16()
    w = (torch.randn(E, H, device="cuda", generator=g) * 0.05).contiguous()
    bias = (torch.randn(E, device="cuda", generator=g) * 0.1).contiguous()
    ssq = _ssq(x)
    scores = torch.zeros(16, E, device="cuda")
    ticket = torch.zeros(1, dtype=torch.int32, device="cuda")
    n_active = torch.zeros(1, dtype=torch.int32, device="cuda")
    active = torch.zeros(128, dtype=torch.int32, device="cuda")
    probs = torch.zeros(128, 16, device="cuda")
    ids = torch.zeros(16, top_k, dtype=torch.int32, device="cuda")
    tp = torch.zeros(16, top_k, device="cuda")
    r = K.RouterArgs()
    r.x, r.gamma, r.eps, r.ssq = x.data_ptr(), gamma.data_ptr(), 1e-5, ssq.data_ptr()
    r.w, r.bias, r.hidden, r.experts, r.rows, r.top_k = w.data_ptr(), bias.data_ptr(), H, E, rows, top_k
    r.sigmoid, r.normalize, r.route_scale = 1, 1, 1.0
    r.scores, r.ticket, r.n_active, r.active_ids, r.probs = (scores.data_ptr(), ticket.data_ptr(), n_active.data_ptr(),
                                                            active.data_ptr(), probs.data_ptr())
    r.topk_ids, r.topk_p, r.max_slots = ids.data_ptr(), tp.data_ptr(), 128
    K.router(r, pdl=False)
    torch.cuda.synchronize()
    xn = _rmsnorm_ref(x[:rows], gamma, 1e-5).float()
    sc = xn.double() @ w.double().T
    assert (scores[:rows].double() - sc).abs().max().item() < 2e-4 * sc.abs().max().item()
    sig = torch.sigmoid(scores[:rows].double())            # the choice is made on the kernel's own fp32 scores
    choice = sig + bias.double()
    for row in range(rows):
        order = sorted(range(E), key=lambda e: (-choice[row, e].item(), e))[:top_k]
        assert ids[row].tolist() == order
        p = sig[row, order] / (sig[row, order].sum() + 1e-20)
        assert torch.allclose(tp[row].double(), p, rtol=1e-5, atol=1e-7)
    want_active = sorted(set(ids[:rows].flatten().tolist()))
    assert int(n_active) == len(want_active) and active[: len(want_active)].tolist() == want_active
    for s_, e in enumerate(want_active):
        for row in range(rows):
            exp = tp[row][ids[row] == e].sum().item()
            assert abs(probs[s_, row].item() - exp) < 1e-7


def _two_runtimes(layers=4, capacity=512):
    from naivert_b200.models.naive_n0p5 import small_w8a8_spec
    from naivert_b200.models.weights import init_state_dict, prepare_weights, shard_weights
    from naivert_b200.runtime.target import LocalFabric, TargetRuntime
    spec = small_w8a8_spec(layers)
    w = prepare_weights(spec, init_state_dict(spec, seed=0, device="cuda"))
    out = []
    for legacy in ("0", "1"):
        os.environ["NAIVERT_LEGACY_STEP"] = legacy
        try:
            out.append(TargetRuntime(spec, shard_weights(spec, w, 0, 1), LocalFabric("cuda"), rows=8, capacity=capacity))
        finally:
            os.environ.pop("NAIVERT_LEGACY_STEP", None)
    return spec, out[0], out[1]


def test_fused_step_matches_separate_kernels():
    """Same weights, same tokens: the fused step (norm in the operand build, post-processing in the epilogue,
    tensor-core attention) against the step of separate kernels.  The first layer's caches depend only on the
    embedding, the norm and the projection: keys and values must agree bit for bit, the indexer keys up to the
    last bit of their per-row scale.  Deeper layers see the bf16 probabilities of the tensor-core attention and the
    last-bit differences of the sums of squares, which can flip an e4m3 code or an expert choice now and then:
    they are compared in the mean."""
    spec, fused, legacy = _two_runtimes()
    assert fused.fused and not legacy.fused
    g = torch.Generator().manual_seed(3)
    steps = 36                                          # crosses the indexer's top-k boundary (256 positions)
    toks = torch.randint(0, spec.vocab, (steps * 8,), generator=g)
    worst = 0.0
    for i in range(steps):
        for rt in (fused, legacy):
            rt.set_inputs(toks[i * 8:(i + 1) * 8], i * 8)
            rt.step()
        torch.cuda.synchronize()
        fused.fab.check()
        a, b = fused.logits[:8].float(), legacy.logits[:8].float()
        assert torch.isfinite(a).all()
        worst = max(worst, ((a - b).abs().mean() / b.abs().mean()).item())
    n = steps * 8
    first = True
    for df, dl in zip(fused.layers, legacy.layers):
        if df["ring"] != 0:
            continue
        kf, kl = df["k"][:n].float(), dl["k"][:n].float()
        vf = df["ik"][:n].view(torch.float8_e4m3fn).float() * df["iks"][:n, None]
        vl = dl["ik"][:n].view(torch.float8_e4m3fn).float() * dl["iks"][:n, None]
        if first:
            assert torch.equal(df["k"][:n], dl["k"][:n]) and torch.equal(df["v"][:n], dl["v"][:n])
            assert ((vf - vl).abs() > 0.07 * vl.abs().amax(-1, keepdim=True)).float().mean().item() < 0.01
            first = False
        else:
            dk = ((kf - kl).abs().mean() / kl.abs().mean()).item()
            di = ((vf - vl).abs().mean() / vl.abs().mean()).item()
            assert dk < 0.12 and di < 0.15, (dk, di)
    assert worst < 0.12, worst


def _attn_ref(q, keys, vals, scale, sink=None):
    """fp32 softmax attention of one row: q [heads, hd], keys [n, hd], vals [n, vd]; optional sink logit per head
    (an extra softmax column without a value)."""
    s = (q.float() @ keys.float().T) * scale
    if sink is not None:
        s = torch.cat([s, sink.float()[:, None]], dim=1)
    p = torch.softmax(s, dim=-1)
    if sink is not None:
        p = p[:, :-1]
    return p @ vals.float()


@pytest.mark.parametrize("mode,heads,kvh,hd,pos0,splits", [(0, 8, 1, 192, 1000, 1), (0, 8, 8, 192, 57, 1), (1, 8, 1, 192, 5000, 16),
                                                           (1, 16, 4, 192, 300, 4), (2, 4, 1, 128, 1500, 8)])
def test_tensor_core_decode_attention_matches_torch(mode, heads, kvh, hd, pos0, splits):
    K = _K()
    g = torch.Generator(device="cuda").manual_seed(20 + mode)
    rows, vd, cap, top_k, window = 8, 128, 6144, 2048, 128 if mode == 0 else 1024
    ring = window + 16 if mode == 0 else 0
    q = torch.randn(16, heads, hd, device="cuda", generator=g).bfloat16()
    kc = torch.randn(cap if not ring else ring, kvh, hd, device="cuda", generator=g).bfloat16()
    vc = torch.randn(cap if not ring else ring, kvh, vd, device="cuda", generator=g).bfloat16()
    kb = torch.randn(16, kvh, hd, device="cuda", generator=g).bfloat16()
    vb = torch.randn(16, kvh, vd, device="cuda", generator=g).bfloat16()
    sink = torch.randn(heads, device="cuda", generator=g).bfloat16() if mode == 0 else None
    sel = torch.zeros(16, top_k, dtype=torch.int32, device="cuda")
    for r in range(rows):
        sel[r] = torch.sort(torch.randperm(pos0 + r + 1, device="cuda", generator=g)[:top_k]).values if pos0 + r + 1 > top_k else 0
    p = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    o = torch.zeros(16, heads * vd, device="cuda", dtype=torch.bfloat16)
    o8 = torch.zeros(16, heads * vd, device="cuda", dtype=torch.uint8)
    osc = torch.ones(16, heads, device="cuda")
    part = torch.zeros(K.attn_decode_part_floats(16, kvh, max(splits, 1)), device="cuda")
    tickets = torch.zeros(16 * kvh, dtype=torch.int32, device="cuda")
    a = K.AttnArgs()
    a.q, a.k_cache, a.v_cache, a.pos0 = q.data_ptr(), kc.data_ptr(), vc.data_ptr(), p.data_ptr()
    a.rows, a.heads, a.kv_heads, a.head_dim, a.v_dim = rows, heads, kvh, hd, vd
    a.scale, a.mode, a.window, a.ring = hd ** -0.5, mode, window, ring
    a.sink = None if sink is None else sink.data_ptr()
    a.sel, a.top_k = sel.data_ptr(), top_k
    a.k_blk, a.v_blk = kb.data_ptr(), vb.data_ptr()
    a.o_bf16, a.o8, a.o_scale = o.data_ptr(), o8.data_ptr(), osc.data_ptr()
    a.part, a.tickets = part.data_ptr(), tickets.data_ptr()
    for _ in range(2):                                    # the tickets reset themselves: a second launch must agree
        K.attn_decode(a, splits, pdl=False)
    torch.cuda.synchronize()
    hpg = heads // kvh
    worst = 0.0
    for r in range(rows):
        pos = pos0 + r
        for gi in range(kvh):
            if mode == 0:
                ids = torch.arange(max(0, pos - window + 1), pos + 1, device="cuda") % ring
                keys, vals = kc[ids, gi], vc[ids, gi]
            elif mode == 1:
                ids = sel[r].long() if pos + 1 > top_k else torch.arange(pos + 1, device="cuda")
                keys, vals = kc[ids, gi], vc[ids, gi]
            else:
                lo = max(0, pos0 - window)
                keys = torch.cat([kc[lo:pos0, gi], kb[:rows, gi]])
                vals = torch.cat([vc[lo:pos0, gi], vb[:rows, gi]])
            hs = slice(gi * hpg, (gi + 1) * hpg)
            want = _attn_ref(q[r, hs], keys, vals, hd ** -0.5, None if sink is None else sink[hs])
            got = o[r].view(heads, vd)[hs].float()
            worst = max(worst, ((got - want).abs().max() / want.abs().max()).item())
            deq = o8[r].view(heads, vd)[hs].view(torch.float8_e4m3fn).float() * osc[r, hs, None]
            assert ((deq - want).abs() <= want.abs().amax(-1, keepdim=True) / 14 + 1e-6).all()
    assert worst < 0.02, worst                             # bf16 probabilities and outputs
    assert (tickets == 0).all()
