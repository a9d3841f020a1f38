"""Kernels of the step against plain torch fp32 references of the same ops, at the full model's dimensions:
the fused q/k/v(/indexer) projection epilogue (RMSNorm operand, RoPE, KV append, indexer query / key
quantisation), the indexer logits in both forms (CUDA-core kernel and tcgen05 sweep) and one Markov proposal step."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _K():
    from naivert_b200.ops import kernels as K
    K.lib()
    K.aux_lib()
    return K


def _rope(x, tab):
    """x [..., 2 * n] adjacent pairs, tab [n, 2] (cos, sin)."""
    xr = x.reshape(*x.shape[:-1], -1, 2)
    re = xr[..., 0] * tab[:, 0] - xr[..., 1] * tab[:, 1]
    im = xr[..., 0] * tab[:, 1] + xr[..., 1] * tab[:, 0]
    return torch.stack((re, im), dim=-1).reshape(x.shape)


def _bf(x):
    return x.bfloat16().float()


def test_qkv_projection_epilogue_matches_torch():
    """hidden 4096, 8 query heads x 192 + 1 KV head (192 / 128), indexer 16 x 128 + key + head weights, 8 rows."""
    K = _K()
    from naivert_b200.models.reference import rope_table
    g = torch.Generator(device="cuda").manual_seed(31)
    H, nh, hd, vd, rope, ih, idim, irope, rows, pos0, cap = 4096, 8, 192, 128, 64, 16, 128, 64, 8, 37, 128
    col_k, col_v = nh * hd, nh * hd + hd
    col_iq = -(-(col_v + vd) // 128) * 128
    col_ik, col_iw = col_iq + ih * idim, col_iq + ih * idim + idim
    n = -(-(col_iw + ih) // 128) * 128
    W = torch.zeros(n, H, device="cuda", dtype=torch.bfloat16)
    W[:col_v + vd] = (torch.randn(col_v + vd, H, device="cuda", generator=g) * 0.03).bfloat16()
    W[col_iq:col_iw + ih] = (torch.randn(col_iw + ih - col_iq, H, device="cuda", generator=g) * 0.03).bfloat16()
    x = torch.zeros(16, H, device="cuda", dtype=torch.bfloat16)
    x[:rows] = (torch.randn(rows, H, device="cuda", generator=g) * 2).bfloat16()
    gamma = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).bfloat16()
    ik_w = (1 + 0.1 * torch.randn(idim, device="cuda", generator=g)).bfloat16()
    ik_b = (0.1 * torch.randn(idim, device="cuda", generator=g)).bfloat16()
    ssq = x.float().pow(2).view(16, H // 128, 128).sum(-1).t().contiguous()
    pos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    positions = torch.arange(pos0, pos0 + rows, device="cuda")
    tab = torch.zeros(16, rope // 2, 2, device="cuda")
    tab[:rows] = rope_table(positions, rope, 1e7)
    itab = torch.zeros(16, irope // 2, 2, device="cuda")
    itab[:rows] = rope_table(positions, irope, 1e7)
    q_out = torch.zeros(16, nh, hd, device="cuda", dtype=torch.bfloat16)
    kc = torch.zeros(cap, 1, hd, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros(cap, 1, vd, device="cuda", dtype=torch.bfloat16)
    iq8 = torch.zeros(16 * ih, idim, device="cuda", dtype=torch.uint8)
    iqs = torch.ones(16, ih, device="cuda")
    ihw = torch.zeros(16, ih, device="cuda")
    ikc = torch.zeros(cap, idim, device="cuda", dtype=torch.uint8)
    iks = torch.ones(cap, device="cuda")
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    a = K.GemmArgs()
    a.n_total, a.k_total, a.rows, a.out_scale = n, H, rows, 1.0
    a.nx, a.ngamma, a.nssq, a.neps = x.data_ptr(), gamma.data_ptr(), ssq.data_ptr(), 1e-5
    a.status = st.data_ptr()
    p = a.post
    p.rows, p.pos0 = rows, pos.data_ptr()
    p.heads, p.kv_heads, p.head_dim, p.v_dim, p.rope_dim, p.value_scale = nh, 1, hd, vd, rope, 0.707
    p.rope, p.q_out, p.k_cache, p.v_cache, p.ring = tab.data_ptr(), q_out.data_ptr(), kc.data_ptr(), vc.data_ptr(), 0
    p.norm_eps = 1e-5
    p.idx_heads, p.idx_dim, p.idx_rope, p.idx_rope_tab = ih, idim, irope, itab.data_ptr()
    p.ik_w, p.ik_b, p.ln_eps, p.idx_weight_scale = ik_w.data_ptr(), ik_b.data_ptr(), 1e-5, ih ** -0.5
    p.iq8, p.ihw, p.ik_cache, p.ik_scale, p.iq_scale = iq8.data_ptr(), ihw.data_ptr(), ikc.data_ptr(), iks.data_ptr(), iqs.data_ptr()
    p.col_q, p.col_k, p.col_v, p.col_iq, p.col_ik, p.col_iw = 0, col_k, col_v, col_iq, col_ik, col_iw
    nt = n // 128
    K.gemm(K.gemm_variant(False, False, K.EPI_QKV_POST, K.GROUP_NONE, K.B_NORM), K.weight_tmap(W), None, None, a, nt,
           K.pick_split(nt, H // 64, max_split=8), pdl=False)
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    # ---- torch fp32 reference
    xf = x[:rows].float()
    xn = _bf(xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma.float())
    proj = xn @ W.float().T                                               # [rows, n] fp32
    t, it = tab[:rows, None], itab[:rows, None]                           # [rows, 1, pairs, 2]

    def rope_heads(v, table, dims):                                       # v [rows, heads, dim]
        out = v.clone()
        xr = v[..., :dims].reshape(*v.shape[:-1], dims // 2, 2)
        re = xr[..., 0] * table[..., 0] - xr[..., 1] * table[..., 1]
        im = xr[..., 0] * table[..., 1] + xr[..., 1] * table[..., 0]
        out[..., :dims] = torch.stack((re, im), dim=-1).reshape(*v.shape[:-1], dims)
        return out

    q_ref = _bf(rope_heads(_bf(proj[:, :col_k]).view(rows, nh, hd), t, rope))
    k_ref = _bf(rope_heads(_bf(proj[:, col_k:col_v]).view(rows, 1, hd), t, rope))
    v_ref = _bf(proj[:, col_v:col_v + vd] * 0.707)
    tol = lambda ref: 0.01 * ref.abs().max().item()                        # one bf16 step of the largest value
    assert (q_out[:rows].float() - q_ref).abs().max().item() <= tol(q_ref)
    assert (kc[pos0:pos0 + rows].float() - k_ref).abs().max().item() <= tol(k_ref)
    assert (vc[pos0:pos0 + rows, 0].float() - v_ref).abs().max().item() <= tol(v_ref)
    assert float(kc[:pos0].abs().sum()) == 0 and float(kc[pos0 + rows:].abs().sum()) == 0
    # indexer queries: bf16 -> RoPE -> bf16 -> e4m3 with scale amax / 448 per (row, head)
    iq = _bf(rope_heads(_bf(proj[:, col_iq:col_ik]).view(rows, ih, idim), it, irope))
    got_iq = iq8.view(16, ih, idim)[:rows].view(torch.float8_e4m3fn).float() * iqs[:rows, :, None]
    assert torch.allclose(iqs[:rows], iq.abs().amax(-1) / 448, rtol=2e-2)
    assert (got_iq - iq).abs().max().item() <= iq.abs().max().item() / 14
    assert torch.allclose(ihw[:rows], proj[:, col_iw:col_iw + ih] * ih ** -0.5, rtol=1e-3, atol=1e-5)
    # indexer key: LayerNorm -> bf16 -> RoPE -> bf16 -> e4m3 with scale amax / 448 per row
    kraw = proj[:, col_ik:col_ik + idim]
    kn = _bf(torch.nn.functional.layer_norm(kraw, (idim,), ik_w.float(), ik_b.float(), 1e-5))
    kn = _bf(rope_heads(kn.view(rows, 1, idim), it, irope)).view(rows, idim)
    got_k = ikc[pos0:pos0 + rows].view(torch.float8_e4m3fn).float() * iks[pos0:pos0 + rows, None]
    assert torch.allclose(iks[pos0:pos0 + rows], kn.abs().amax(-1) / 448, rtol=2e-2)
    assert (got_k - kn).abs().max().item() <= kn.abs().max().item() / 14


@pytest.mark.parametrize("use_sweep", [False, True])
def test_indexer_logits_match_torch(use_sweep):
    """logit[r, t] = (sum_h relu(q8[r, h] . k8[t]) * w[r, h]) * k_scale[t] over 16 heads x 128 dims, 8 rows."""
    K = _K()
    g = torch.Generator(device="cuda").manual_seed(32)
    rows, heads, dim, cap, pos0, top_k = 8, 16, 128, 4096, 3000, 2048
    q = (torch.randn(16 * heads, dim, device="cuda", generator=g) * 40).to(torch.float8_e4m3fn)
    kk = (torch.randn(cap, dim, device="cuda", generator=g) * 40).to(torch.float8_e4m3fn)
    ks = torch.rand(cap, device="cuda", generator=g) + 0.5
    hw = torch.randn(16, heads, device="cuda", generator=g)
    qs = torch.rand(16, heads, device="cuda", generator=g) + 0.5
    logits = torch.zeros(16, cap, device="cuda")
    p = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    q8, k8 = q.view(torch.uint8), kk.view(torch.uint8)
    if use_sweep:
        km, qm = K.sweep_maps(k8, q8)
        sw = K.SweepArgs()
        sw.ihw, sw.iks, sw.pos0, sw.iq_scale = hw.data_ptr(), ks.data_ptr(), p.data_ptr(), qs.data_ptr()
        sw.rows, sw.heads, sw.top_k, sw.logits, sw.ld, sw.status = rows, heads, top_k, logits.data_ptr(), cap, st.data_ptr()
        K.index_sweep(km, qm, sw, 32, pdl=False)
    else:
        ia = K.IndexArgs()
        ia.iq8, ia.ihw, ia.ik, ia.iks, ia.pos0, ia.iq_scale = q8.data_ptr(), hw.data_ptr(), k8.data_ptr(), ks.data_ptr(), p.data_ptr(), qs.data_ptr()
        ia.rows, ia.heads, ia.dim, ia.top_k, ia.logits, ia.ld = rows, heads, dim, top_k, logits.data_ptr(), cap
        K.index_logits_simple(ia, 64, pdl=False)
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    qf = q.float().view(16, heads, dim)[:rows]
    total = pos0 + rows
    dots = torch.einsum("rhd,td->rht", qf.double(), kk.float().double()[:total])
    ref = (dots.clamp_min(0) * (hw[:rows] * qs[:rows]).double()[:, :, None]).sum(1) * ks[:total].double()
    got = logits[:rows, :total].double()
    for r in range(rows):                                  # every row sees the keys up to its own position (at least)
        n = pos0 + r + 1
        assert (got[r, :n] - ref[r, :n]).abs().max().item() <= 2e-5 * ref[r, :n].abs().max().item()


def test_markov_step_matches_torch():
    """z = head logits + bf16(W2_shard . W1[prev]); proposal = arg max of z / T + Gumbel noise from the Philox stream."""
    K = _K()
    g = torch.Generator(device="cuda").manual_seed(33)
    vocab, vlocal, vbase, rank_dim, step, rnd = 4096, 1500, 1024, 256, 2, 5
    w1 = (torch.randn(vocab, rank_dim, device="cuda", generator=g) * 0.1).bfloat16()
    w2 = (torch.randn(vlocal, rank_dim, device="cuda", generator=g) * 0.1).bfloat16()
    logits = torch.randn(16, vlocal, device="cuda", generator=g) * 2
    zq = torch.zeros(8, vlocal, device="cuda")
    block = torch.tensor([7, 99, 1234, 0, 0, 0, 0, 0], dtype=torch.int32, device="cuda")
    params = torch.tensor([2.5, 0.95, 1, 0, 0, -1, 2.5, 0], dtype=torch.float32, device="cuda")
    seed = torch.tensor([4242], dtype=torch.int64, device="cuda")
    ctrl = torch.zeros(16, dtype=torch.int32, device="cuda")
    ctrl[8] = rnd
    best = torch.zeros(8, dtype=torch.int64, device="cuda")
    ticket = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    epoch = torch.ones(1, dtype=torch.int32, device="cuda")
    m = K.MarkovArgs()
    m.logits, m.ld, m.w1, m.w2, m.rank_dim = logits.data_ptr(), vlocal, w1.data_ptr(), w2.data_ptr(), rank_dim
    m.vlocal, m.vbase, m.vocab = vlocal, vbase, vocab
    m.block_ids, m.zq, m.params, m.seed, m.ctrl = block.data_ptr(), zq.data_ptr(), params.data_ptr(), seed.data_ptr(), ctrl.data_ptr()
    m.best, m.ticket = best.data_ptr(), ticket.data_ptr()
    m.x.epoch, m.x.status, m.x.tp, m.x.rank, m.x.timeout_ns = epoch.data_ptr(), st.data_ptr(), 1, 0, 10 ** 9
    K.markov_step(m, step, pdl=False)
    torch.cuda.synchronize()
    prev = int(block[step])
    bias = (w2.float() @ w1[prev].float()).bfloat16().float()
    z = logits[step] + bias
    assert (zq[step] - z).abs().max().item() <= 2e-2                      # bf16 rounding of the bias near a tie
    u = torch.tensor([K.philox_uniform(4242, 3, rnd * 8 + step, t + vbase) for t in range(vlocal)], device="cuda")
    score = zq[step].double() * 2.5 - torch.log(-torch.log(u.double()))
    tok = int(block[step + 1]) - vbase
    assert 0 <= tok < vlocal
    assert score[tok].item() >= score.max().item() - 1e-3
