"""tcgen05 skinny GEMM engine vs the fp32 torch oracle of the same op (single GPU, tp=1)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup():
    from naivert_b200.ops import kernels as K
    K.lib()
    return K


def _status():
    return torch.zeros(4, dtype=torch.int32, device="cuda")


def _packet(x, K):
    from naivert_b200.ops.quant import quantize_act_pow2
    r, k = x.shape
    x8 = torch.zeros(16, k, dtype=torch.uint8, device="cuda")
    xs = torch.ones(16, k // 128, dtype=torch.float32, device="cuda")
    q, s = quantize_act_pow2(x)
    x8[:r] = q.view(torch.uint8)
    xs[:r] = s
    return x8, xs


def _fab(K, status, epoch, features):
    f = K.FabricArgs()
    f.epoch = epoch.data_ptr()
    f.status = status.data_ptr()
    f.tp, f.rank, f.call_idx, f.features = 1, 0, 0, features
    f.timeout_ns = 1_000_000_000
    return f


@pytest.mark.parametrize("rows,n,k", [(8, 512, 1024), (1, 256, 256), (16, 1024, 4096)])
def test_fp8_linear_store(rows, n, k):
    K = _setup()
    from naivert_b200.ops.quant import quantize_fp8_block, w8a8_linear_ref
    g = torch.Generator(device="cuda").manual_seed(1)
    w = torch.randn(n, k, device="cuda", generator=g) * 0.05
    x = (torch.randn(rows, k, device="cuda", generator=g)).bfloat16().float()
    w8, ws = quantize_fp8_block(w)
    x8, xs = _packet(x, K)
    out = torch.zeros(rows, n, device="cuda")
    st = _status()
    a = K.GemmArgs()
    a.n_total, a.k_total, a.rows, a.a_group = n, k, rows, 0
    a.w_scale0, a.a_scale = ws.data_ptr(), xs.data_ptr()
    a.out_f32, a.ld_out, a.out_scale = out.data_ptr(), n, 1.0
    a.status = st.data_ptr()
    tmA, tmB = K.weight_tmap(w8.view(torch.uint8)), K.act_tmap(x8)
    K.gemm(K.gemm_variant(True, False, K.EPI_STORE_F32, K.GROUP_NONE), tmA, None, tmB, a, n // 128)
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    ref = w8a8_linear_ref(x, w8, ws)
    err = (out - ref).abs().max().item()
    assert err <= 1e-4 * ref.abs().max().item() + 1e-6, err


def test_bf16_linear_store():
    K = _setup()
    g = torch.Generator(device="cuda").manual_seed(2)
    rows, n, k = 8, 640, 1024                       # 640 = 5 tiles
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).bfloat16()
    x = torch.zeros(16, k, device="cuda", dtype=torch.bfloat16)
    x[:rows] = torch.randn(rows, k, device="cuda", generator=g).bfloat16()
    out = torch.zeros(rows, n, device="cuda")
    st = _status()
    a = K.GemmArgs()
    a.n_total, a.k_total, a.rows = n, k, rows
    a.out_f32, a.ld_out, a.out_scale = out.data_ptr(), n, 1.0
    a.status = st.data_ptr()
    K.gemm(K.gemm_variant(False, False, K.EPI_STORE_F32, K.GROUP_NONE), K.weight_tmap(w), None, K.act_tmap(x), a, n // 128)
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    ref = x[:rows].float() @ w.float().T
    assert (out - ref).abs().max().item() <= 2e-3 * ref.abs().max().item()


def test_fp8_allreduce_tp1_residual():
    K = _setup()
    from naivert_b200.ops.quant import quantize_fp8_block, w8a8_linear_ref
    g = torch.Generator(device="cuda").manual_seed(3)
    rows, n, k = 8, 1024, 512
    w8, ws = quantize_fp8_block(torch.randn(n, k, device="cuda", generator=g) * 0.05)
    x = torch.randn(rows, k, device="cuda", generator=g).bfloat16().float()
    resid = torch.randn(rows, n, device="cuda", generator=g).bfloat16()
    x8, xs = _packet(x, K)
    out = torch.zeros(rows, n, device="cuda", dtype=torch.bfloat16)
    st, epoch = _status(), torch.ones(1, dtype=torch.int32, device="cuda")
    a = K.GemmArgs()
    a.n_total, a.k_total, a.rows = n, k, rows
    a.w_scale0, a.a_scale = ws.data_ptr(), xs.data_ptr()
    a.out_bf16, a.ld_out, a.resid = out.data_ptr(), n, resid.data_ptr()
    a.fab = _fab(K, st, epoch, n)
    a.status = st.data_ptr()
    K.gemm(K.gemm_variant(True, False, K.EPI_ALLREDUCE, K.GROUP_NONE), K.weight_tmap(w8.view(torch.uint8)), None,
           K.act_tmap(x8), a, n // 128)
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    ref = (resid.float() + w8a8_linear_ref(x, w8, ws).bfloat16().float()).bfloat16()
    diff = (out.float() - ref.float()).abs()
    assert diff.max().item() <= 0.02 * ref.float().abs().max().item()
    assert (diff > 0).float().mean().item() < 0.01       # at most rare 1-ulp flips


def test_moe_gate_up_down_grouped():
    """Grouped gate/up (SiLU + e4m3 requantisation) followed by the probability-weighted down
    projection, against the W8A8 recipe evaluated in torch."""
    K = _setup()
    from naivert_b200.ops.quant import quantize_act_pow2, quantize_fp8_block, w8a8_linear_ref
    g = torch.Generator(device="cuda").manual_seed(4)
    E, H, I, rows, slots = 8, 512, 256, 8, 5
    gate = torch.randn(E, I, H, device="cuda", generator=g) * 0.05
    up = torch.randn(E, I, H, device="cuda", generator=g) * 0.05
    down = torch.randn(E, H, I, device="cuda", generator=g) * 0.05
    g8, gs = quantize_fp8_block(gate)
    u8, us = quantize_fp8_block(up)
    d8, ds = quantize_fp8_block(down)
    x = torch.randn(rows, H, device="cuda", generator=g).bfloat16().float()
    x8, xs = _packet(x, K)
    active = torch.tensor([1, 2, 4, 6, 7, 0, 0, 0], dtype=torch.int32, device="cuda")
    n_active = torch.tensor([slots], dtype=torch.int32, device="cuda")
    probs = torch.zeros(8, 16, device="cuda")
    probs[:slots, :rows] = torch.rand(slots, rows, device="cuda", generator=g)
    probs[1, 3] = 0.0
    y8 = torch.zeros(8 * 16, I, dtype=torch.uint8, device="cuda")
    ys = torch.ones(8 * 16, I // 128, device="cuda")
    st, epoch = _status(), torch.ones(1, dtype=torch.int32, device="cuda")

    a = K.GemmArgs()
    a.n_total, a.k_total, a.rows = I, H, rows
    a.n_active, a.active_ids, a.max_slots = n_active.data_ptr(), active.data_ptr(), 8
    a.w_scale0, a.w_scale1, a.a_scale = gs.data_ptr(), us.data_ptr(), xs.data_ptr()
    a.out_q, a.out_qscale = y8.data_ptr(), ys.data_ptr()
    a.status = st.data_ptr()
    K.gemm(K.gemm_variant(True, True, K.EPI_SILU_QUANT, K.GROUP_ITEM), K.weight_tmap(g8.view(torch.uint8)),
           K.weight_tmap(u8.view(torch.uint8)), K.act_tmap(x8), a, I // 128, 8)

    resid = torch.randn(rows, H, device="cuda", generator=g).bfloat16()
    out = torch.zeros(rows, H, device="cuda", dtype=torch.bfloat16)
    b = K.GemmArgs()
    b.n_total, b.k_total, b.rows = H, I, rows
    b.n_active, b.active_ids, b.probs, b.max_slots = n_active.data_ptr(), active.data_ptr(), probs.data_ptr(), 8
    b.n_experts = E
    b.w_scale0, b.a_scale = ds.data_ptr(), ys.data_ptr()
    b.out_bf16, b.ld_out, b.resid = out.data_ptr(), H, resid.data_ptr()
    b.fab = _fab(K, st, epoch, H)
    b.status = st.data_ptr()
    K.gemm(K.gemm_variant(True, False, K.EPI_ALLREDUCE, K.GROUP_LOOP), K.weight_tmap(d8.view(torch.uint8)), None,
           K.act_tmap(y8), b, H // 128, 1)
    torch.cuda.synchronize()
    assert int(st[0]) == 0

    mix = torch.zeros(rows, H, device="cuda")
    for s in range(slots):
        e = int(active[s])
        gg = w8a8_linear_ref(x, g8[e], gs[e])
        uu = w8a8_linear_ref(x, u8[e], us[e])
        y = torch.nn.functional.silu(gg) * uu
        yq, ysc = quantize_act_pow2(y)
        got_q = y8[s * 16:s * 16 + rows].view(torch.float8_e4m3fn).float() * ys[s * 16:s * 16 + rows].repeat_interleave(128, 1)
        want_q = yq.float() * ysc.repeat_interleave(128, 1)
        assert (got_q - want_q).abs().max().item() <= 0.07 * want_q.abs().max().item()   # one e4m3 step
        assert ((got_q - want_q).abs() > 0).float().mean().item() < 0.02
        mix += probs[s, :rows, None] * w8a8_linear_ref(y, d8[e], ds[e])
    ref = (resid.float() + mix.bfloat16().float()).bfloat16().float()
    assert (out.float() - ref).abs().max().item() <= 0.02 * ref.abs().max().item()


def test_prep_norm_packet():
    K = _setup()
    from naivert_b200.ops.quant import quantize_act_pow2
    g = torch.Generator(device="cuda").manual_seed(5)
    rows, H = 8, 1024
    x = torch.randn(16, H, device="cuda", generator=g).bfloat16()
    gamma = (1 + 0.05 * torch.randn(H, device="cuda", generator=g)).bfloat16()
    xn = torch.empty(16, H, device="cuda", dtype=torch.bfloat16)
    x8 = torch.empty(16, H, device="cuda", dtype=torch.uint8)
    xs = torch.empty(16, H // 128, device="cuda")
    K.prep_norm(x, gamma, rows, 1e-5, xn, x8, xs, pdl=False)
    torch.cuda.synchronize()
    xf = x[:rows].float()
    ref = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma.float()).bfloat16()
    d = (xn[:rows].float() - ref.float()).abs()
    assert d.max().item() <= 0.01 * ref.float().abs().max().item()
    q, s = quantize_act_pow2(xn[:rows].float())
    assert torch.equal(xs[:rows], s)
    assert torch.equal(x8[:rows], q.view(torch.uint8))
    assert int(xn[rows:].abs().sum()) == 0 and int(x8[rows:].sum()) == 0


def _items(n_items, step=64):
    off = (torch.arange(n_items, dtype=torch.int32, device="cuda") * step).contiguous()
    ids = torch.zeros(n_items, dtype=torch.int32, device="cuda")
    cnt = torch.tensor([n_items], dtype=torch.int32, device="cuda")
    return off, ids, cnt


@pytest.mark.parametrize("order", [False, True])
def test_chunk_gemm_bf16_matches_torch(order):
    """64-column persistent chunk GEMM (bf16, fp32 store) against torch on 320 rows x 640 features x K 1024."""
    K = _setup()
    g = torch.Generator(device="cuda").manual_seed(3)
    rows, n, k = 320, 640, 1024
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).bfloat16()
    x = torch.randn(rows, k, device="cuda", generator=g).bfloat16()
    out = torch.zeros(rows, n, device="cuda")
    st = _status()
    off, ids, cnt = _items(rows // 64)
    a = K.GemmArgs()
    a.n_total, a.k_total, a.rows, a.out_scale = n, k, 64, 1.0
    a.n_active, a.active_ids, a.max_slots, a.row_offsets = cnt.data_ptr(), ids.data_ptr(), rows // 64, off.data_ptr()
    a.out_f32, a.ld_out, a.status = out.data_ptr(), n, st.data_ptr()
    K.wide_gemm(K.gemm_variant(False, False, K.EPI_STORE_F32, K.GROUP_ITEM), K.weight_tmap(w), None, K.act_tmap(x, 64), a,
                n // 128, rows // 64, items_fastest=order)
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    ref = x.float() @ w.float().T
    assert (out - ref).abs().max().item() <= 2e-3 * ref.abs().max().item()


def test_chunk_gemm_fp8_gate_up_matches_torch():
    """e4m3 block-scaled gate/up with SiLU and e4m3 re-quantisation on the chunk engine vs the torch recipe."""
    K = _setup()
    from naivert_b200.ops.quant import dequant_act, quantize_act_pow2, quantize_fp8_block, w8a8_linear_ref
    g = torch.Generator(device="cuda").manual_seed(4)
    rows, n, k = 192, 256, 1024
    wg = torch.randn(n, k, device="cuda", generator=g) * 0.05
    wu = torch.randn(n, k, device="cuda", generator=g) * 0.05
    x = torch.randn(rows, k, device="cuda", generator=g).bfloat16().float()
    g8, gs = quantize_fp8_block(wg)
    u8, us = quantize_fp8_block(wu)
    xq, xs = quantize_act_pow2(x)
    x8 = xq.view(torch.uint8).contiguous()
    xs = xs.float().contiguous()
    y8 = torch.zeros(rows, n, dtype=torch.uint8, device="cuda")
    ys = torch.zeros(rows, n // 128, device="cuda")
    st = _status()
    off, ids, cnt = _items(rows // 64)
    a = K.GemmArgs()
    a.n_total, a.k_total, a.rows, a.out_scale = n, k, 64, 1.0
    a.n_active, a.active_ids, a.max_slots, a.row_offsets = cnt.data_ptr(), ids.data_ptr(), rows // 64, off.data_ptr()
    a.w_scale0, a.w_scale1, a.a_scale = gs.data_ptr(), us.data_ptr(), xs.data_ptr()
    a.out_q, a.out_qscale, a.status = y8.data_ptr(), ys.data_ptr(), st.data_ptr()
    K.wide_gemm(K.gemm_variant(True, True, K.EPI_SILU_QUANT, K.GROUP_ITEM), K.weight_tmap(g8.view(torch.uint8)),
                K.weight_tmap(u8.view(torch.uint8)), K.act_tmap(x8, 64), a, n // 128, rows // 64)
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    gg, uu = w8a8_linear_ref(x, g8, gs), w8a8_linear_ref(x, u8, us)
    want = torch.nn.functional.silu(gg) * uu
    got = dequant_act(y8.view(torch.float8_e4m3fn), ys)
    # one e4m3 rounding of the reference value (relative step 2^-3, half of it as error) plus accumulation noise
    assert (got - want).abs().max().item() <= 0.07 * want.abs().max().item()
    wq, wsc = quantize_act_pow2(want)
    assert torch.equal(ys, wsc.float()) or (ys - wsc.float()).abs().max().item() <= ys.max().item()
