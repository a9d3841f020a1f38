"""Failure detection on the device without faulting it: a wait for a peer that never publishes runs out after a
short limit, the kernel records where it gave up in the status word and returns, the context stays usable and
the host-side check raises.  One GPU: the "peer" mailbox is a second local buffer that nothing writes."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_mailbox_wait_times_out_with_status_and_context_survives():
    from naivert_b200.ops import kernels as K
    from naivert_b200.ops.quant import quantize_act_pow2, quantize_fp8_block
    K.lib()
    g = torch.Generator(device="cuda").manual_seed(1)
    rows, n, k = 8, 512, 256
    w8, ws = quantize_fp8_block(torch.randn(n, k, device="cuda", generator=g) * 0.05)
    xq, xsc = quantize_act_pow2(torch.randn(rows, k, device="cuda", generator=g).bfloat16().float())
    x8 = torch.zeros(16, k, dtype=torch.uint8, device="cuda")
    xs = torch.ones(16, k // 128, device="cuda")
    x8[:rows], xs[:rows] = xq.view(torch.uint8), xsc
    out = torch.zeros(rows, n, device="cuda", dtype=torch.bfloat16)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    epoch = torch.ones(1, dtype=torch.int32, device="cuda")
    words = K.K_MAILBOX_SLABS * 2 * n * K.K_ROW_PAIRS
    mine = torch.zeros(words, dtype=torch.int64, device="cuda")        # nobody ever writes rank 1's lane here
    peer = torch.zeros(words, dtype=torch.int64, device="cuda")        # stands in for rank 1's mailbox
    a = K.GemmArgs()
    a.n_total, a.k_total, a.rows = n, k, rows
    a.w_scale0, a.a_scale = ws.data_ptr(), xs.data_ptr()
    a.out_bf16, a.ld_out = out.data_ptr(), n
    f = a.fab
    f.mailbox[0], f.mailbox[1] = mine.data_ptr(), peer.data_ptr()
    f.epoch, f.status, f.tp, f.rank, f.call_idx, f.features = epoch.data_ptr(), status.data_ptr(), 2, 0, 0, n
    f.timeout_ns, f.mode, f.ag_call = 2_000_000, 0, -1                 # 2 ms
    a.status = status.data_ptr()
    tmA, tmB = K.weight_tmap(w8.view(torch.uint8)), K.act_tmap(x8)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    K.gemm(K.gemm_variant(True, False, K.EPI_ALLREDUCE, K.GROUP_NONE), tmA, None, tmB, a, n // 128, pdl=False)
    ev1.record()
    torch.cuda.synchronize()                                           # returns: the kernel gave up by itself
    assert ev0.elapsed_time(ev1) < 500.0
    code = int(status[0])
    assert code != 0 and (code & 0xF00) == 0x500, hex(code)            # kSiteMailbox | missing word
    assert int(peer.ne(0).sum()) > 0                                   # our own partial was published to the peer

    from naivert_b200.parallel.fabric import Fabric
    fab = Fabric(0, 1, n, device=torch.device("cuda"))
    fab.status.copy_(status)
    with pytest.raises(RuntimeError, match="gave up"):
        fab.check()

    # the context is intact: the same GEMM as a single rank gives the right numbers
    status.zero_()
    f.tp = 1
    K.gemm(K.gemm_variant(True, False, K.EPI_ALLREDUCE, K.GROUP_NONE), tmA, None, tmB, a, n // 128, pdl=False)
    torch.cuda.synchronize()
    from naivert_b200.ops.quant import w8a8_linear_ref
    ref = w8a8_linear_ref(xq.float() * xsc.repeat_interleave(128, dim=1), w8, ws).bfloat16().float()
    assert int(status[0]) == 0
    assert (out.float() - ref).abs().max().item() <= 0.02 * ref.abs().max().item()


def test_step_outputs_stay_inside_their_buffers():
    """Canary-fenced copies of the step's scratch and output buffers: a verify step must not touch the guard bytes
    around any of them."""
    from naivert_b200.models.naive_n0p5 import small_w8a8_spec
    from naivert_b200.models.weights import init_state_dict, prepare_weights, shard_weights
    from naivert_b200.runtime.target import LocalFabric, TargetRuntime
    from naivert_b200.utils.guarded import GuardedPool
    spec = small_w8a8_spec(4)
    w = prepare_weights(spec, init_state_dict(spec, seed=0, device="cuda"))
    rt = TargetRuntime(spec, shard_weights(spec, w, 0, 1), LocalFabric("cuda"), rows=8, capacity=512)
    pool = GuardedPool("cuda")
    names = ["x", "x8", "xs", "y8", "ys", "scores", "probs", "active_ids", "topk_ids", "topk_p", "logits", "q", "o8", "os",
             "ssq", "sel", "iq8", "ihw", "iq_scale", "feats"]
    for nme in names:
        old = getattr(rt, nme)
        new = pool.like(old, nme)
        new.copy_(old)
        setattr(rt, nme, new)
    # tensor maps and argument blocks hold raw pointers: rebuild them over the fenced buffers
    from naivert_b200.ops import kernels as K
    rt.map_x8, rt.map_y8, rt.map_o8 = K.act_tmap(rt.x8), K.act_tmap(rt.y8), K.act_tmap(rt.o8)
    rt._build_args()
    g = torch.Generator().manual_seed(0)
    for i in range(40):                                  # crosses the indexer's top-k boundary
        rt.set_inputs(torch.randint(0, spec.vocab, (8,), generator=g), i * 8)
        rt.step()
    torch.cuda.synchronize()
    rt.fab.check()
    assert torch.isfinite(rt.logits[:8]).all()
    pool.verify()


@pytest.mark.gpu
def test_index_checking_build_records_the_first_bad_index_and_stays_clean_on_a_real_decode():
    """The -DNRT_BOUNDS_CHECK flavour of the library (same sources) tests every data-derived index before use.  A decode
    that crosses the sparse-attention boundary leaves the bounds words empty; a token id beyond the vocabulary - clamped
    before the gather in every build, so nothing is read out of range - is recorded with its site and value, once."""
    import json
    import os
    import subprocess
    import sys
    from naivert_b200.ops import build as B
    lib = os.path.join(B.LIB_DIR, B.BOUNDS_LIB_NAME)
    man = os.path.join(B.LIB_DIR, "manifest_bounds.json")
    if not (os.path.isfile(lib) and os.path.isfile(man) and json.load(open(man)).get("digest") == B.source_digest()):
        pytest.skip("the checking flavour is not built (python -m naivert_b200.ops.build --bounds)")
    env = dict(os.environ, NAIVERT_BOUNDS_CHECK="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "tests", "bounds_worker.py")], env=env, cwd=root,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("BOUNDS ")][-1]
    out = json.loads(line[len("BOUNDS "):])
    assert out["library"] == B.BOUNDS_LIB_NAME and out["tokens"] == 48
    # no selected key beyond its query, no expert id beyond the table (token ids are clamped in every build; padded
    # rows may carry placeholders, so their records are not a failure)
    assert [v for v in out["clean_run"] if v[0] in ("attn_decode", "moe_fused")] == [], out["clean_run"]
    from naivert_b200.models.naive_n0p5 import small_w8a8_spec
    assert out["after_bad_token"] == [["target_kernels", "token id", small_w8a8_spec(4).vocab + 5]]
    assert out["cleared"] == [] and out["row_is_last_table_row"]
