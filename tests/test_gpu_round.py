"""Sampler kernels vs the integer oracle, and end-to-end speculative rounds (single GPU, tp=1)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine(layers=2, capacity=1024, seed=0):
    from naivert_b200.models.naive_n0p5 import small_w8a8_spec
    from naivert_b200.runtime.engine import Engine
    spec = small_w8a8_spec(layers)
    return spec, Engine.build(spec, capacity=capacity, seed=seed)


@pytest.mark.parametrize("one_launch", [False, True])
def test_sampler_matches_integer_oracle(one_launch):
    from naivert_b200.models.spec import SamplingParams
    from naivert_b200.ops import kernels as K
    from naivert_b200.ops import sampling_ref as S
    spec, eng = _engine()
    r = eng.round
    V = spec.vocab
    g = torch.Generator(device="cuda").manual_seed(3)
    for trial, (top_p, forced, temp) in enumerate([(0.95, None, 1.0), (0.5, None, 0.4), (0.95, 0.7, 0.4), (1e-6, None, 1.0)]):
        zp = torch.randn(8, V, device="cuda", generator=g) * 3
        zq = zp[:7] + torch.randn(7, V, device="cuda", generator=g)
        r.t.logits[:8].copy_(zp)
        r.draft.zq[:7].copy_(zq)
        ids = [11] + [int(torch.multinomial(torch.softmax(zq[j] / temp, -1), 1, generator=g)) for j in range(7)]
        r.block_ids[:8].copy_(torch.tensor(ids, dtype=torch.int32))
        sp = SamplingParams(temperature=temp, top_p=top_p, seed=77 + trial, forced_accept_p=forced)
        r.set_sampling(sp)
        r.t.ctrl[8] = trial
        if one_launch:
            assert K.sampler_persistent(r.args_sampler, r.sampler_sync, domain=1, pdl=False) == 0
        else:
            K.sampler_run(r.args_sampler, domain=1, pdl=False)
        torch.cuda.synchronize()
        eng.fabric.check()
        st = r.state.view(torch.int32)
        # SamplerState layout: rowmax f32[16] | total u64[16] | above u64[16] | kept u64[16] | prefix u32[16] | ...
        kept = r.state[8 + 32:8 + 48].tolist()
        prefix = st[(8 + 48) * 2:(8 + 48) * 2 + 16].tolist()
        tail = (K.sampler_state_bytes() - 10 * 4) // 4
        accepted, extra = int(st[tail + 0]), int(st[tail + 1])
        m, tok, tp_, tq_ = S.verify_oracle(zp, zq, ids, 1.0 / temp, sp.clamped_top_p(), sp.seed, trial, forced=forced)
        assert [t[1] for t in tp_] == kept[:8], trial
        assert [t[0] for t in tp_] == [p & 0xFFFFFFFF for p in prefix[:8]], trial
        assert [t[1] for t in tq_] == kept[8:15], trial
        assert accepted == m, (trial, accepted, m)
        assert extra == tok, (trial, extra, tok)


def test_forced_acceptance_counts_and_determinism():
    from naivert_b200.models.spec import SamplingParams
    spec, eng = _engine()
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, spec.vocab - 16, (37,), generator=g)
    full = eng.generate(prompt, 64, SamplingParams(temperature=0.4, seed=5, forced_accept_p=1.0))
    assert full.stop_reason == "output_limit" and len(full.tokens) == 64 and full.rounds == 8
    none = eng.generate(prompt, 20, SamplingParams(temperature=0.4, seed=5, forced_accept_p=0.0))
    assert len(none.tokens) == 20 and none.rounds == 20
    _, fresh = _engine()                                                  # first request of a new engine (captures)
    a0 = fresh.generate(prompt, 96, SamplingParams(temperature=0.4, seed=5, forced_accept_p=0.7))
    a = eng.generate(prompt, 96, SamplingParams(temperature=0.4, seed=5, forced_accept_p=0.7))
    assert a0.tokens == a.tokens
    b = eng.generate(prompt, 96, SamplingParams(temperature=0.4, seed=5, forced_accept_p=0.7))
    assert a.tokens == b.tokens and a.rounds == b.rounds                 # bitwise reproducible
    assert 2.0 < len(a.tokens) / a.rounds < 4.5
    c = eng.generate(prompt, 96, SamplingParams(temperature=0.4, seed=6, forced_accept_p=0.7))
    assert c.tokens != a.tokens
    assert all(0 <= t < spec.vocab for t in a.tokens)


def test_speculative_equals_target_greedy():
    """With a one-token nucleus the committed sequence must equal plain greedy decoding of the
    target (every position rejected -> one verified token per round), whatever the draft proposes."""
    from naivert_b200.models.spec import SamplingParams
    spec, eng = _engine(layers=3)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, spec.vocab - 16, (50,), generator=g)
    greedy = eng.generate(prompt, 40, SamplingParams(temperature=1.0, top_p=1e-6, seed=9, forced_accept_p=0.0))
    spec_run = eng.generate(prompt, 40, SamplingParams(temperature=1.0, top_p=1e-6, seed=9))
    assert spec_run.tokens == greedy.tokens
    eager = eng.generate(prompt, 40, SamplingParams(temperature=1.0, top_p=1e-6, seed=9), use_graphs=False)
    assert eager.tokens == greedy.tokens                                  # graph replay == eager launches


def test_stop_on_eos_and_cancel():
    from naivert_b200.models.spec import SamplingParams
    spec, eng = _engine()
    prompt = torch.arange(20)
    base = eng.generate(prompt, 32, SamplingParams(temperature=0.4, seed=2, forced_accept_p=0.7))
    eos = base.tokens[10]
    eng.round.stop_ids[0] = eos
    cut = eng.generate(prompt, 32, SamplingParams(temperature=0.4, seed=2, forced_accept_p=0.7))
    first = base.tokens.index(eos)
    assert cut.stop_reason == "eos" and cut.tokens == base.tokens[:first + 1]
    eng.round.stop_ids[0] = spec.stop_token_ids[0]
    eng.open(prompt, 512, SamplingParams(temperature=0.4, seed=2, forced_accept_p=0.7))
    recs = []
    for i, rec in enumerate(eng.stream_rounds(ahead=2)):
        recs.append(rec)
        if i == 3:
            eng.round.cancel()
    assert recs[-1].stop_reason == "cancelled" and len(recs) < 40


def test_session_prefix_reuse_is_bitwise_identical():
    """A parked session prefix resumed by a longer prompt gives exactly the tokens of a cold run."""
    from naivert_b200.models.spec import SamplingParams
    from naivert_b200.runtime.session_engine import SessionEngine
    spec, eng = _engine(layers=3, capacity=2048)
    se = SessionEngine(eng, store_gb=1.0)
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, spec.vocab - 16, (300,), generator=g).tolist()     # beyond top_k = 256: sparse path
    sp = SamplingParams(temperature=0.7, seed=21)

    def run(engine, toks, sid, n=48):
        s = engine.open_session(toks, n, sid, sp)
        out = []
        while not s.done:
            out += s.step(30)
        stats = s.finish()
        return s, out, stats

    s1, out1, st1 = run(se, prompt, "conv")
    assert s1.cached_tokens == 0 and len(out1) == 48 and st1["segments"]["total"]["tokens"] == 48
    follow = prompt + out1 + torch.randint(0, spec.vocab - 16, (25,), generator=g).tolist()
    s2, out2, _ = run(se, follow, "conv")
    assert s2.cached_tokens >= 300, s2.prefill_info
    s3, out3, _ = run(se, follow, "conv")                       # same prompt again: resumes from its own checkpoint/park
    _, cold_eng = _engine(layers=3, capacity=2048)
    cold = SessionEngine(cold_eng, store_gb=1.0)
    _, out_cold, _ = run(cold, follow, None)
    assert out2 == out_cold and out3 == out_cold
    # a branch that diverges inside the first prompt falls back to the ring checkpoint or a cold start
    branch = prompt[:280] + [5, 6, 7, 8, 9] * 8
    s4, out4, _ = run(se, branch, "conv")
    _, out4_cold, _ = run(cold, branch, None)
    assert out4 == out4_cold
    assert se.store.bytes() > 0 and any("#" in k for k in se.store.entries) or len(se.store.entries) >= 1


def test_device_chain_matches_host_launched_rounds():
    """The self-relaunching graph (one host launch per request) commits exactly the tokens of host-launched rounds."""
    from naivert_b200.models.naive_n0p5 import small_w8a8_spec
    from naivert_b200.models.spec import SamplingParams
    from naivert_b200.runtime.engine import Engine
    spec = small_w8a8_spec(2)
    host = Engine.build(spec, capacity=1024, seed=0)
    chain = Engine.build(spec, capacity=1024, seed=0, device_chain=True)
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, spec.vocab - 16, (41,), generator=g)
    sp = SamplingParams(temperature=0.6, seed=3)
    a = host.generate(prompt, 200, sp)
    b = chain.generate(prompt, 200, sp)
    assert a.tokens == b.tokens and b.stop_reason == "output_limit"
    assert chain.round.host_launches == 1 and host.round.host_launches > 10
    info = chain.round.native_graph.info
    assert info["kernel_nodes"] == info["nodes"] and info["kernel_nodes"] > 20
    c = chain.generate(prompt, 64, sp)                      # a second request restarts the chain
    assert c.tokens == a.tokens[:64]


def test_round_graph_carries_programmatic_edges():
    """With programmatic dependent launch on, the captured round graph holds one programmatic edge per kernel-to-kernel
    dependency (they come from the launch attribute, nothing rewrites the graph afterwards), the plain capture holds
    none, and both commit the same tokens."""
    from naivert_b200.models.naive_n0p5 import small_w8a8_spec
    from naivert_b200.models.spec import SamplingParams
    from naivert_b200.runtime.engine import Engine
    spec = small_w8a8_spec(2)
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, spec.vocab - 16, (41,), generator=g)
    sp = SamplingParams(temperature=0.6, seed=3)
    toks, infos = [], []
    for pdl in (False, True):
        eng = Engine.build(spec, capacity=1024, seed=0, device_chain=True, pdl=pdl)
        try:
            toks.append(eng.generate(prompt, 96, sp).tokens)
            infos.append(eng.round.native_graph.info)
        finally:
            eng.close()
    assert toks[0] == toks[1]
    plain, prog = infos
    assert plain["programmatic_edges"] == 0 and plain["kernel_nodes"] == prog["kernel_nodes"]
    # every kernel but the first and the relaunch node (an ordinary launch) hangs on a programmatic edge
    assert prog["programmatic_edges"] >= prog["kernel_nodes"] - 2, prog
