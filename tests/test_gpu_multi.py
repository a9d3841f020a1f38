"""Tensor-parallel engine over the peer-memory fabric on 2+ GPUs (child processes via torchrun)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _free_port() -> int:
    """A rendezvous port nobody on this (shared) host listens on right now."""
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(n):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(os.path.dirname(__file__), "mp_tp_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    lines = [l for l in p.stdout.splitlines() if l.startswith("RESULT ")]
    assert p.returncode == 0 and lines, p.stdout[-2000:] + p.stderr[-4000:]
    return json.loads(lines[-1][7:])


@pytest.mark.parametrize("n", [2, 4, 8])
def test_tensor_parallel_engine(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    r = _run(n)
    assert r["status"] == 0
    assert r["residual_identical"] and r["lockstep"] and r["deterministic"] and r["spec_equals_greedy"], r
    assert r["verify_mean_rel"] < 0.08 and r["argmax_ok"] and r["sampler_matches_oracle"], r
    assert r["real_sampling_tokens"] == 64


def _run_worker(n, script, **extra_env):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", **extra_env)
    path = os.path.join(os.path.dirname(__file__), script)
    cmd = [sys.executable, path] if n == 1 else [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                                                 "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), path]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    lines = [l for l in p.stdout.splitlines() if l.startswith("RESULT ")]
    assert p.returncode == 0 and lines, p.stdout[-2000:] + p.stderr[-4000:]
    return json.loads(lines[-1][7:])


def test_device_chain_pauses_by_rank_consensus():
    """TP2 self-relaunching rounds with a 32-record ring and one lagging host: the chains pause together (the pause
    is max-reduced over the ranks in the tail kernel), are restarted by their hosts and commit the host-launched tokens."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    r = _run_worker(2, "mp_chain_worker.py")
    assert r["status"] == 0 and r["tokens_match_host_rounds"] and r["lockstep"], r
    assert min(r["host_launches"]) >= 2 and max(r["host_launches"]) < 40, r


@pytest.mark.parametrize("n", [1, 2])
def test_expert_parallel_all_to_all(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    r = _run_worker(n, "mp_ep_worker.py")
    assert r["status"] == 0 and r["repeat_identical"], r
    assert r.get("worst_err", r["max_rel_err"]) < 0.02 and r["wide_err"] < 0.02, r
    assert r["wide_identical"], r                       # the 64-column chunk engine adds in the same order
    assert r["layout_ok"], r                            # segments / work list / rows as the host restatement predicts
    assert r.get("total_rows", r["rows"]) == 96 * 4 * n


@pytest.mark.parametrize("n,exact", [(1, True), (1, False), (2, False)])
def test_native_prefill_matches_replay(n, exact):
    """Chunked prefill (TP attention; EP experts at n > 1) leaves the caches the eight-row replay leaves.
    ``exact``: the chunk path runs the row attention kernel instead of the grouped-head one.  The step path sums the
    squares of a row per 128-feature tile and runs its attention on tensor cores, so the two paths agree to
    rounding, not bit for bit."""
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    r = _run_worker(n, "mp_prefill_worker.py", NAIVERT_PREFILL_GROUP_ATTN="0" if exact else "1")
    assert r["status"] == 0 and r["repeat_identical"], r
    assert r["prefill"]["path"] == "native" and r["prefill"]["native_rows"] >= 672, r
    if exact:
        assert r["worst"] < 0.08, r
    if n > 1:
        assert r["lockstep"], r
    assert r["worst"] < 0.1, r
    assert r["token_prefix_agreement"] >= 1, r


def test_native_prefill_is_bitwise_equal_to_the_unfused_replay():
    """Against the step path built from separate kernels (full-row RMSNorm, row attention, no K split) the chunk
    path with the row attention kernel reproduces the first layers' caches bit for bit: both add in the same order."""
    r = _run_worker(1, "mp_prefill_worker.py", NAIVERT_PREFILL_GROUP_ATTN="0", NAIVERT_LEGACY_STEP="1")
    assert r["status"] == 0 and r["repeat_identical"], r
    assert {"L0.k", "L0.v", "L0.ik", "L0.iks", "L1.k", "L1.v"} <= set(r["bitwise"]), r
    assert r["worst"] < 0.03 and r["token_prefix_agreement"] >= 4, r


def test_native_prefill_tensor_parallel_experts():
    """Without expert-parallel weight copies every rank runs all rows through its slice of every expert and the
    partial sums are all-reduced (the path bench.py uses for its prompt)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    r = _run_worker(2, "mp_prefill_worker.py", PREFILL_MOE="tp")
    assert r["moe"] == "tp" and r["status"] == 0 and r["repeat_identical"] and r["lockstep"], r
    assert r["prefill"]["path"] == "native" and r["worst"] < 0.1 and r["token_prefix_agreement"] >= 1, r
