"""CPU checks of the sampler oracle: Philox matches the C implementation, nucleus and draws."""
import os

import pytest
import torch

from naivert_b200.ops import sampling_ref as S


def test_philox_known_properties():
    u = [S.philox_uniform(1234, d, a, b) for d in range(3) for a in range(4) for b in range(4)]
    assert all(0.0 < x < 1.0 for x in u)
    assert len(set(u)) == len(u)
    assert S.philox_uniform(1234, 0, 1, 2) == S.philox_uniform(1234, 0, 1, 2)
    assert abs(sum(S.philox_uniform(7, 0, 0, i) for i in range(4000)) / 4000 - 0.5) < 0.03


def test_philox_matches_native_library():
    from naivert_b200.ops import build
    if not os.path.isfile(os.path.join(build.LIB_DIR, build.LIB_NAME)):
        pytest.skip("kernel library not built")
    from naivert_b200.ops import kernels as K
    try:
        K.aux_lib()
    except OSError:
        pytest.skip("kernel library needs the CUDA runtime")
    for args in [(1234, 0, 1, 2), (2 ** 40 + 17, 3, 99, 152575), (0, 2, 0, 0)]:
        assert abs(K.philox_uniform(*args) - S.philox_uniform(*args)) < 1e-9


def test_nucleus_and_draw():
    z = torch.tensor([0.0, 1.0, 2.0, 3.0, -50.0])
    e = S.codes(z, 1.0)
    tau, Z = S.nucleus(e, 0.6)
    assert tau == int(e[3]) and Z == int(e[3])            # the top token alone holds 64 %
    tau, Z = S.nucleus(e, 0.7)
    assert tau == int(e[2]) and Z == int(e[2] + e[3])
    tau, Z = S.nucleus(e, 1.0 - 2 ** -20)
    assert Z >= int(e[:4].sum())
    mass = torch.tensor([0, 5, 0, 5])
    assert S.draw(mass, 0.0) == 1 and S.draw(mass, 0.49) == 1 and S.draw(mass, 0.5) == 3 and S.draw(mass, 0.999) == 3


def test_verify_oracle_forced_and_greedy():
    g = torch.Generator().manual_seed(0)
    zp, zq = torch.randn(8, 512, generator=g) * 3, torch.randn(7, 512, generator=g) * 3
    ids = [5] + [int(zp[j].argmax()) for j in range(7)]          # proposals equal the target arg-max
    m, tok, _, _ = S.verify_oracle(zp, zq, ids, 1.0, 1e-6, seed=1, rnd=0)
    assert m == 7 and tok == int(zp[7].argmax())                 # greedy nucleus accepts all, bonus = arg-max
    ids[3] = (ids[3] + 1) % 512
    m, tok, _, _ = S.verify_oracle(zp, zq, ids, 1.0, 1e-6, seed=1, rnd=0)
    assert m == 2 and tok == int(zp[2].argmax())
    m, _, _, _ = S.verify_oracle(zp, zq, ids, 1.0, 0.95, seed=1, rnd=0, forced=1.0)
    assert m == 7
    m, _, _, _ = S.verify_oracle(zp, zq, ids, 1.0, 0.95, seed=1, rnd=0, forced=0.0)
    assert m == 0
    counts = [S.verify_oracle(zp, zq, ids, 1.0, 0.95, seed=1, rnd=r, forced=0.7)[0] for r in range(300)]
    assert 1.7 < sum(counts) / 300 < 2.6                         # E[accepted] = sum 0.7^k ~ 2.14
