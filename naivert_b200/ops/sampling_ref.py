"""Torch/Python oracle of the integer-mass speculative sampler (same math as csrc/sampler.cu).

Distributions are 31-bit integer codes e = rint(exp(z/T - max) * 2^31); the nucleus is the
largest threshold tau with mass{e >= tau} >= top_p * total mass; accept iff u q'(d) < p'(d);
the rejected position draws from max(p' - q', 0) (from p' when that is empty) by inverse CDF
in vocabulary order over 40-bit fixed-point masses; a fully accepted block draws the bonus
token from p' of the last row.  Uniforms come from Philox4x32-10 keyed by the request seed.

Parity: the CPU sort/CDF oracles of the reference sampler benches
(tests/gpu/naive_n0p5_draft/sampling/) and naivert/body/dspark_sampling/random.cuh.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

DOM_ACCEPT, DOM_RESAMPLE, DOM_FORCED, DOM_DRAFT, DOM_ANCHOR = 0, 1, 2, 3, 4
_M0, _M1, _W0, _W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
_MASK = 0xFFFFFFFF


def philox_u32(seed: int, domain: int, a: int, b: int) -> int:
    c0, c1, c2, c3 = domain & _MASK, a & _MASK, b & _MASK, 0
    k0, k1 = seed & _MASK, (seed >> 32) & _MASK
    for _ in range(10):
        p0, p1 = _M0 * c0, _M1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & _MASK, p1 & _MASK, ((p0 >> 32) ^ c3 ^ k1) & _MASK, p0 & _MASK
        k0, k1 = (k0 + _W0) & _MASK, (k1 + _W1) & _MASK
    return c0


def philox_uniform(seed: int, domain: int, a: int, b: int) -> float:
    """Uniform in (0, 1) with 23 bits (+ 1/2), an exactly representable fp32 value."""
    return ((philox_u32(seed, domain, a, b) >> 9) + 0.5) / 8388608.0


def codes(z: torch.Tensor, inv_t: float) -> torch.Tensor:
    """Integer codes of one row (fp32 arithmetic on the tensor's device) as int64."""
    v = z.float() * torch.tensor(inv_t, dtype=torch.float32, device=z.device)
    e = torch.exp(v - v.max()) * 2147483648.0
    return torch.round(e).to(torch.int64)


def nucleus(e: torch.Tensor, top_p: float) -> Tuple[int, int]:
    """(tau, kept mass Z): largest tau with sum(e[e >= tau]) >= ceil(top_p * sum e)."""
    total = int(e.sum())
    target = math.ceil(float(torch.tensor(top_p, dtype=torch.float32)) * float(total))
    vals, _ = torch.sort(e, descending=True)
    cum = torch.cumsum(vals, 0)
    idx = int(torch.searchsorted(cum, torch.tensor(target, device=e.device)))
    idx = min(idx, e.numel() - 1)
    tau = int(vals[idx])
    return tau, int(e[e >= tau].sum())


def draw(mass: torch.Tensor, u: float) -> int:
    total = int(mass.sum())
    target = min(int(u * float(total)), total - 1)
    cum = torch.cumsum(mass, 0)
    return int(torch.searchsorted(cum, torch.tensor(target, device=mass.device), right=True))


def verify_oracle(zp: torch.Tensor, zq: torch.Tensor, block_ids: List[int], inv_t: float, top_p: float, seed: int,
                  rnd: int, forced: Optional[float] = None, inv_t_draft: Optional[float] = None):
    """zp [8, V] target logits, zq [7, V] draft logits; returns (accepted, extra_token, kept masses)."""
    inv_td = inv_t if inv_t_draft is None else inv_t_draft
    ep = [codes(zp[r], inv_t) for r in range(zp.shape[0])]
    eq = [codes(zq[r], inv_td) for r in range(zq.shape[0])]
    tp_ = [nucleus(e, top_p) for e in ep]
    tq_ = [nucleus(e, top_p) for e in eq]
    nq = zq.shape[0]
    m = 0
    while m < nq:
        tok = block_ids[m + 1]
        p = int(ep[m][tok]) if int(ep[m][tok]) >= tp_[m][0] else 0
        q = int(eq[m][tok]) if int(eq[m][tok]) >= tq_[m][0] else 0
        if forced is not None:
            acc = philox_uniform(seed, DOM_FORCED, rnd, m) < float(torch.tensor(forced, dtype=torch.float32))
        else:
            u = philox_uniform(seed, DOM_ACCEPT, rnd, m)
            acc = u * float(q) * float(tp_[m][1]) < float(p) * float(tq_[m][1])
        if not acc:
            break
        m += 1
    pk = torch.where(ep[m] >= tp_[m][0], ep[m], torch.zeros_like(ep[m]))
    if m < nq:
        qk = torch.where(eq[m] >= tq_[m][0], eq[m], torch.zeros_like(eq[m]))
        r = pk.double() / float(tp_[m][1]) - qk.double() / float(tq_[m][1])
        mass = torch.where(r > 0, (r * 1099511627776.0).to(torch.int64), torch.zeros_like(pk))
        if int(mass.sum()) == 0:
            mass = pk
    else:
        mass = pk
    u = philox_uniform(seed, DOM_RESAMPLE, rnd, m)
    return m, draw(mass, u), tp_, tq_
