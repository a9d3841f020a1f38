"""FP8 (e4m3) quantisation recipes and their torch oracles.

* ``quantize_fp8_block`` / ``dequant_block``: 128x128 block-scaled weights with an
  fp32 ``weight_scale_inv`` per block (the checkpoint format; reference
  naivert/models/naive_n0p5/checkpoint_fp8.py:50-66,174-184).
* ``quantize_act_pow2``: the W8A8 activation recipe - e4m3 round-to-nearest with one
  power-of-two scale per 128-wide K block, the smallest 2^e >= amax/448, zero block -> 1
  (reference naivert/common/block128_activation.cuh:9-33 and
  naivert/models/naive_n0p5/training_moe.py:16).
* ``quantize_rows_e4m3``: per-row amax/448 scale used for the indexer key cache
  (reference tests/gpu/attn_dsa/run_attn_dsa.py ``quantize_e4m3_rows``).
"""
from __future__ import annotations

import torch

E4M3_MAX = 448.0
BLOCK = 128


def _pad_to(x: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    if x.shape[-2] == rows and x.shape[-1] == cols:
        return x
    out = x.new_zeros(*x.shape[:-2], rows, cols)
    out[..., : x.shape[-2], : x.shape[-1]] = x
    return out


def quantize_fp8_block(w: torch.Tensor, block: int = BLOCK):
    """[N, K] float -> (e4m3 [N, K], fp32 scale_inv [ceil(N/b), ceil(K/b)]); w ~= w8 * scale_inv."""
    n, k = w.shape[-2:]
    nb, kb = -(-n // block), -(-k // block)
    wf = _pad_to(w.float(), nb * block, kb * block)
    tiles = wf.reshape(*w.shape[:-2], nb, block, kb, block)
    amax = tiles.abs().amax(dim=(-3, -1))
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (tiles / scale[..., :, None, :, None]).reshape(*w.shape[:-2], nb * block, kb * block)
    q = q[..., :n, :k].to(torch.float8_e4m3fn)
    return q, scale.contiguous()


def dequant_block(w8: torch.Tensor, scale_inv: torch.Tensor, block: int = BLOCK) -> torch.Tensor:
    n, k = w8.shape[-2:]
    s = scale_inv.repeat_interleave(block, dim=-2).repeat_interleave(block, dim=-1)[..., :n, :k]
    return w8.float() * s


def pow2_scale(amax: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= amax/448 (exact exponent arithmetic); 1 where amax == 0."""
    t = (amax.float() / E4M3_MAX)
    m, e = torch.frexp(t)                       # t = m * 2^e, m in [0.5, 1)
    e = torch.where(m == 0.5, e - 1, e)         # exact powers of two keep their exponent
    s = torch.ldexp(torch.ones_like(t), e)
    return torch.where(amax > 0, s, torch.ones_like(s))


def quantize_act_pow2(x: torch.Tensor, block: int = BLOCK):
    """[..., K] -> (e4m3 [..., K], fp32 scale [..., K/block]); x ~= x8 * scale (per K block)."""
    k = x.shape[-1]
    if k % block:
        raise ValueError(f"K={k} is not a multiple of {block}")
    xb = x.float().reshape(*x.shape[:-1], k // block, block)
    s = pow2_scale(xb.abs().amax(dim=-1))
    q = (xb / s[..., None]).reshape(x.shape).to(torch.float8_e4m3fn)
    return q, s


def dequant_act(x8: torch.Tensor, scale: torch.Tensor, block: int = BLOCK) -> torch.Tensor:
    return (x8.float().reshape(*x8.shape[:-1], -1, block) * scale[..., None]).reshape(x8.shape)


def quantize_rows_e4m3(x: torch.Tensor):
    """Per-row scale amax/448: returns (e4m3 rows, fp32 scale[rows])."""
    amax = x.float().abs().amax(dim=-1)
    s = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    return (x.float() / s[..., None]).to(torch.float8_e4m3fn), s


def w8a8_linear_ref(x: torch.Tensor, w8: torch.Tensor, w_scale: torch.Tensor,
                    block: int = BLOCK) -> torch.Tensor:
    """Oracle of the block-scaled GEMM: y[m, n] = sum_kb (x8[m,kb,:] . w8[n,kb,:]) * xs[m,kb] * ws[n/b,kb]
    with fp32 accumulation inside a K block and fp32 promotion across K blocks in ascending order."""
    x8, xs = quantize_act_pow2(x, block)
    m, k = x8.shape
    n = w8.shape[0]
    kb = k // block
    xa = x8.float().reshape(m, kb, block)
    wa = w8.float().reshape(n, kb, block)
    ws = w_scale.repeat_interleave(block, dim=0)[:n]          # [n, kb]
    out = torch.zeros(m, n, dtype=torch.float32, device=x.device)
    for b in range(kb):
        part = xa[:, b] @ wa[:, b].T                           # exact products, fp32 accumulate
        out = out + part * (xs[:, b, None] * ws[None, :, b])
    return out


# --------------------------------------------------------------------------- power-of-two (UE8M0) scale variants
def ue8m0_round_up(scale: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= scale (the exponent-only 'UE8M0' scale format); zeros map to one."""
    s = scale.float()
    m, e = torch.frexp(s)                       # s = m * 2^e, m in [0.5, 1)
    e = torch.where(m == 0.5, e - 1, e)
    out = torch.ldexp(torch.ones_like(s), e)
    return torch.where(s > 0, out, torch.ones_like(s))


def requant_block_ue8m0(w8: torch.Tensor, scale_inv: torch.Tensor, block: int = BLOCK):
    """Re-express block-scaled e4m3 weights with power-of-two block scales: dequantise, round every block
    scale up to a power of two, quantise again.  Values change by at most one e4m3 rounding.
    Parity: the UE8M0 re-quantisation of expert weights in naivert/kernels/naive_n0p5/prefill.py."""
    w = dequant_block(w8, scale_inv, block)
    s2 = ue8m0_round_up(scale_inv)
    n, k = w.shape[-2], w.shape[-1]
    sf = s2.repeat_interleave(block, -2)[..., :n, :].repeat_interleave(block, -1)[..., :k]
    return (w / sf).clamp(-448, 448).to(torch.float8_e4m3fn), s2


def quantize_mxfp8(x: torch.Tensor, group: int = 32):
    """MX-style e4m3: one power-of-two scale per ``group`` consecutive elements of the last dimension.
    Returns (e4m3 tensor, scales [..., K / group]).  Parity: the mxfp8 packers of naivert/kernels/packing.py."""
    xf = x.float()
    k = xf.shape[-1]
    if k % group:
        raise ValueError(f"last dimension {k} is not a multiple of {group}")
    g = xf.reshape(*xf.shape[:-1], k // group, group)
    s = pow2_scale(g.abs().amax(-1))
    q = (g / s.unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q.reshape(xf.shape), s


def dequant_mxfp8(q: torch.Tensor, s: torch.Tensor, group: int = 32) -> torch.Tensor:
    k = q.shape[-1]
    return (q.float().reshape(*q.shape[:-1], k // group, group) * s.unsqueeze(-1)).reshape(q.shape)
