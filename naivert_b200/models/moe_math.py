"""Stand-alone MoE arithmetic of the W8A8 recipe, as small pure functions (CPU/torch oracle).

These are the pieces the kernels are tested against one by one: RMSNorm with bf16 rounding, sigmoid/softmax
routing with the selection bias, the e4m3 re-quantisation of the down-projection input, the probability-weighted
combine in ascending expert order, and the rank-order sum of bf16-rounded tensor-parallel partials.
Parity: naivert/models/naive_n0p5/training_moe.py:16-88 (``quantize_down_activation_reference``, ``rmsnorm``,
``route``, ``combine``, ``combine_tp_partials``).
"""
from __future__ import annotations

from typing import Sequence, Tuple

import torch

from ..ops.quant import dequant_act, quantize_act_pow2
from .spec import MoeRoutingSpec


def _bf16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).float()


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    """bf16(x * rsqrt(mean(x^2) + eps) * gamma), statistics in fp32."""
    xf = x.float()
    return _bf16(xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gamma.float())


def route(xn: torch.Tensor, router_w: torch.Tensor, router_b: torch.Tensor, rt: MoeRoutingSpec) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-k experts per row: (ids [rows, k] in selection order, probabilities [rows, k]).
    Sigmoid routing chooses by score + bias and weights by the unbiased score; ties go to the lowest id."""
    logits = xn.float() @ router_w.float().t()
    if rt.score_func == "sigmoid":
        score = torch.sigmoid(logits)
        choice = score + router_b.float()
    else:
        score = torch.softmax(logits, -1)
        choice = score
    # stable descending order: value desc, index asc
    order = torch.argsort(choice, dim=-1, descending=True, stable=True)
    ids = order[:, : rt.top_k]
    p = torch.gather(score, 1, ids)
    if rt.normalize_top_k:
        p = p / (p.sum(-1, keepdim=True) + 1e-20)
    return ids.int(), (p * rt.route_scale).float()


def quantize_down_activation(y: torch.Tensor) -> torch.Tensor:
    """SiLU(gate) * up as the down projection sees it: e4m3 with one power-of-two scale per 128 channels."""
    q, s = quantize_act_pow2(y.float())
    return dequant_act(q, s)


def combine(resid: torch.Tensor, expert_out: Sequence[torch.Tensor], ids: torch.Tensor, probs: torch.Tensor) -> torch.Tensor:
    """resid + sum over a row's experts in ascending expert id of p * out (fp32), one bf16 rounding.
    ``expert_out[e]`` is expert e's output for every row ([rows, hidden])."""
    acc = torch.zeros_like(resid, dtype=torch.float32)
    rows = resid.shape[0]
    for r in range(rows):
        pairs = sorted(zip(ids[r].tolist(), probs[r].tolist()))
        for e, p in pairs:
            acc[r] += p * expert_out[e][r].float()
    return (resid.float() + acc).to(torch.bfloat16)


def combine_tp_partials(resid: torch.Tensor, partials: Sequence[torch.Tensor]) -> torch.Tensor:
    """Tensor-parallel reduction of the step path: every rank's partial is rounded to bf16, the partials are
    added in rank order in fp32 on top of the residual, and the sum is rounded to bf16 once."""
    acc = resid.float().clone()
    for p in partials:
        acc += _bf16(p.float())
    return acc.to(torch.bfloat16)
