"""Synthetic router outputs for tests and benchmarks (any device, seeded by the caller).

Generators return ``scores [tokens, experts]``; :func:`topk_from_scores` turns them into
``(topk_idx int64, topk_weights float32)`` with softmax-renormalised weights.

Parity: deep_ep/utils/gate.py:4-180 of the reference (balanced and unbalanced generators, which
are hard-wired to CUDA there) and the group-limited gating of tests/legacy/test_internode.py:42-47.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .math import create_grouped_scores


def get_balanced_scores(num_tokens: int, num_experts: int, device='cpu', generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """i.i.d. N(0, 1) logits: every expert is equally likely."""
    return torch.randn((num_tokens, num_experts), device=device, generator=generator)


def get_scores_by_factor(num_tokens: int, num_experts: int, num_ranks: int, factor: float, hot_rank: int = 0,
                         device='cpu', generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Positive scores where the experts of ``hot_rank`` are scaled by ``factor``."""
    scores = torch.rand((num_tokens, num_experts), device=device, generator=generator) + 1e-3
    per_rank = num_experts // num_ranks
    scores[:, hot_rank * per_rank:(hot_rank + 1) * per_rank] *= factor
    return scores


def measure_unbalanced_ratio(topk_idx: torch.Tensor, num_experts: int, num_ranks: int) -> float:
    """Traffic of the busiest rank over the mean of the others (token counted once per rank)."""
    per_rank = num_experts // num_ranks
    ranks = torch.where(topk_idx >= 0, topk_idx // per_rank, torch.full_like(topk_idx, -1))
    load = torch.stack([(ranks == r).any(dim=1).sum() for r in range(num_ranks)]).double()
    hot = load.max()
    rest = (load.sum() - hot) / max(num_ranks - 1, 1)
    return float(hot / rest.clamp(min=1))


def get_unbalanced_scores(num_tokens: int, num_experts: int, num_ranks: int, num_topk: int, ratio: float,
                          device='cpu', generator: Optional[torch.Generator] = None, iters: int = 12) -> torch.Tensor:
    """Scores whose top-k routing sends about ``ratio`` times more tokens to rank 0 than to the others.

    The multiplicative factor on rank 0's experts is found by bisection on the measured ratio.
    """
    assert ratio >= 1.0
    if ratio == 1.0 or num_ranks == 1:
        return torch.rand((num_tokens, num_experts), device=device, generator=generator)
    base = torch.rand((num_tokens, num_experts), device=device, generator=generator) + 1e-3
    per_rank = num_experts // num_ranks
    lo, hi = 1.0, 64.0
    for _ in range(iters):
        mid = (lo * hi) ** 0.5
        trial = base.clone()
        trial[:, :per_rank] *= mid
        got = measure_unbalanced_ratio(torch.topk(trial, num_topk, dim=1).indices, num_experts, num_ranks)
        lo, hi = (mid, hi) if got < ratio else (lo, mid)
    base[:, :per_rank] *= (lo * hi) ** 0.5
    return base


def get_zipf_scores(num_tokens: int, num_experts: int, s: float = 1.2, device='cpu',
                    generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Gumbel-perturbed log-popularity with Zipf(s) expert popularity (expert 0 the most popular)."""
    pop = torch.arange(1, num_experts + 1, device=device, dtype=torch.float32).pow(-s)
    u = torch.rand((num_tokens, num_experts), device=device, generator=generator).clamp_(1e-9, 1 - 1e-9)
    return pop.log().unsqueeze(0) - torch.log(-torch.log(u))


def topk_from_scores(scores: torch.Tensor, num_topk: int, num_groups: int = 0, num_topk_groups: int = 0,
                     masked_ratio: float = 0.0, generator: Optional[torch.Generator] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-k selection (optionally group-limited), softmax weights renormalised over the selection.

    ``masked_ratio`` randomly drops that share of the selections (index -1, weight 0).
    """
    if num_groups > 0 and num_topk_groups > 0:
        group_scores = scores.view(scores.size(0), num_groups, -1).amax(dim=-1)
        group_idx = torch.topk(group_scores, num_topk_groups, dim=-1, sorted=False).indices
        scores = create_grouped_scores(scores - scores.min() + 1e-6, group_idx, num_groups)
    vals, idx = torch.topk(scores, num_topk, dim=-1, largest=True, sorted=False)
    weights = torch.softmax(vals.float(), dim=-1)
    idx = idx.to(torch.int64)
    if masked_ratio > 0:
        drop = torch.rand(idx.shape, device=idx.device, generator=generator) < masked_ratio
        idx = idx.masked_fill(drop, -1)
        weights = weights.masked_fill(drop, 0.0)
    return idx, weights
