"""Synthetic routing-score generators for tests and benchmarks.

Every generator returns ``scores [num_tokens, num_experts]`` (fp32); callers take ``topk`` of it.  Experts are
block-partitioned over ranks (``rank = expert // (num_experts // num_ranks)``).  Covers balanced routing, a
"hot rank" that receives ``ratio`` times the tokens of every other rank (exact-quota and score-scaled
flavours) and a Zipf skew over experts (parity: deep_ep/utils/gate.py:4-180).
"""
from typing import Optional

import torch


def _dev(device: Optional[torch.device]) -> torch.device:
    if device is not None:
        return torch.device(device)
    return torch.device('cuda') if torch.cuda.is_available() else torch.device('cpu')


def get_balanced_scores(num_tokens: int, num_experts: int, device=None, generator=None) -> torch.Tensor:
    """Uniform random scores: every expert is equally likely to be in the top-k."""
    return torch.rand(num_tokens, num_experts, device=_dev(device), generator=generator)


def get_scores_by_factor(num_tokens: int, num_experts: int, num_ranks: int, factor: float,
                         device=None, generator=None) -> torch.Tensor:
    """Uniform scores with rank 0's experts stretched to ``[0, factor)`` so they win the top-k more often."""
    per_rank = num_experts // num_ranks
    scores = torch.rand(num_tokens, num_experts, device=_dev(device), generator=generator)
    scores[:, :per_rank] *= factor
    return scores


def rank_hit_counts(topk_idx: torch.Tensor, num_experts: int, num_ranks: int) -> torch.Tensor:
    """Number of tokens that reach each rank (a token counts once per rank)."""
    per_rank = num_experts // num_ranks
    ranks = torch.where(topk_idx >= 0, topk_idx // per_rank, torch.full_like(topk_idx, num_ranks))
    hit = torch.zeros(topk_idx.shape[0], num_ranks + 1, dtype=torch.bool, device=topk_idx.device)
    hit.scatter_(1, ranks, True)
    return hit[:, :num_ranks].sum(dim=0)


def map_unbalanced_ratio_to_factor(num_tokens: int, num_experts: int, num_ranks: int, num_topk: int,
                                   ratio: float, device=None, iterations: int = 20) -> float:
    """Bisect the stretch factor of :func:`get_scores_by_factor` until rank 0 receives ``ratio`` times the
    mean of the other ranks."""
    lo, hi = 1.0, 100.0
    for _ in range(iterations):
        mid = (lo + hi) / 2
        scores = get_scores_by_factor(max(num_tokens, 1024), num_experts, num_ranks, mid, device)
        counts = rank_hit_counts(scores.topk(num_topk, dim=-1).indices, num_experts, num_ranks).float()
        if counts[0].item() > counts[1:].mean().item() * ratio:
            hi = mid
        else:
            lo = mid
    return lo


def get_random_unbalanced_scores(num_tokens: int, num_experts: int, num_ranks: int, num_topk: int,
                                 ratio: float, device=None) -> torch.Tensor:
    factor = 1.0 if ratio == 1.0 or num_ranks == 1 else \
        map_unbalanced_ratio_to_factor(num_tokens, num_experts, num_ranks, num_topk, ratio, device)
    return get_scores_by_factor(num_tokens, num_experts, num_ranks, factor, device)


def get_precise_unbalanced_scores(num_tokens: int, num_experts: int, num_ranks: int, num_topk: int,
                                  ratio: float, device=None) -> torch.Tensor:
    """Exact-quota construction: every token reaches exactly ``m`` ranks; rank 0 is among them for a fixed
    quota of tokens chosen so that its token count is ``ratio`` times that of each other rank, and the other
    ranks are dealt round-robin so their counts differ by at most one."""
    dev = _dev(device)
    per_rank = num_experts // num_ranks
    assert ratio >= 1.0
    if num_ranks == 1:
        return torch.rand(num_tokens, num_experts, device=dev)
    others = num_ranks - 1
    m_min = max(1, -(-num_topk // per_rank))
    m_max = min(num_topk, num_ranks, int(others / ratio) + 1)
    assert m_min <= m_max, 'ratio not reachable with this expert/top-k shape'
    m = m_max
    total = num_tokens * m
    hot = min(num_tokens, int(round(total * ratio / (others + ratio))))
    hot_tokens = torch.randperm(num_tokens, device=dev)[:hot]
    is_hot = torch.zeros(num_tokens, dtype=torch.bool, device=dev)
    is_hot[hot_tokens] = True
    need = torch.where(is_hot, m - 1, m)                       # non-hot ranks per token
    start = torch.cumsum(need, 0) - need                        # round-robin deal over ranks 1..R-1
    cols = torch.arange(m, device=dev).unsqueeze(0)
    dealt = (start.unsqueeze(1) + cols) % others + 1
    member = torch.zeros(num_tokens, num_ranks, dtype=torch.bool, device=dev)
    valid = cols < need.unsqueeze(1)
    member.scatter_(1, torch.where(valid, dealt, torch.zeros_like(dealt)), valid)
    member[:, 0] = is_hot
    # spread top-k slots over the member ranks: one each, the remainder round-robin
    member_rank = torch.argsort(member.int(), dim=1, descending=True, stable=True)[:, :m]   # [T, m]
    n_members = member.sum(1, keepdim=True)
    slot_rank = torch.gather(member_rank, 1, torch.arange(num_topk, device=dev).unsqueeze(0) % n_members)
    per_rank_slots = torch.zeros(num_tokens, num_ranks, dtype=torch.long, device=dev)
    per_rank_slots.scatter_add_(1, slot_rank, torch.ones_like(slot_rank))
    scores = torch.rand(num_tokens, num_experts, device=dev) * 0.9
    order = torch.argsort(torch.rand(num_tokens, num_ranks, per_rank, device=dev), dim=-1)
    chosen = order < per_rank_slots.unsqueeze(-1)
    boost = 0.9 + 0.1 * torch.rand(num_tokens, num_ranks, per_rank, device=dev).clamp_min(1e-6)
    return torch.where(chosen, boost, scores.view(num_tokens, num_ranks, per_rank)).view(num_tokens, num_experts)


def get_unbalanced_scores(num_tokens: int, num_experts: int, num_ranks: int, num_topk: int, ratio: float,
                          precise: bool, device=None) -> torch.Tensor:
    fn = get_precise_unbalanced_scores if precise else get_random_unbalanced_scores
    return fn(num_tokens, num_experts, num_ranks, num_topk, ratio, device)


def get_zipf_scores(num_tokens: int, num_experts: int, s: float = 1.2, device=None, generator=None) -> torch.Tensor:
    """Gumbel-perturbed log-probabilities of a Zipf(s) law over experts: ``topk`` of the result samples
    ``k`` experts without replacement with probability proportional to ``rank^-s``."""
    dev = _dev(device)
    logp = -s * torch.log(torch.arange(1, num_experts + 1, device=dev, dtype=torch.float32))
    u = torch.rand(num_tokens, num_experts, device=dev, generator=generator).clamp_min(1e-20)
    return logp.unsqueeze(0) - torch.log(-torch.log(u))
