"""Plain-PyTorch statement of the routing layout that the dispatch kernels compute on the GPU.

The layout is deterministic by construction (no arrival-order atomics), so this file is both the CPU
backend's implementation and the bitwise oracle for the CUDA kernels.

Definitions (experts are block-partitioned: ``rank(e) = e // (E / R)``):

* non-expand layout: rank ``d`` receives one row per (source rank ``s``, token ``t``) that selected any of
  ``d``'s experts; rows are ordered by ``(s, t)``.
* expand layout: rank ``d`` receives one row per (token, selected local expert); rows are grouped by local
  expert, each group starts at a multiple of ``expert_alignment`` and is ordered by ``(s, t)``.
* ``lane_src[t, k]`` packs ``(dst_rank << 24) | row`` for top-k lane ``k`` (-1 when the lane is empty).
* ``plan[t, k]`` equals ``lane_src[t, k]`` on the lanes that actually move a row: every valid lane in expand
  layout, and in non-expand layout only the last lane of each distinct destination rank.  Dispatch sends one
  row per non-negative plan entry; combine accumulates the plan entries in lane order.

Parity: the counts, prefix sums and localised indices match what deep_ep computes in the notify warps of
deep_ep/include/deep_ep/impls/dispatch.cuh:79-258 and csrc/kernels/legacy/layout.cu:10-150; the explicit
row assignment replaces the atomic slot claim of dispatch.cuh:344-345.
"""
from dataclasses import dataclass
from typing import Optional

import torch

ROW_BITS = 24
ROW_MASK = (1 << ROW_BITS) - 1


def pack_lane(rank: torch.Tensor, row: torch.Tensor) -> torch.Tensor:
    return ((rank.to(torch.int64) << ROW_BITS) | row.to(torch.int64)).to(torch.int32)


def unpack_lane(packed: torch.Tensor):
    """-> (rank, row); both -1 where ``packed`` is negative."""
    p = packed.to(torch.int64)
    valid = p >= 0
    rank = torch.where(valid, p >> ROW_BITS, torch.full_like(p, -1))
    row = torch.where(valid, p & ROW_MASK, torch.full_like(p, -1))
    return rank, row


def align_up(x: torch.Tensor, a: int) -> torch.Tensor:
    return (x + a - 1) // a * a


@dataclass
class LocalLayout:
    """What one rank derives from its own ``topk_idx`` before talking to anyone."""
    lane_rank: torch.Tensor        # [T, K] int64, -1 for empty lanes
    lane_expert: torch.Tensor      # [T, K] int64 global expert id, -1 for empty lanes
    is_last_of_rank: torch.Tensor  # [T, K] bool
    master_lane: torch.Tensor      # [T, K] int64: last lane with the same destination rank
    rank_count: torch.Tensor       # [R] int64 tokens per destination rank (a token counts once per rank)
    expert_count: torch.Tensor     # [E] int64 selections per expert
    rank_pos: torch.Tensor         # [T, K] int64 index of token t among my tokens that reach lane_rank[t,k]
    expert_pos: torch.Tensor       # [T, K] int64 index of token t among my tokens that selected that expert
    is_token_in_rank: torch.Tensor  # [T, R] bool


def local_layout(topk_idx: torch.Tensor, num_experts: int, num_ranks: int) -> LocalLayout:
    T, K = topk_idx.shape
    dev = topk_idx.device
    idx = topk_idx.to(torch.int64)
    per_rank = num_experts // num_ranks
    valid = idx >= 0
    lane_rank = torch.where(valid, idx // per_rank, torch.full_like(idx, -1))

    # last lane of each distinct destination rank inside a token
    same = (lane_rank.unsqueeze(2) == lane_rank.unsqueeze(1)) & valid.unsqueeze(2) & valid.unsqueeze(1)   # [T,K,K]
    lanes = torch.arange(K, device=dev)
    later = lanes.view(1, 1, K) > lanes.view(1, K, 1)
    is_last = valid & ~(same & later).any(dim=2)
    master = torch.where(same, lanes.view(1, 1, K).expand(T, K, K), torch.full((1, 1, 1), -1, device=dev)).amax(dim=2)

    in_rank = torch.zeros(T, num_ranks + 1, dtype=torch.bool, device=dev)
    in_rank.scatter_(1, torch.where(valid, lane_rank, torch.full_like(lane_rank, num_ranks)), True)
    in_rank = in_rank[:, :num_ranks]
    rank_count = in_rank.sum(dim=0)
    rank_excl = torch.cumsum(in_rank.to(torch.int64), dim=0) - in_rank.to(torch.int64)       # [T, R]
    rank_pos = torch.gather(rank_excl, 1, lane_rank.clamp_min(0))
    rank_pos = torch.where(valid, rank_pos, torch.full_like(rank_pos, -1))

    sel = torch.zeros(T, num_experts + 1, dtype=torch.int64, device=dev)
    sel.scatter_add_(1, torch.where(valid, idx, torch.full_like(idx, num_experts)), torch.ones_like(idx))
    sel = sel[:, :num_experts]
    expert_count = sel.sum(dim=0)
    expert_excl = torch.cumsum(sel, dim=0) - sel
    expert_pos = torch.gather(expert_excl, 1, idx.clamp_min(0))
    expert_pos = torch.where(valid, expert_pos, torch.full_like(expert_pos, -1))
    return LocalLayout(lane_rank, torch.where(valid, idx, torch.full_like(idx, -1)), is_last, master, rank_count, expert_count, rank_pos, expert_pos, in_rank)


@dataclass
class GlobalLayout:
    """What a rank knows once every rank's counts were exchanged."""
    lane_src: torch.Tensor                 # [T, K] int32
    plan: torch.Tensor                     # [T, K] int32
    num_recv_tokens: int                   # rows this rank receives (deduplicated per rank)
    num_expanded_tokens: int               # rows of the expand layout (aligned), 0 in non-expand layout
    psum_recv_per_rank: torch.Tensor       # [R] int32 inclusive
    psum_recv_per_expert: torch.Tensor     # [E_local] int32 (see EPHandle docs for the two forms)
    recv_per_expert: torch.Tensor          # [E_local] int32 unaligned


def global_layout(local: LocalLayout, rank_counts: torch.Tensor, expert_counts: torch.Tensor, rank: int,
                  num_experts: int, do_expand: bool, expert_alignment: int) -> GlobalLayout:
    """``rank_counts [R, R]`` is (source, destination); ``expert_counts [R, E]`` is (source, expert)."""
    R = rank_counts.shape[0]
    per_rank = num_experts // R
    rank_counts = rank_counts.to(torch.int64)
    expert_counts = expert_counts.to(torch.int64)
    valid = local.lane_rank >= 0
    lane_rank = local.lane_rank.clamp_min(0)

    recv_from = rank_counts[:, rank]                          # [R] rows from each source
    psum_rank = torch.cumsum(recv_from, 0)
    totals = expert_counts.sum(dim=0).view(R, per_rank)       # [R, E_local] per destination rank
    a = max(1, expert_alignment)
    if do_expand:
        starts = torch.zeros_like(totals)
        ends = torch.zeros_like(totals)
        end_prev = torch.zeros(R, dtype=torch.int64, device=totals.device)
        for j in range(per_rank):
            starts[:, j] = align_up(end_prev, a)
            ends[:, j] = starts[:, j] + totals[:, j]
            end_prev = ends[:, j]
        before_me = expert_counts[:rank].sum(dim=0)           # [E] selections from lower source ranks
        e = local.lane_expert.clamp_min(0)
        row = starts.view(-1)[e] + before_me[e] + local.expert_pos
        psum_expert = ends[rank]
        num_expanded = int(align_up(ends[rank, -1], a).item()) if per_rank > 0 else 0
        plan_mask = valid
    else:
        base = torch.cumsum(rank_counts, 0) - rank_counts     # [R(src), R(dst)] rows of lower sources
        row = base[rank][lane_rank] + local.rank_pos
        psum_expert = torch.cumsum(align_up(totals[rank], a), 0)
        num_expanded = 0
        plan_mask = local.is_last_of_rank
    lane_src = torch.where(valid, pack_lane(lane_rank, row.clamp_min(0)), torch.full_like(row, -1).to(torch.int32))
    plan = torch.where(plan_mask, lane_src, torch.full_like(lane_src, -1))
    return GlobalLayout(lane_src.to(torch.int32), plan.to(torch.int32), int(psum_rank[-1].item()), num_expanded,
                        psum_rank.to(torch.int32), psum_expert.to(torch.int32), totals[rank].to(torch.int32))


def get_dispatch_layout_ref(topk_idx: torch.Tensor, num_experts: int, num_ranks: int):
    """(num_tokens_per_rank [R] int32, num_tokens_per_expert [E] int32, is_token_in_rank [T, R] bool)."""
    local = local_layout(topk_idx, num_experts, num_ranks)
    return local.rank_count.to(torch.int32), local.expert_count.to(torch.int32), local.is_token_in_rank


def localize_topk_idx(topk_idx: torch.Tensor, dst_rank: int, num_experts: int, num_ranks: int) -> torch.Tensor:
    """Expert ids relative to ``dst_rank``'s first expert; experts of other ranks become -1."""
    per_rank = num_experts // num_ranks
    lo = dst_rank * per_rank
    mask = (topk_idx >= lo) & (topk_idx < lo + per_rank)
    return torch.where(mask, topk_idx - lo, torch.full_like(topk_idx, -1))


def combine_ref(rows_of, plan: torch.Tensor, hidden: int, bias0: Optional[torch.Tensor] = None,
                bias1: Optional[torch.Tensor] = None, weights: Optional[torch.Tensor] = None,
                out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """fp32 reference of combine: start from ``bias0 + bias1`` (fp32), add the row of every non-negative
    plan entry in lane order (times ``weights[t, k]`` when given), round once to ``out_dtype`` (bf16 on the GPU).
    ``rows_of(rank) -> [rows, hidden]`` tensor of that rank's combine input."""
    T, K = plan.shape
    acc = torch.zeros(T, hidden, dtype=torch.float32)
    if bias0 is not None:
        acc += bias0.float().cpu()
    if bias1 is not None:
        acc += bias1.float().cpu()
    rank, row = unpack_lane(plan.cpu())
    for k in range(K):
        for r in rank[:, k].unique().tolist():
            if r < 0:
                continue
            m = rank[:, k] == r
            contrib = rows_of(int(r))[row[m, k]].float().cpu()
            if weights is not None:
                contrib = contrib * weights[m, k].float().cpu().unsqueeze(1)
            acc[m] += contrib
    return acc.to(out_dtype)
