"""Oracles for dispatch / combine.

* ``dispatch_all`` / ``combine_all``: single-process oracles that take EVERY rank's inputs (lists indexed by rank)
  and return every rank's expected outputs; used with the emulated multi-rank world and in CPU tests.
* ``dispatch_nccl`` / ``combine_nccl``: distributed oracles built only from ``torch.distributed`` collectives
  (``all_to_all_single``), used as the correctness reference and timing baseline of multi-process runs
  (parity: deep_ep/utils/refs.py:10-243).
"""
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import layout_ref


def _cpu(t):
    return None if t is None else t.detach().cpu()


def dispatch_all(xs: Sequence[torch.Tensor], sfs: Optional[Sequence[Optional[torch.Tensor]]], topk_idxs: Sequence[torch.Tensor],
                 topk_ws: Optional[Sequence[Optional[torch.Tensor]]], num_experts: int, num_max_tokens: int,
                 do_expand: bool = False, expert_alignment: int = 1):
    """-> per rank dict(x, sf, idx, w, meta, layout(GlobalLayout))."""
    R = len(xs)
    xs = [_cpu(x) for x in xs]
    sfs = [_cpu(s) for s in sfs] if sfs is not None else [None] * R
    idxs = [_cpu(i) for i in topk_idxs]
    ws = [_cpu(w) for w in topk_ws] if topk_ws is not None else [None] * R
    locals_ = [layout_ref.local_layout(idxs[r], num_experts, R) for r in range(R)]
    rank_counts = torch.stack([l.rank_count for l in locals_])
    expert_counts = torch.stack([l.expert_count for l in locals_])
    gls = [layout_ref.global_layout(locals_[r], rank_counts, expert_counts, r, num_experts, do_expand, expert_alignment)
           for r in range(R)]
    outs = []
    for d in range(R):
        rows = gls[d].num_expanded_tokens if do_expand else gls[d].num_recv_tokens
        K = idxs[0].shape[1]
        H = xs[0].shape[1]
        o = {
            'x': torch.zeros((rows, H), dtype=xs[0].dtype), 'idx': None if do_expand else torch.full((rows, K), -1, dtype=idxs[0].dtype),
            'sf': None if sfs[0] is None else torch.zeros((rows, sfs[0].shape[1]), dtype=torch.float32),
            'w': None if ws[0] is None else (torch.zeros((rows,)) if do_expand else torch.zeros((rows, K))),
            'meta': torch.zeros((rows, 2), dtype=torch.int32), 'valid': torch.zeros((rows,), dtype=torch.bool), 'layout': gls[d]}
        outs.append(o)
    for s in range(R):
        rank, row = layout_ref.unpack_lane(gls[s].plan)
        K = idxs[s].shape[1]
        t_idx, k_idx = torch.nonzero(rank >= 0, as_tuple=True)
        for t, k in zip(t_idx.tolist(), k_idx.tolist()):
            d, rw = int(rank[t, k]), int(row[t, k])
            o = outs[d]
            assert not o['valid'][rw], 'two senders were assigned the same row'
            o['valid'][rw] = True
            if o['x'].dtype == torch.float8_e4m3fn:
                o['x'].view(torch.uint8)[rw] = xs[s].view(torch.uint8)[t]
            else:
                o['x'][rw] = xs[s][t]
            if o['sf'] is not None:
                o['sf'][rw] = sfs[s][t]
            if o['idx'] is not None:
                o['idx'][rw] = layout_ref.localize_topk_idx(idxs[s][t], d, num_experts, R)
            if o['w'] is not None:
                if do_expand:
                    o['w'][rw] = ws[s][t, k]
                else:
                    o['w'][rw] = ws[s][t]
            o['meta'][rw, 0] = s * num_max_tokens + t
            o['meta'][rw, 1] = s * K + k
    return outs


def combine_all(ys: Sequence[torch.Tensor], layouts: Sequence[layout_ref.GlobalLayout], hidden: int,
                bias0: Optional[Sequence] = None, bias1: Optional[Sequence] = None,
                mul_weights: Optional[Sequence] = None) -> List[torch.Tensor]:
    """ys[d] = rank d's combine input rows; -> per rank combined bf16 [T, H]."""
    R = len(ys)
    ys = [_cpu(y) for y in ys]
    return [layout_ref.combine_ref(lambda r: ys[r], layouts[r].plan, hidden,
                                   None if bias0 is None else bias0[r], None if bias1 is None else bias1[r],
                                   None if mul_weights is None else mul_weights[r]) for r in range(R)]


# --------------------------------------------------------------------------------------------- distributed oracles
def dispatch_nccl(x, topk_idx: torch.Tensor, topk_weights: Optional[torch.Tensor], num_max_tokens_per_rank: int,
                  num_experts: int, group: Optional[dist.ProcessGroup] = None):
    """Non-expand dispatch with only torch.distributed collectives; rows ordered by (source rank, token).
    Returns ``(recv_x | (recv_x, recv_sf), recv_topk_idx, recv_topk_weights, recv_src_token_idx, recv_counts)``."""
    rank, R = dist.get_rank(group), dist.get_world_size(group)
    use_fp8 = isinstance(x, tuple)
    x, sf = x if use_fp8 else (x, None)
    per_rank = num_experts // R
    dest = torch.where(topk_idx >= 0, topk_idx // per_rank, torch.full_like(topk_idx, -1))
    send_tok, send_counts = [], []
    for d in range(R):
        tok = (dest == d).any(dim=1).nonzero(as_tuple=True)[0]
        send_tok.append(tok)
        send_counts.append(tok.numel())
    order = torch.cat(send_tok)
    send_counts_t = torch.tensor(send_counts, dtype=torch.int64, device=x.device)
    recv_counts_t = torch.empty_like(send_counts_t)
    dist.all_to_all_single(recv_counts_t, send_counts_t, group=group)
    recv_counts = recv_counts_t.tolist()
    total = sum(recv_counts)

    def exchange(t: torch.Tensor) -> torch.Tensor:
        payload = t[order].contiguous()
        as_u8 = payload.dtype == torch.float8_e4m3fn
        if as_u8:
            payload = payload.view(torch.uint8)
        out = torch.empty((total,) + tuple(payload.shape[1:]), dtype=payload.dtype, device=payload.device)
        dist.all_to_all_single(out, payload, recv_counts, send_counts, group=group)
        return out.view(torch.float8_e4m3fn) if as_u8 else out
    recv_x = exchange(x)
    recv_sf = exchange(sf) if use_fp8 else None
    recv_idx = exchange(topk_idx)
    recv_w = exchange(topk_weights) if topk_weights is not None else None
    src = exchange((torch.arange(x.shape[0], device=x.device, dtype=torch.int32) + rank * num_max_tokens_per_rank).unsqueeze(1)).squeeze(1)
    lo = rank * per_rank
    mask = (recv_idx >= lo) & (recv_idx < lo + per_rank)
    recv_idx = torch.where(mask, recv_idx - lo, torch.full_like(recv_idx, -1))
    return ((recv_x, recv_sf) if use_fp8 else recv_x), recv_idx, recv_w, src, recv_counts_t.to(torch.int32)


def generate_pre_combine_data(src_token_global_idx: torch.Tensor, num_rows_total: int, hidden: int, seed: int = 0) -> torch.Tensor:
    """Deterministic bf16 rows that depend only on the source token id, so any rank can regenerate them."""
    cols = torch.arange(1, hidden + 1, device=src_token_global_idx.device, dtype=torch.float32)
    phase = ((src_token_global_idx.to(torch.int64) * 131071) % max(1, num_rows_total)).float() + 1
    return torch.sin(phase.unsqueeze(1) / max(1, num_rows_total) * cols + float(seed)).to(torch.bfloat16)
