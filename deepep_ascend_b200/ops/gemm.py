"""Python front end of the tcgen05 GEMM kernels (``csrc/kernels/gemm_sm100.cu``) and of the small MoE helpers.

No counterpart in the reference, which contains no tensor-core code; these kernels exist for the fused MoE layer
and for the all-gather / reduce-scatter fused GEMMs.
"""
from typing import Optional, Tuple

import torch

from .. import _native

BLOCK_M = 128   # rows of one output tile; expert segments of the grouped GEMM are aligned to it


def _core_of(buffer):
    return None if buffer is None else buffer.core


def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, num_sms: int = 0, buffer=None) -> torch.Tensor:
    """``a [M, K] @ b [N, K]^T -> bf16 [M, N]`` (bf16 operands, fp32 accumulation in tensor memory).  With ``buffer``
    (an ``ElasticBuffer``) a pipeline wait that runs out inside the kernel is reported through that buffer's status
    block and time limit, so ``buffer.check_status()`` raises and poisons it like any other failed device wait."""
    return _native.load().gemm_nt(a, b, None, None, None, out, num_sms, None, 0, None, _core_of(buffer))


def grouped_gemm_nt(a: torch.Tensor, b: torch.Tensor, tile_group: torch.Tensor, out: Optional[torch.Tensor] = None,
                    sfa: Optional[torch.Tensor] = None, sfb: Optional[torch.Tensor] = None, num_sms: int = 0, buffer=None) -> torch.Tensor:
    """Every 128-row tile ``t`` of ``a`` is multiplied by ``b[tile_group[t]]`` (``-1`` skips the tile).  bf16 operands,
    or e4m3 operands with ``sfa [M, K/128]`` and ``sfb [G, N/128, K/128]`` fp32 block scales.  ``buffer``: see
    :func:`gemm_nt`."""
    return _native.load().gemm_nt(a, b, sfa, sfb, tile_group, out, num_sms, None, 0, None, _core_of(buffer))


def quantize_weight_blocks(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``w [G, N, K]`` -> (e4m3 ``[G, N, K]``, fp32 scales ``[G, ceil(N/128), ceil(K/128)]``), one scale per
    128 x 128 block (the weight format of DeepSeek-V3 style FP8 training)."""
    G, N, K = w.shape
    nb, kb = (N + 127) // 128, (K + 127) // 128
    wp = torch.zeros(G, nb * 128, kb * 128, device=w.device, dtype=torch.float32)
    wp[:, :N, :K] = w
    blocks = wp.view(G, nb, 128, kb, 128)
    amax = blocks.abs().amax(dim=(2, 4)).clamp(1e-4)
    q = (blocks * (448.0 / amax)[:, :, None, :, None]).to(torch.float8_e4m3fn).view(G, nb * 128, kb * 128)[:, :N, :K].contiguous()
    return q, (amax / 448.0).contiguous()


def expert_segments(psum_expert_ends: torch.Tensor, num_rows: int, alignment: int = BLOCK_M) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """From the expand-layout segment ends of ``EPHandle.psum_num_recv_tokens_per_expert`` (segment ``i`` starts at
    ``align(end[i-1], alignment)``) -> (``tile_group int32 [ceil(num_rows / 128)]`` with -1 for tiles that hold no
    token, ``valid_row bool [num_rows]``, ``seg_off int32 [G + 1]`` aligned segment boundaries).  One kernel launch, no host
    synchronisation (CPU tensors take the plain PyTorch statement below)."""
    assert alignment % BLOCK_M == 0, 'expert segments must start on a tile boundary'
    if not psum_expert_ends.is_cuda:
        return expert_segments_ref(psum_expert_ends, num_rows, alignment)
    ends = psum_expert_ends if psum_expert_ends.dtype == torch.int32 else psum_expert_ends.to(torch.int32)
    return tuple(_native.load().expert_segments(ends.contiguous(), num_rows, alignment))


def expert_tile_groups(psum_expert_ends: torch.Tensor, num_rows: int, alignment: int = BLOCK_M) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(tile_group, valid_row)`` of ``expert_segments``."""
    return expert_segments(psum_expert_ends, num_rows, alignment)[:2]


def expert_segments_ref(psum_expert_ends: torch.Tensor, num_rows: int, alignment: int = BLOCK_M):
    """The same three tensors stated with plain PyTorch operations (what the kernel is tested against)."""
    ends = psum_expert_ends.to(torch.int64)
    aligned_ends = (ends + alignment - 1) // alignment * alignment
    starts = torch.cat([torch.zeros(1, dtype=torch.int64, device=ends.device), aligned_ends[:-1]])
    num_tiles = (num_rows + BLOCK_M - 1) // BLOCK_M
    tile_start = torch.arange(num_tiles, device=ends.device, dtype=torch.int64) * BLOCK_M
    grp = torch.searchsorted(aligned_ends, tile_start, right=True)
    grp_c = grp.clamp_max(ends.numel() - 1)
    has_rows = (grp < ends.numel()) & (tile_start < ends[grp_c]) & (tile_start >= starts[grp_c])
    tile_group = torch.where(has_rows, grp_c, torch.full_like(grp_c, -1)).to(torch.int32)
    rows = torch.arange(num_rows, device=ends.device, dtype=torch.int64)
    rgrp = torch.searchsorted(aligned_ends, rows, right=True).clamp_max(ends.numel() - 1)
    valid_row = (rows >= starts[rgrp]) & (rows < ends[rgrp])
    seg_off = torch.cat([torch.zeros(1, dtype=torch.int64, device=ends.device), aligned_ends]).to(torch.int32)
    return tile_group.contiguous(), valid_row, seg_off.contiguous()


def local_expand_plan(recv_idx: torch.Tensor, psum_aligned: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """For the output of a NON-expand dispatch made with ``expert_alignment=128``: ``recv_idx [rows, K]`` (local expert ids,
    -1 elsewhere) and ``EPHandle.psum_num_recv_tokens_per_expert`` (inclusive sums of the aligned counts) ->
    (``pos int32 [rows, K]``: the row of pair (row, k) in the per-expert (expand) layout, -1 if none; ``seg_end int32 [El]``:
    end of the token rows of every expert segment, the input of ``expert_segments``).  Rows of a segment are in received
    order, the same on every run."""
    if not recv_idx.is_cuda:
        return local_expand_plan_ref(recv_idx, psum_aligned)
    pos, seg_end = _native.load().local_expand_plan(recv_idx, psum_aligned.contiguous())
    return pos, seg_end


def local_expand_plan_ref(recv_idx: torch.Tensor, psum_aligned: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """The same two tensors stated with plain PyTorch operations (any device; what the kernels are tested against)."""
    El = psum_aligned.numel()
    ends = psum_aligned.to(torch.int64)
    idx = recv_idx.to(torch.int64)
    valid = (idx >= 0) & (idx < El)
    flat_e = torch.where(valid, idx, torch.full_like(idx, El)).reshape(-1)
    # stable sort by expert keeps the received (row-major) order inside every expert
    order = torch.sort(flat_e, stable=True).indices
    counts = torch.bincount(flat_e, minlength=El + 1)[:El]
    aligned = torch.cat([ends[:1], ends[1:] - ends[:-1]])
    starts = ends - aligned
    first = torch.cumsum(counts, 0) - counts                      # position of every expert's first pair in `order`
    sorted_e = flat_e[order]
    keep = sorted_e < El
    rank_in_e = torch.arange(order.numel(), device=idx.device) - first[sorted_e.clamp(max=El - 1)]
    pos = torch.full((idx.numel(),), -1, dtype=torch.int64, device=idx.device)
    pos[order[keep]] = (starts[sorted_e[keep]] + rank_in_e[keep])
    return pos.reshape(idx.shape).to(torch.int32), (starts + counts).to(torch.int32)


def local_expand_copy(pos: torch.Tensor, x: torch.Tensor, num_out: int, sf: Optional[torch.Tensor] = None,
                      w: Optional[torch.Tensor] = None):
    """Writes every received row of ``x`` (and its scales ``sf [rows, G]`` / weights ``w [rows, K]``) to its expert rows ->
    ``[x_out [num_out, width], sf_out, w_out [num_out]]`` (only those asked for).  Alignment rows of the output are not written."""
    return _native.load().local_expand_copy(pos, x, num_out, sf, w)


def local_reduce(pos: torch.Tensor, y: torch.Tensor, w: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[row] = sum_k w[pos[row, k]] * y[pos[row, k]]`` (``w``: one weight per expert row; plain sum without it) in fp32,
    rounded once to bf16."""
    return _native.load().local_reduce(pos, y, w, out)


def per_token_cast_to_fp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 ``[rows, H]`` -> (e4m3 ``[rows, H]``, fp32 scales ``[rows, ceil(H / 128)]``), one kernel."""
    q, sf = _native.load().per_token_cast_to_fp8(x.contiguous())
    return q, sf


def swiglu_quant(h: torch.Tensor, keep_bf16: bool = False):
    """``h [rows, 2I]`` bf16 (gate | up) -> ``(e4m3 [rows, I], scales [rows, I/128][, bf16 activation])``."""
    return _native.load().swiglu_quant(h, keep_bf16)


def gemm_kgrouped(a_t: torch.Tensor, b_t: torch.Tensor, k_off: torch.Tensor, num_sms: int = 0) -> torch.Tensor:
    """Weight gradients of a grouped layer in one launch: ``out[e] = a_t[:, k0:k1] @ b_t[:, k0:k1]^T`` with
    ``(k0, k1) = (k_off[e], k_off[e + 1])``; ``a_t [M, rows]``, ``b_t [N, rows]`` bf16 (the transposed activations and
    gradients, so that the reduction dimension = rows of the expert segment is contiguous), ``k_off`` int32
    ``[G + 1]`` multiples of 64 on the device.  -> bf16 ``[G, M, N]``; an expert without rows gets zeros."""
    return _native.load().gemm_kgrouped(a_t, b_t, k_off, num_sms)


def segment_offsets(psum_expert_ends: torch.Tensor, alignment: int = BLOCK_M) -> torch.Tensor:
    """Expand-layout segment boundaries as ``int32 [G + 1]``: segment ``e`` covers rows ``[off[e], off[e + 1])``
    including its alignment padding.  Stays on the device."""
    return expert_segments(psum_expert_ends, 0, alignment)[2]


def moe_bwd_prep(g_rows: torch.Tensor, y: torch.Tensor, w: torch.Tensor, valid_row: torch.Tensor):
    """Backward of the weighted combine at the expert rows -> ``(g * w [rows, H], (g * w)^T [H, rows], sum(g * y) [rows])``;
    padding rows give zeros."""
    return _native.load().moe_bwd_prep(g_rows, y, w, valid_row)


def swiglu_bwd(d_act: torch.Tensor, h: torch.Tensor, valid_row: torch.Tensor, row_weight: Optional[torch.Tensor] = None):
    """Backward of ``silu(gate) * up`` -> ``(d_h [rows, 2I], d_h^T [2I, rows], activation^T [I, rows])``.  With
    ``row_weight [rows]`` the incoming gradient is taken as the gradient of the UNWEIGHTED activation: it is multiplied by
    the weight before it flows on, and ``sum_i d_act[r, i] * activation[r, i]`` (= d loss / d weight) is returned as a
    fourth tensor."""
    return _native.load().swiglu_bwd(d_act, h, valid_row, row_weight)


def weighted_transpose(g_rows: torch.Tensor, w: torch.Tensor, valid_row: torch.Tensor) -> torch.Tensor:
    """``(g * w[:, None])^T`` as bf16 ``[H, rows]`` with zero columns for padding rows."""
    return _native.load().weighted_transpose(g_rows, w, valid_row)


def dequant_transpose(q: torch.Tensor, sf: torch.Tensor, valid_row: torch.Tensor) -> torch.Tensor:
    """e4m3 rows with 1 x 128 scales -> bf16 ``(q * scale)^T [H, rows]``; padding rows give zeros."""
    return _native.load().dequant_transpose(q, sf, valid_row)
