"""CPU reference backend: the semantics of ``ElasticBuffer.dispatch`` / ``combine`` on CPU tensors over a gloo
process group.  It computes the same deterministic layout as the CUDA kernels (``ops/layout_ref.py``) and moves
rows with ``all_to_all_single``, so handles, counts and results are interchangeable with the GPU path.
Parity: the oracle of deep_ep/utils/refs.py:10-243 promoted to a backend.
"""
from typing import List

import torch
import torch.distributed as dist

from ..ops import layout_ref
from ..utils.event import EventOverlap
from ..utils.math import align, per_token_cast_to_fp8


def _a2a(group, chunks: List[torch.Tensor]) -> List[torch.Tensor]:
    """Variable-size all-to-all of row blocks: chunks[d] goes to rank d; returns the block from every source."""
    world = dist.get_world_size(group)
    if world == 1:
        return [chunks[0]]
    send_counts = torch.tensor([c.shape[0] for c in chunks], dtype=torch.int64)
    recv_counts = torch.empty(world, dtype=torch.int64)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    proto = chunks[0]
    width = proto.shape[1:]
    send = torch.cat(chunks, dim=0).contiguous()
    as_bytes = send.dtype in (torch.float8_e4m3fn, torch.bfloat16)
    if as_bytes:
        send = send.view(torch.uint8).reshape(send.shape[0], -1)
    recv = torch.empty((int(recv_counts.sum()),) + tuple(send.shape[1:]), dtype=send.dtype)
    dist.all_to_all_single(recv, send, recv_counts.tolist(), send_counts.tolist(), group=group)
    if as_bytes:
        recv = recv.view(proto.dtype).reshape((recv.shape[0],) + tuple(width))
    return list(recv.split(recv_counts.tolist(), dim=0))


class CollectiveMismatch(RuntimeError):
    """The ranks of a group did not make the same call (different arguments, or a rank that never joined)."""


class CpuBackend:
    def __init__(self, group, rank: int, num_ranks: int):
        self.group, self.rank, self.R = group, rank, num_ranks
        self._calls = 0

    def _preflight(self, what: str, signature: tuple) -> None:
        """Every rank publishes (call number, operation, arguments that must agree) before any payload moves; a rank
        that disagrees, or that does not show up before the process group's time limit, turns into an error that names
        the ranks on EVERY rank, instead of a hang or of silently mixed-up rows.  Parity: the collective preflight of
        the reference's Python layer (deep_ep/buffers/elastic.py:555-862)."""
        self._calls += 1
        mine = (self._calls, what) + tuple(signature)
        if self.R == 1:
            return
        everyone = [None] * self.R
        try:
            dist.all_gather_object(everyone, mine, group=self.group)
        except Exception as e:
            raise CollectiveMismatch(f'[EP rank {self.rank}] {what} number {self._calls}: not every rank joined the call '
                                     f'before the process group gave up ({type(e).__name__}: {str(e)[:200]})') from e
        odd = [r for r, sig in enumerate(everyone) if sig != everyone[0]]
        if odd:
            detail = ', '.join(f'rank {r}: {everyone[r]}' for r in ([0] + odd))
            raise CollectiveMismatch(f'[EP rank {self.rank}] {what} number {self._calls}: ranks {odd} disagree with rank 0 '
                                     f'about the call ({detail})')

    def _gather_counts(self, local: layout_ref.LocalLayout):
        mine = torch.cat([local.rank_count, local.expert_count]).to(torch.int64)
        if self.R == 1:
            allc = mine.unsqueeze(0)
        else:
            out = [torch.empty_like(mine) for _ in range(self.R)]
            dist.all_gather(out, mine, group=self.group)
            allc = torch.stack(out)
        return allc[:, :self.R], allc[:, self.R:]

    def dispatch(self, buf, x, topk_idx, topk_weights, stats, num_experts, num_max_tokens, alignment, handle, do_expand,
                 do_zero_padding, do_handle_copy):
        from ..buffers.elastic import EPHandle
        R, me = self.R, self.rank
        x_in, sf_in = x if isinstance(x, tuple) else (x, None)
        if buf.use_fp8_dispatch and x_in.dtype == torch.bfloat16:
            x_in, sf_in = per_token_cast_to_fp8(x_in)
        T, H = x_in.shape
        El = num_experts // R
        self._preflight('dispatch', (num_experts, num_max_tokens, alignment, bool(do_expand), handle is not None, H,
                                     str(x_in.dtype), (handle.topk_idx if handle is not None else topk_idx).shape[1]))
        if handle is not None:
            topk_idx = handle.topk_idx
        K = topk_idx.shape[1]
        local = layout_ref.local_layout(topk_idx, num_experts, R)
        rank_counts, expert_counts = self._gather_counts(local)
        gl = layout_ref.global_layout(local, rank_counts, expert_counts, me, num_experts, do_expand, alignment)
        rows_total = gl.num_expanded_tokens if do_expand else gl.num_recv_tokens

        dst_rank, dst_row = layout_ref.unpack_lane(gl.plan)
        payload = {'x': [], 'sf': [], 'idx': [], 'w': [], 'meta': [], 'row': []}
        for d in range(R):
            t_idx, k_idx = torch.nonzero(dst_rank == d, as_tuple=True)
            order = torch.argsort(dst_row[t_idx, k_idx])
            t_idx, k_idx = t_idx[order], k_idx[order]
            payload['row'].append(dst_row[t_idx, k_idx].to(torch.int64).unsqueeze(1))
            payload['x'].append(x_in[t_idx])
            if sf_in is not None:
                payload['sf'].append(sf_in[t_idx].float())
            payload['idx'].append(layout_ref.localize_topk_idx(topk_idx[t_idx], d, num_experts, R))
            if topk_weights is not None:
                payload['w'].append(topk_weights[t_idx, k_idx].unsqueeze(1) if do_expand else topk_weights[t_idx])
            payload['meta'].append(torch.stack([me * num_max_tokens + t_idx, me * K + k_idx], dim=1).to(torch.int32))
        rows = torch.cat(_a2a(self.group, payload['row'])).squeeze(1)

        def place(chunks, dtype, width):
            out = torch.zeros((rows_total,) + width, dtype=dtype)
            data = torch.cat(_a2a(self.group, chunks))
            if out.dtype == torch.float8_e4m3fn:
                out.view(torch.uint8)[rows] = data.view(torch.uint8)
            else:
                out[rows] = data
            return out
        recv_x = place(payload['x'], x_in.dtype, (H,))
        recv_sf = place(payload['sf'], torch.float32, (sf_in.shape[1],)) if sf_in is not None else None
        recv_idx = None if do_expand else place(payload['idx'], topk_idx.dtype, (K,))
        recv_w = None
        if topk_weights is not None:
            recv_w = place(payload['w'], torch.float32, (1,)).squeeze(1) if do_expand else place(payload['w'], torch.float32, (K,))
        meta = place(payload['meta'], torch.int32, (2,))
        if stats is not None:
            stats += gl.recv_per_expert
        per_expert_list = [align(int(c), alignment) for c in gl.recv_per_expert.tolist()]
        if handle is None:
            handle = EPHandle(do_expand, num_experts, alignment, num_max_tokens, 0,
                              topk_idx.clone() if do_handle_copy else topk_idx, gl.num_recv_tokens, gl.num_expanded_tokens,
                              per_expert_list, gl.psum_recv_per_rank, gl.psum_recv_per_expert, gl.recv_per_expert, meta,
                              gl.lane_src, gl.plan, H, 0, topk_weights, stamp=buf._stamp(T, K))
        else:
            handle.recv_src_metadata = meta
        x_out = (recv_x, recv_sf) if sf_in is not None else recv_x
        return x_out, recv_idx, recv_w, handle, EventOverlap(None)

    def combine(self, buf, x, handle, topk_weights, bias0, bias1, weighted):
        R, me = self.R, self.rank
        T, K = handle.plan.shape
        H = x.shape[1]
        self._preflight('combine', (handle.num_experts, handle.num_max_tokens_per_rank, bool(handle.do_expand), H, str(x.dtype),
                                    K, topk_weights is not None, bool(weighted)))
        meta = handle.recv_src_metadata.to(torch.int64)
        rows = handle.num_rows
        # expert rank side: send every row (and its carried weights) back to the rank it came from, in row order
        src_rank = (meta[:rows, 0] // handle.num_max_tokens_per_rank)
        send_x, send_w, send_row = [], [], []
        w_cols = 1 if handle.do_expand else K
        for s in range(R):
            sel = torch.nonzero(src_rank == s, as_tuple=True)[0]
            if handle.do_expand and handle.expert_alignment > 1:
                sel = sel[self._valid_rows(handle)[sel]]
            send_x.append(x[sel])
            send_row.append(sel.to(torch.int64).unsqueeze(1))
            if topk_weights is not None:
                send_w.append(topk_weights[:rows].reshape(rows, w_cols)[sel])
        got_x, got_row = _a2a(self.group, send_x), _a2a(self.group, send_row)
        got_w = _a2a(self.group, send_w) if topk_weights is not None else None

        def rows_of(rank: int):
            table = torch.zeros((int(got_row[rank].max().item()) + 1 if got_row[rank].numel() else 1, H), dtype=x.dtype)
            if got_row[rank].numel():
                table[got_row[rank].squeeze(1)] = got_x[rank]
            return table
        mul = handle.topk_weights if weighted else None
        out = layout_ref.combine_ref(rows_of, handle.plan, H, bias0, bias1, mul, out_dtype=x.dtype)
        out_w = None
        if topk_weights is not None:
            out_w = torch.zeros((T, K), dtype=torch.float32)
            lrank, lrow = layout_ref.unpack_lane(handle.dst_buffer_slot_idx)
            for r in range(R):
                if not got_row[r].numel():
                    continue
                table = torch.zeros((int(got_row[r].max().item()) + 1, w_cols), dtype=torch.float32)
                table[got_row[r].squeeze(1)] = got_w[r]
                t_idx, k_idx = torch.nonzero(lrank == r, as_tuple=True)
                vals = table[lrow[t_idx, k_idx]]
                out_w[t_idx, k_idx] = vals[:, 0] if w_cols == 1 else vals[torch.arange(len(k_idx)), k_idx]
        return out, out_w, EventOverlap(None)

    @staticmethod
    def _valid_rows(handle) -> torch.Tensor:
        """Rows of the expand layout that hold a token (not alignment padding)."""
        ends = handle.psum_num_recv_tokens_per_expert.to(torch.int64)
        a = handle.expert_alignment
        starts = torch.cat([torch.zeros(1, dtype=torch.int64), (ends[:-1] + a - 1) // a * a])
        r = torch.arange(handle.num_rows).unsqueeze(1)
        return ((r >= starts.unsqueeze(0)) & (r < ends.unsqueeze(0))).any(dim=1)
