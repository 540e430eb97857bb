"""CPU / gloo versions of the non-MoE operations of ``ElasticBuffer`` and of the low-latency pair, with the
same arguments, results and handle tuples as the CUDA paths (``buffers/collectives.py``, ``buffers/low_latency.py``):
all-gather / reduce-scatter sessions, pipeline send / recv, Engram tables, low-latency dispatch / combine.

They exist so that the host-side logic built on these calls (session bookkeeping, schedules, packed layouts, handles)
can be run and tested on machines without a GPU, the way the dispatch / combine backend in ``backends/cpu.py`` does
for the MoE pair.  Data moves through ``torch.distributed`` collectives of the caller's (gloo) group.
"""
import math
from typing import Callable, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist

from ..utils.event import EventOverlap
from ..utils.math import logfmt10_roundtrip, per_token_cast_to_fp8
from .cpu import _a2a


def _no_wait() -> None:
    return None


class CpuCollectives:
    def __init__(self, group, rank: int, num_ranks: int):
        self.group, self.rank, self.R = group, rank, num_ranks
        self._agrs = None
        self._pp = None
        self._engram = None
        self._ll_mask = torch.zeros(num_ranks, dtype=torch.int32)
        self._ll_combine_x = None

    # ------------------------------------------------------------------------------------------ AG / RS sessions
    def agrs_set_config(self, num_max_session_bytes: int, num_max_agrs_per_session: int = 32, use_stream_memops: bool = False) -> None:
        assert num_max_agrs_per_session <= 32
        assert self._agrs is None or not self._agrs['open'], 'destroy the open session first'
        self._agrs = {'bytes': num_max_session_bytes, 'cursor': 0, 'open': False, 'count': 0, 'max': num_max_agrs_per_session,
                      'inplace': {}}

    def create_agrs_session(self) -> None:
        assert self._agrs is not None, 'call agrs_set_config first'
        assert not self._agrs['open'], 'one session at a time'
        self._agrs.update(open=True, cursor=0, count=0, inplace={})

    def destroy_agrs_session(self) -> None:
        assert self._agrs is not None and self._agrs['open']
        if self.R > 1:
            dist.barrier(group=self.group)       # every rank is done with the gathered tensors
        self._agrs['open'] = False

    def _agrs_alloc(self, shape: Sequence[int], dtype: torch.dtype) -> None:
        a = self._agrs
        assert a is not None and a['open'], 'no open AG/RS session'
        assert a['count'] < a['max'], 'too many collectives in this session'
        total = (self.R * math.prod(shape) * dtype.itemsize + 31) // 32 * 32
        assert a['cursor'] + total <= a['bytes'], 'session region exhausted: raise num_max_session_bytes'
        a['cursor'] += total
        a['count'] += 1

    def agrs_get_inplace_tensor(self, shape: Sequence[int], dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        self._agrs_alloc(shape, dtype)
        full = torch.zeros([self.R] + list(shape), dtype=dtype)
        mine = full[self.rank]
        self._agrs['inplace'][mine.data_ptr()] = full
        return mine

    def all_gather(self, tensors: Union[torch.Tensor, Sequence[torch.Tensor]]):
        single = isinstance(tensors, torch.Tensor)
        outs = []
        for t in ([tensors] if single else list(tensors)):
            full = self._agrs['inplace'].pop(t.data_ptr(), None) if t.is_contiguous() else None
            if full is None:
                t = t.contiguous()
                self._agrs_alloc(t.shape, t.dtype)
                full = torch.empty([self.R] + list(t.shape), dtype=t.dtype)
                full[self.rank] = t
            if self.R > 1:
                as_bytes = full.dtype in (torch.float8_e4m3fn, torch.bfloat16)
                view = full.view(torch.uint8) if as_bytes else full
                parts = list(view.unbind(0))
                dist.all_gather(parts, parts[self.rank].clone(), group=self.group)
            outs.append(full)
        return (outs[0] if single else outs), _no_wait

    def reduce_scatter(self, tensor: torch.Tensor) -> Tuple[torch.Tensor, Callable]:
        assert tensor.shape[0] == self.R and tensor.dtype in (torch.bfloat16, torch.float32)
        shape = list(tensor.shape[1:])
        self._agrs_alloc(shape, tensor.dtype)
        slices = _a2a(self.group, [tensor[p].reshape(1, -1).contiguous() for p in range(self.R)])
        acc = torch.zeros(slices[0].shape, dtype=torch.float32)
        for s in slices:                       # fp32 accumulation in rank order, like the kernel
            acc += s.float()
        return acc.to(tensor.dtype).reshape(shape), _no_wait

    # ------------------------------------------------------------------------------------------ pipeline parallel
    def pp_set_config(self, num_max_tensor_bytes: int, num_max_inflight_tensors: int) -> None:
        self._pp = {'prev': (self.rank - 1) % self.R, 'next': (self.rank + 1) % self.R, 'max_bytes': num_max_tensor_bytes,
                    'inflight': num_max_inflight_tensors, 'pending': []}

    def _pp_check(self, t: torch.Tensor, peer: int) -> None:
        assert self._pp is not None, 'call pp_set_config first'
        assert peer in (self._pp['prev'], self._pp['next']), 'pipeline peers are the ring neighbours'
        assert t.numel() * t.element_size() <= self._pp['max_bytes'], 'tensor exceeds num_max_tensor_bytes'
        if len(self._pp['pending']) >= 2 * self._pp['inflight']:
            self._pp['pending'].pop(0).wait()

    def pp_send(self, t: torch.Tensor, dst_rank_idx: int) -> None:
        self._pp_check(t, dst_rank_idx)
        payload = t.contiguous()
        if payload.dtype in (torch.float8_e4m3fn, torch.bfloat16):
            payload = payload.view(torch.uint8)
        self._pp['pending'].append(dist.isend(payload, dist.get_global_rank(self.group, dst_rank_idx), group=self.group))

    def pp_recv(self, t: torch.Tensor, src_rank_idx: int) -> None:
        self._pp_check(t, src_rank_idx)
        assert t.is_contiguous()
        target = t.view(torch.uint8) if t.dtype in (torch.float8_e4m3fn, torch.bfloat16) else t
        dist.irecv(target, dist.get_global_rank(self.group, src_rank_idx), group=self.group).wait()

    # ------------------------------------------------------------------------------------------ Engram
    def engram_write(self, storage: torch.Tensor, sf: Optional[torch.Tensor] = None) -> None:
        storage = storage.contiguous()
        N, H = storage.shape
        assert (H * storage.element_size()) % 16 == 0, 'an entry must be a multiple of 16 bytes'
        if self._engram is not None:
            assert (N, H, storage.dtype) == self._engram['key'], 'the Engram table shape is fixed per buffer'
        if sf is not None:
            assert sf.dim() == 2 and sf.is_contiguous() and sf.element_size() == 4 and sf.shape[0] == N * self.R, \
                '`sf` must be a contiguous [num_ranks * N, packs] table of 4-byte packs'
        # every rank keeps a copy of all tables: a fetch is then a local gather
        table, _ = self._gather_rows(storage)
        self._engram = {'key': (N, H, storage.dtype), 'table': table, 'sf': sf}

    def _gather_rows(self, t: torch.Tensor):
        as_bytes = t.dtype in (torch.float8_e4m3fn, torch.bfloat16)
        mine = t.view(torch.uint8) if as_bytes else t
        parts = [torch.empty_like(mine) for _ in range(self.R)]
        if self.R > 1:
            dist.all_gather(parts, mine.contiguous(), group=self.group)
        else:
            parts[0] = mine
        full = torch.cat(parts, dim=0)
        return (full.view(t.dtype) if as_bytes else full), None

    def engram_fetch(self, indices: torch.Tensor, use_tma_aligned_col_major_sf: bool = False):
        e = self._engram
        assert e is not None, 'call engram_write first'
        idx = indices.to(torch.int64)
        T, n = idx.shape
        H = e['key'][1]
        out = e['table'][idx.reshape(-1)].reshape(T, n * H)
        fetched_sf = None
        if e['sf'] is not None:
            packs = e['sf'].shape[1]
            rows = e['sf'][idx.reshape(-1)].reshape(T, n * packs)
            if use_tma_aligned_col_major_sf:
                fetched_sf = torch.empty_strided((T, n * packs), (1, (T + 3) // 4 * 4), dtype=rows.dtype)
                fetched_sf.copy_(rows)
            else:
                fetched_sf = rows.contiguous()

        def hook():
            return out, fetched_sf
        return hook

    # ------------------------------------------------------------------------------------------ low latency
    def low_latency_dispatch(self, x, topk_idx, M: int, E: int, stats=None, use_fp8: bool = True, round_scale: bool = False,
                             use_ue8m0: bool = False):
        R, me = self.R, self.rank
        El = E // R
        T, H = x.shape
        K = topk_idx.shape[1]
        assert T <= M, 'more tokens than num_max_dispatch_tokens_per_rank'
        if use_fp8:
            q, sf = per_token_cast_to_fp8(x, round_scale=round_scale or use_ue8m0, use_ue8m0=use_ue8m0)
        else:
            q, sf = x, None
        # one message per (token, lane) with a valid expert, to the rank that owns the expert; ordered by (expert, token, lane)
        t_idx, k_idx = torch.nonzero(topk_idx >= 0, as_tuple=True)
        e_of = topk_idx[t_idx, k_idx].to(torch.int64)
        dst = e_of // El
        alive = self._ll_mask[dst] == 0 if self._ll_mask.any() else torch.ones_like(dst, dtype=torch.bool)
        chunks_x, chunks_sf, chunks_meta = [], [], []
        for d in range(R):
            sel = torch.nonzero((dst == d) & alive, as_tuple=True)[0]
            order = torch.argsort(e_of[sel] * (M * K) + t_idx[sel] * K + k_idx[sel])
            sel = sel[order]
            chunks_x.append(q[t_idx[sel]])
            if sf is not None:
                chunks_sf.append(sf[t_idx[sel]])
            chunks_meta.append(torch.stack([e_of[sel] % El, t_idx[sel], k_idx[sel]], dim=1).to(torch.int64))
        got_x, got_meta = _a2a(self.group, chunks_x), _a2a(self.group, chunks_meta)
        got_sf = _a2a(self.group, [c.view(torch.int32) if c.dtype != torch.float32 else c for c in chunks_sf]) if sf is not None else None
        recv_x = torch.zeros((El, R * M, H), dtype=q.dtype)
        sf_cols = sf.shape[1] if sf is not None else 0
        store = torch.zeros((El, sf_cols, R * M), dtype=sf.dtype) if sf is not None else None
        src_info = torch.zeros((El, R * M), dtype=torch.int32)
        layout_range = torch.zeros((El, R), dtype=torch.int64)
        count = torch.zeros(El, dtype=torch.int32)
        for j in range(El):
            begin = 0
            for s in range(R):
                m = got_meta[s]
                if int(self._ll_mask[s]):          # a masked source is ignored, as the kernels do not wait for its counts
                    m = m[:0]
                rows = torch.nonzero(m[:, 0] == j, as_tuple=True)[0] if m.numel() else m.new_zeros(0)
                n = rows.numel()
                if n:
                    if q.dtype == torch.float8_e4m3fn:
                        recv_x[j, begin:begin + n].view(torch.uint8).copy_(got_x[s][rows].view(torch.uint8))
                    else:
                        recv_x[j, begin:begin + n] = got_x[s][rows]
                    if sf is not None:
                        store[j, :, begin:begin + n] = got_sf[s][rows].view(sf.dtype).t()
                    src_info[j, begin:begin + n] = ((m[rows, 2] << 20) | m[rows, 1]).to(torch.int32)
                layout_range[j, s] = (begin << 32) | n
                begin += n
            count[j] = begin
        if stats is not None:
            stats += count
        handle = (src_info, layout_range, M, H, E)
        recv = (recv_x, store.transpose(1, 2)) if sf is not None else recv_x
        return recv, count, handle, EventOverlap(None), None

    def low_latency_combine(self, x, topk_idx, topk_weights, handle, use_logfmt: bool = False, out=None):
        src_info, layout_range, M, H, E = handle
        R = self.R
        El = E // R
        T, K = topk_idx.shape
        # every expert rank returns the rows of a source in the packed order, tagged with (token, lane)
        send_x, send_meta = [], []
        for s in range(R):
            rows, metas = [], []
            for j in range(El):
                begin, n = int(layout_range[j, s]) >> 32, int(layout_range[j, s]) & 0xffffffff
                if n and not int(self._ll_mask[s]):
                    rows.append(x[j, begin:begin + n])
                    info = src_info[j, begin:begin + n].to(torch.int64)
                    metas.append(torch.stack([info & 0xfffff, info >> 20], dim=1))
            send_x.append(torch.cat(rows) if rows else x.new_zeros((0, H)))
            send_meta.append(torch.cat(metas) if metas else torch.zeros((0, 2), dtype=torch.int64))
        got_x, got_meta = _a2a(self.group, send_x), _a2a(self.group, send_meta)
        table = torch.zeros((T, K, H), dtype=torch.float32)
        for s in range(R):
            if got_meta[s].numel():
                rows = got_x[s]
                vals = logfmt10_roundtrip(rows) if use_logfmt else rows.float()
                table[got_meta[s][:, 0], got_meta[s][:, 1]] = vals
        w = torch.where(topk_idx >= 0, topk_weights.float(), torch.zeros(()))
        acc = torch.zeros((T, H), dtype=torch.float32)
        for k in range(K):                      # lane order, fp32
            acc += w[:, k].unsqueeze(1) * table[:, k]
        result = acc.to(torch.bfloat16)
        if out is not None:
            out.copy_(result)
            result = out
        return result, EventOverlap(None), None

    def get_next_low_latency_combine_buffer(self, handle: tuple) -> torch.Tensor:
        _, _, M, H, E = handle
        if self._ll_combine_x is None:
            self._ll_combine_x = [torch.zeros((E // self.R, self.R * M, H), dtype=torch.bfloat16) for _ in range(2)]
            self._ll_next = 0
        buf = self._ll_combine_x[self._ll_next & 1]
        self._ll_next += 1
        return buf

    def mask(self) -> torch.Tensor:
        return self._ll_mask
