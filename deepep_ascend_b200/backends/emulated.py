"""Several virtual ranks on ONE GPU in one process.

Kernels of different ranks wait on one another, so they can never be separate launches on one device.  Here every
collective call of the virtual ranks is issued as ONE cooperative launch whose ``blockIdx.y`` selects the rank;
each virtual rank has its own symmetric buffer and the peer tables point at the other ranks' buffers.  The device
code is exactly the code that runs with one process per GPU, which makes this the way to test the multi-rank
protocol (layout exchange, peer stores, peer pulls, barriers) on a single GPU.
"""
from typing import List, Optional, Sequence

import torch

from ..buffers.elastic import ElasticBuffer


class EmulatedWorld:
    def __init__(self, num_ranks: int, **buffer_kwargs):
        self.num_ranks = num_ranks
        self.buffers: List[ElasticBuffer] = [
            ElasticBuffer(None, _virtual=(r, num_ranks), **buffer_kwargs) for r in range(num_ranks)]
        self._C = self.buffers[0]._C
        self._C.ElasticBuffer.link_local([b.core for b in self.buffers])
        torch.cuda.synchronize()

    @property
    def cores(self):
        return [b.core for b in self.buffers]

    def max_sms_per_rank(self) -> int:
        """All virtual ranks' CTAs must be co-resident: one CTA per SM."""
        return max(1, torch.cuda.get_device_properties('cuda').multi_processor_count // self.num_ranks)

    def dispatch(self, xs: Sequence, topk_idxs: Sequence[Optional[torch.Tensor]], topk_weights: Sequence[Optional[torch.Tensor]],
                 num_experts: int, num_sms: int = 0, expert_alignment: int = 1, do_expand: bool = False,
                 do_cpu_sync: bool = True, handles: Optional[Sequence] = None, stats: Optional[Sequence] = None,
                 use_tma_aligned_col_major_sf: bool = False, do_zero_padding: bool = False):
        """Per-rank lists in, per-rank list of ``(recv_x, recv_topk_idx, recv_topk_weights, handle)`` out."""
        num_sms = min(num_sms or 8, self.max_sms_per_rank())
        states = []
        for r, b in enumerate(self.buffers):
            h = handles[r] if handles is not None else None
            if h is not None:
                b._attest(h, 'cached dispatch')
            states.append(b._prepare_dispatch(
                xs[r], None if h is not None else topk_idxs[r], topk_weights[r], stats[r] if stats is not None else None,
                num_experts, b.num_max_tokens_per_rank, expert_alignment if h is None else h.expert_alignment, num_sms, h, True,
                do_cpu_sync and h is None, do_expand if h is None else h.do_expand, use_tma_aligned_col_major_sf,
                None, do_zero_padding))
        self._C.ElasticBuffer.dispatch_group(self.cores, [s.call for s in states], num_sms)
        return [b._finish_dispatch(s) for b, s in zip(self.buffers, states)]

    def combine(self, xs: Sequence[torch.Tensor], handles: Sequence, topk_weights: Optional[Sequence] = None,
                bias0: Optional[Sequence] = None, bias1: Optional[Sequence] = None, weighted: bool = False, num_sms: int = 0):
        """Per-rank list of ``(combined_x, combined_topk_weights)``."""
        num_sms = min(num_sms or 8, self.max_sms_per_rank())
        calls, outs = [], []
        for r, b in enumerate(self.buffers):
            b._attest(handles[r], 'combine')
            call, out, out_w, staged = b._prepare_combine(
                xs[r], handles[r], topk_weights[r] if topk_weights is not None else None,
                bias0[r] if bias0 is not None else None, bias1[r] if bias1 is not None else None, weighted)
            for dst, src in staged:
                dst.copy_(src)
            calls.append(call)
            outs.append((out, out_w))
        self._C.ElasticBuffer.combine_group(self.cores, calls, num_sms)
        return outs

    def low_latency_dispatch(self, xs, topk_idxs, num_max_tokens: int, num_experts: int, use_fp8: bool = True,
                             round_scale: bool = False, use_ue8m0: bool = False, num_sms: int = 0, stats=None,
                             split_phases: bool = False):
        """Per-rank list of ``(recv_x | (recv_x, scales), recv_count, handle)``.  ``split_phases`` launches the
        send and the receive half separately, as the hook mode does."""
        num_sms = min(num_sms or 8, self.max_sms_per_rank())
        prepared = [b._ll_prepare_dispatch(xs[r], topk_idxs[r], num_max_tokens, num_experts,
                                           stats[r] if stats is not None else None, None, use_fp8, round_scale, use_ue8m0, 3)
                    for r, b in enumerate(self.buffers)]
        calls = [c for c, _ in prepared]
        for phases in ((1, 2) if split_phases else (3,)):
            for c in calls:
                c.phases = phases
            self._C.ll_dispatch_group(self.cores, calls, num_sms)
        outs = []
        for (c, sf), x in zip(prepared, xs):
            handle = (c.packed_src_info, c.layout_range, num_max_tokens, x.shape[1], num_experts)
            outs.append(((c.packed_x, sf) if use_fp8 else c.packed_x, c.packed_count, handle))
        return outs

    def low_latency_combine(self, xs, topk_idxs, topk_weights, handles, num_sms: int = 0, split_phases: bool = False,
                            use_logfmt: bool = False):
        num_sms = min(num_sms or 8, self.max_sms_per_rank())
        calls = [b._ll_prepare_combine(xs[r], topk_idxs[r], topk_weights[r], handles[r], None, None, 3, use_logfmt)
                 for r, b in enumerate(self.buffers)]
        for phases in ((1, 2) if split_phases else (3,)):
            for c in calls:
                c.phases = phases
            self._C.ll_combine_group(self.cores, calls, num_sms)
        return [c.out for c in calls]

    def agrs_set_config(self, num_max_session_bytes: int, num_max_agrs_per_session: int = 32) -> None:
        for b in self.buffers:
            b.agrs_set_config(num_max_session_bytes, num_max_agrs_per_session)

    def create_agrs_session(self) -> None:
        for b in self.buffers:
            b.create_agrs_session()

    def destroy_agrs_session(self) -> None:
        self._C.ElasticBuffer.barrier_group(self.cores, self._C.CH_AGRS)
        for b in self.buffers:
            b._agrs['open'] = False

    def all_gather(self, tensors: Sequence[torch.Tensor]):
        """tensors[r] is rank r's contribution -> per-rank ``[num_ranks, *shape]`` views."""
        from ..buffers.collectives import _contiguous_strides
        outs = []
        for r, b in enumerate(self.buffers):
            t = tensors[r].contiguous()
            off, nbytes = b._agrs_alloc(t.shape, t.dtype)
            for peer in range(self.num_ranks):
                b.core.peer_copy(peer, off + r * nbytes, t)
            shape = [self.num_ranks] + list(t.shape)
            outs.append(b.core.view(off, shape, list(_contiguous_strides(shape)), t.dtype))
        self._C.ElasticBuffer.barrier_group(self.cores, self._C.CH_AGRS)
        return outs

    def reduce_scatter(self, tensors: Sequence[torch.Tensor]):
        """tensors[r] is rank r's ``[num_ranks, *shape]`` input -> per-rank reduced ``[*shape]``."""
        from ..buffers.collectives import _contiguous_strides
        views = []
        for r, b in enumerate(self.buffers):
            t = tensors[r].contiguous()
            shape = list(t.shape[1:])
            off, nbytes = b._agrs_alloc(shape, t.dtype)
            for peer in range(self.num_ranks):
                b.core.peer_copy(peer, off + r * nbytes, t[peer])
            sshape = [self.num_ranks] + shape
            views.append((b.core.view(off, sshape, list(_contiguous_strides(sshape)), t.dtype), shape, t))
        self._C.ElasticBuffer.barrier_group(self.cores, self._C.CH_AGRS)
        outs = []
        for slots, shape, t in views:
            out = torch.empty(shape, dtype=t.dtype, device=t.device)
            self._C.reduce_slots(slots, out)
            outs.append(out)
        return outs

    def engram_write(self, storages: Sequence[torch.Tensor], sfs: Optional[Sequence[torch.Tensor]] = None) -> None:
        self._C.ElasticBuffer.barrier_group(self.cores, self._C.CH_ENGRAM)
        for r, (b, st) in enumerate(zip(self.buffers, storages)):
            st = st.contiguous()
            e = b._engram_place(st.shape[0], st.shape[1], st.dtype)
            e['sf'] = sfs[r] if sfs is not None else None
            b._engram_store(e, st)
        self._C.ElasticBuffer.barrier_group(self.cores, self._C.CH_ENGRAM)

    def engram_fetch(self, indices: Sequence[torch.Tensor], num_sms: int = 4, use_tma_aligned_col_major_sf: bool = False):
        """-> per-rank list of ``(fetched, fetched_sf | None)``."""
        e = self.buffers[0]._engram
        idx = [i.contiguous().to(torch.int32) for i in indices]
        outs = [b._engram_fetch_outputs(i, use_tma_aligned_col_major_sf) for b, i in zip(self.buffers, idx)]
        has_sf = e['sf'] is not None
        self._C.ElasticBuffer.engram_fetch_group(
            self.cores, [i.view(-1) for i in idx], [o for o, _ in outs], e['N'], e['entry'], e['offset'], e['cpu'],
            [b._engram['sf'] for b in self.buffers] if has_sf else [], [f for _, f in outs] if has_sf else [],
            idx[0].shape[1], num_sms)
        return outs

    def barrier(self) -> None:
        self._C.ElasticBuffer.barrier_group(self.cores)

    def destroy(self) -> None:
        torch.cuda.synchronize()
        for b in self.buffers:
            b.core.destroy()
            b._destroyed = True
