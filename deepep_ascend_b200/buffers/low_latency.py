"""Low-latency (decode) dispatch / combine on ``ElasticBuffer``.

Same results and handle tuple as the reference's ``Buffer.low_latency_dispatch`` / ``low_latency_combine``
(deep_ep/buffers/legacy.py:553-670): tokens are cast to FP8 on the fly, packed per local expert into
``[E_local, ranks * max_tokens, hidden]``, and combine returns ``sum_k w_k * x_k``.  Both calls are free of host
synchronisation and of protocol state on the host, so they can be captured in a CUDA graph and replayed;
``return_recv_hook=True`` splits a call into a send launch and a receive launch so that no SM is held while the
data is in flight.
"""
from typing import Optional

import torch

from ..utils.event import EventHandle, EventOverlap
from ..utils.math import align


class LowLatencyMixin:
    """Mixed into ``ElasticBuffer``; uses ``self.core``, ``self.reserve`` and the rank attributes."""

    _ll = None

    @staticmethod
    def get_low_latency_size_hint(num_max_dispatch_tokens_per_rank: int, hidden: int, num_ranks: int, num_experts: int,
                                  num_topk: int = 8) -> int:
        """Bytes to pass as ``extra_bytes`` so that the low-latency regions fit."""
        from .. import _native
        return _native.load().get_low_latency_rdma_size_hint(num_max_dispatch_tokens_per_rank, hidden, num_ranks,
                                                             num_experts, num_topk)

    def _ll_setup(self, M: int, H: int, E: int, K: int):
        """Reserve the two buffer sets on first use (every rank makes the same calls in the same order, so the
        offsets agree everywhere)."""
        key = (M, H, E, K)
        if self._ll is not None:
            assert self._ll['key'] == key, 'low-latency shape changed; create another buffer for a different shape'
            return self._ll
        C = self._C
        msg = C.ll_message_bytes(H)
        d_bytes = align(E * M * msg, 1024)
        c_bytes = align(M * K * H * 2, 1024)
        self._ll = {
            'key': key, 'msg': msg,
            'dispatch': [self.reserve(d_bytes), self.reserve(d_bytes)],
            'combine': [self.reserve(c_bytes), self.reserve(c_bytes)],
            'mask': torch.zeros(self.num_ranks, dtype=torch.int32, device='cuda'),
            'c_bytes': c_bytes, 'calls': 0,
        }
        return self._ll

    def _ll_num_sms(self, num_sms: int) -> int:
        if num_sms:
            return num_sms
        return min(torch.cuda.get_device_properties('cuda').multi_processor_count, 148) if self._virtual is None else 8

    # ------------------------------------------------------------------------------------------ dispatch
    def _ll_prepare_dispatch(self, x, topk_idx, M, E, cumulative_stats, wait_stats, use_fp8, round_scale, use_ue8m0, phases):
        C = self._C
        T, H = x.shape
        K = topk_idx.shape[1]
        ll = self._ll_setup(M, H, E, K)
        R, El = self.num_ranks, E // self.num_ranks
        dev = x.device
        G = (H + 127) // 128
        call = C.LLDispatchCall()
        call.x, call.topk_idx = x.contiguous(), topk_idx.contiguous()
        call.num_experts, call.num_max_tokens = E, M
        call.use_fp8, call.round_scale, call.use_ue8m0 = use_fp8, round_scale or use_ue8m0, use_ue8m0
        call.phases = phases
        call.off_slab0, call.off_slab1 = ll['dispatch'][0], ll['dispatch'][1]
        call.msg_bytes = ll['msg']
        call.packed_x = torch.empty((El, R * M, H), dtype=torch.float8_e4m3fn if use_fp8 else torch.bfloat16, device=dev)
        sf_view = None
        if use_fp8:
            if use_ue8m0:
                store = torch.zeros((El, (G + 3) // 4, R * M), dtype=torch.int32, device=dev)
            else:
                store = torch.empty((El, G, R * M), dtype=torch.float32, device=dev)
            call.packed_sf = store
            sf_view = store.transpose(1, 2)      # [E_local, R*M, G(/4)], column-major in the last two dims
        call.packed_src_info = torch.empty((El, R * M), dtype=torch.int32, device=dev)
        call.layout_range = torch.empty((El, R), dtype=torch.int64, device=dev)
        call.packed_count = torch.empty((El,), dtype=torch.int32, device=dev)
        if cumulative_stats is not None:
            call.stats = cumulative_stats
        if wait_stats is not None:
            call.wait_stats = wait_stats
        if self.profile is not None:
            call.prof = self.profile['ll_dispatch']
        call.mask = ll['mask']
        call.shrink = self.low_latency_shrink
        return call, sf_view

    def low_latency_dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, num_max_dispatch_tokens_per_rank: int,
                             num_experts: int, cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                             dispatch_wait_recv_cost_stats: Optional[torch.Tensor] = None, use_fp8: bool = True,
                             round_scale: bool = False, use_ue8m0: bool = False, async_finish: bool = False,
                             return_recv_hook: bool = False, num_sms: int = 0):
        """-> ``(recv_x | (recv_x, recv_scales), recv_count, handle, event, hook)``.

        ``recv_x [E_local, ranks * max_tokens, H]`` (e4m3 with ``use_fp8`` else bf16), ``recv_scales
        [E_local, ranks * max_tokens, H / 128]`` fp32 (or ``H / 512`` int32 of packed UE8M0) column-major in the
        last two dims, ``recv_count [E_local]``; only the first ``recv_count[e]`` rows of expert ``e`` are valid.
        ``handle = (src_info, layout_range, max_tokens, hidden, num_experts)``.
        """
        M, E = num_max_dispatch_tokens_per_rank, num_experts
        if self.is_cpu:
            return self._cpu_coll.low_latency_dispatch(x, topk_idx, M, E, cumulative_local_expert_recv_stats, use_fp8, round_scale,
                                                       use_ue8m0)
        C = self._C
        num_sms = self._ll_num_sms(num_sms)
        stream = torch.cuda.current_stream() if return_recv_hook else self.comm_stream
        if not return_recv_hook:
            stream.wait_stream(torch.cuda.current_stream())
        phases = 1 if return_recv_hook else 3
        with torch.cuda.stream(stream):
            call, sf_view = self._ll_prepare_dispatch(x, topk_idx, M, E, cumulative_local_expert_recv_stats,
                                                      dispatch_wait_recv_cost_stats, use_fp8, round_scale, use_ue8m0, phases)
            C.ll_dispatch_group([self.core], [call], num_sms)
        handle = (call.packed_src_info, call.layout_range, M, x.shape[1], E)
        recv_x = (call.packed_x, sf_view) if use_fp8 else call.packed_x
        event, hook = EventOverlap(None), None
        if return_recv_hook:
            def hook():
                call.phases = 2
                C.ll_dispatch_group([self.core], [call], num_sms)
        elif async_finish:
            event = EventOverlap(EventHandle(stream, (call.packed_x,)))
        else:
            torch.cuda.current_stream().wait_stream(stream)
        return recv_x, call.packed_count, handle, event, hook

    # ------------------------------------------------------------------------------------------ combine
    def _ll_prepare_combine(self, x, topk_idx, topk_weights, handle, out, wait_stats, phases, use_logfmt=False):
        C = self._C
        src_info, layout_range, M, H, E = handle
        K = topk_idx.shape[1]
        ll = self._ll_setup(M, H, E, K)
        call = C.LLCombineCall()
        call.x = x
        call.topk_idx, call.topk_weights = topk_idx.contiguous(), topk_weights.contiguous()
        call.src_info, call.layout_range = src_info, layout_range
        call.out = out if out is not None else torch.empty((topk_idx.shape[0], H), dtype=torch.bfloat16, device=x.device)
        call.num_experts, call.num_max_tokens = E, M
        call.phases = phases
        call.off_slab0, call.off_slab1 = ll['combine'][0], ll['combine'][1]
        if wait_stats is not None:
            call.wait_stats = wait_stats
        if self.profile is not None:
            call.prof = self.profile['ll_combine']
        call.mask = ll['mask']
        call.shrink = self.low_latency_shrink
        call.use_logfmt = bool(use_logfmt)
        return call

    def low_latency_combine(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, handle: tuple,
                            use_logfmt: bool = False, zero_copy: bool = False, async_finish: bool = False,
                            return_recv_hook: bool = False, out: Optional[torch.Tensor] = None,
                            combine_wait_recv_cost_stats: Optional[torch.Tensor] = None, num_sms: int = 0):
        """-> ``(combined_x [T, H] bf16 = sum_k topk_weights[t, k] * x_k, event, hook)``.

        ``x [E_local, ranks * max_tokens, H]`` bf16 holds the expert outputs in the packed order of the dispatch.
        Rows are read in place from ``x`` whether or not it came from :meth:`get_next_low_latency_combine_buffer`, so
        ``zero_copy`` changes nothing here.  With ``use_logfmt`` the rows cross the wire as LogFMT-10: 10-bit
        logarithmic codes with one range per 128 channels (36 % fewer bytes; ``H`` must be a multiple of 128), coded by
        the sender and decoded inside the weighted reduction
        (csrc/kernels/legacy/internode_ll.cu:556-712 of the reference; ``utils.math.logfmt10_roundtrip`` states the code).
        """
        if self.is_cpu:
            return self._cpu_coll.low_latency_combine(x, topk_idx, topk_weights, handle, use_logfmt, out)
        C = self._C
        num_sms = self._ll_num_sms(num_sms)
        stream = torch.cuda.current_stream() if return_recv_hook else self.comm_stream
        if not return_recv_hook:
            stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            call = self._ll_prepare_combine(x, topk_idx, topk_weights, handle, out, combine_wait_recv_cost_stats,
                                            1 if return_recv_hook else 3, use_logfmt)
            C.ll_combine_group([self.core], [call], num_sms)
        event, hook = EventOverlap(None), None
        if return_recv_hook:
            def hook():
                call.phases = 2
                C.ll_combine_group([self.core], [call], num_sms)
        elif async_finish:
            event = EventOverlap(EventHandle(stream, (call.out,)))
        else:
            torch.cuda.current_stream().wait_stream(stream)
        return call.out, event, hook

    def get_next_low_latency_combine_buffer(self, handle: tuple) -> torch.Tensor:
        """The bf16 ``[E_local, ranks * max_tokens, H]`` tensor that the expert outputs of the next combine should be
        written to.  The combine kernel reads its input rows in place wherever they live, so no copy is saved or added by
        using it; what it gives is ONE allocation with a stable address that is reused by every call (the two sets alternate
        like the kernels' own buffer sets), which is what a captured CUDA graph needs."""
        if self.is_cpu:
            return self._cpu_coll.get_next_low_latency_combine_buffer(handle)
        _, _, M, H, E = handle
        ll = self._ll
        assert ll is not None, 'a handle comes from low_latency_dispatch, which sets the low-latency regions up'
        if 'combine_x' not in ll:
            shape = (E // self.num_ranks, self.num_ranks * M, H)
            ll['combine_x'] = [torch.empty(shape, dtype=torch.bfloat16, device='cuda') for _ in range(2)]
            ll['combine_x_next'] = 0
        buf = ll['combine_x'][ll['combine_x_next'] & 1]
        ll['combine_x_next'] += 1
        return buf

    # ------------------------------------------------------------------------------------------ shrink mode
    low_latency_shrink = False

    def low_latency_update_mask_buffer(self, rank_to_mask: int, mask: bool = False) -> None:
        """Mark a rank as failed (``mask=True``) or healthy; masked ranks are skipped by both kernels."""
        if self.is_cpu:
            self._cpu_coll.mask()[rank_to_mask] = 1 if mask else 0
            return
        assert self._ll is not None, 'run a low-latency call (or _ll_setup) first'
        self._ll['mask'][rank_to_mask] = 1 if mask else 0

    def low_latency_query_mask_buffer(self, mask_status: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.is_cpu:
            if mask_status is None:
                return self._cpu_coll.mask().clone()
            mask_status.copy_(self._cpu_coll.mask())
            return mask_status
        assert self._ll is not None
        if mask_status is None:
            return self._ll['mask'].clone()
        mask_status.copy_(self._ll['mask'])
        return mask_status

    def low_latency_clean_mask_buffer(self) -> None:
        if self.is_cpu:
            self._cpu_coll.mask().zero_()
            return
        if self._ll is not None:
            self._ll['mask'].zero_()

    def clean_low_latency_buffer(self, num_max_dispatch_tokens_per_rank: int = 0, hidden: int = 0, num_experts: int = 0) -> None:
        """Nothing to clean: every signal word of the low-latency protocol carries the call number it belongs
        to, so stale contents are never mistaken for new data.  Kept for API parity."""
        return None
