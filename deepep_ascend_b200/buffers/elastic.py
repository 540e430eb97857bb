"""``ElasticBuffer``: expert-parallel dispatch / combine over one NVLink domain, with the call signatures of
deep_ep's class of the same name (deep_ep/buffers/elastic.py:298-1712).

How it differs from the reference by design:

* one fused kernel per call; dispatch writes rows straight into the receivers' final output tensors (which
  live in the symmetric buffer) and combine pulls + reduces in one pass, so there are no epilogue kernels;
* the row layout is deterministic (ordered by source rank, then token), so ``deterministic=True`` costs nothing;
* dispatch can fuse the bf16 -> e4m3 (1x128 scales) cast (``use_fp8_dispatch=True`` with bf16 input);
* combine can fuse the top-k weighting (``weighted=True`` in expand layout);
* outputs of dispatch are views into one of ``num_recv_slots`` receive regions and stay valid until that
  region is reused, i.e. for ``num_recv_slots - 1`` further dispatches (``zero_copy=False`` returns copies);
* device waits are bounded and report through a status block; a failed wait poisons the buffer.

The same class runs on CPU tensors with a gloo group (``backends/cpu.py``) with identical handle semantics.
"""
import itertools
import math
import os
from typing import List, Optional, Tuple, Union

import torch
import torch.distributed as dist

from ..ops import layout_ref
from .low_latency import LowLatencyMixin
from .collectives import CollectivesMixin
from ..utils.comm import all_gather_object
from ..utils.event import EventHandle, EventOverlap
from ..utils.math import align
from ..utils.semantic import value_or

topk_idx_t = torch.int64 if int(os.environ.get('EP_NUM_TOPK_IDX_BITS', '64')) == 64 else torch.int32

_comm_streams = {}
_buffer_uids = itertools.count(1)


class HandleError(RuntimeError):
    """A handle was given to a buffer it does not belong to (another buffer, a destroyed or re-created one, or a
    call whose shape differs from the dispatch that made it)."""


def _get_comm_stream() -> 'torch.cuda.Stream':
    """Process-wide high-priority communication stream of the current device."""
    dev = torch.cuda.current_device()
    if dev not in _comm_streams:
        _comm_streams[dev] = torch.cuda.Stream(priority=-1)
    return _comm_streams[dev]


class EPHandle:
    """What ``dispatch`` returns for ``combine`` (and for cached re-dispatch).

    Attributes kept from the reference handle (deep_ep/buffers/elastic.py:40-113): ``do_expand, num_experts,
    expert_alignment, num_max_tokens_per_rank, num_sms, topk_idx, num_recv_tokens, num_expanded_tokens,
    num_recv_tokens_per_expert_list, psum_num_recv_tokens_per_scaleup_rank, psum_num_recv_tokens_per_expert,
    num_unaligned_recv_tokens_per_expert, recv_src_metadata, dst_buffer_slot_idx``.

    ``dst_buffer_slot_idx [T, K] int32`` packs ``(dst_rank << 24) | row`` per top-k lane (-1 for empty lanes);
    ``plan [T, K]`` keeps only the lanes that move a row.  ``recv_src_metadata [rows, 2] int32`` holds, per
    received row, ``src_rank * num_max_tokens_per_rank + src_token`` and ``src_rank * K + lane``.
    ``psum_num_recv_tokens_per_expert`` is the inclusive prefix sum of alignment-padded counts (non-expand), or
    the end row of each expert's segment (expand; segment i starts at ``align(psum[i-1], expert_alignment)``).
    """

    def __init__(self, do_expand: bool, num_experts: int, expert_alignment: int, num_max_tokens_per_rank: int,
                 num_sms: int, topk_idx: torch.Tensor, num_recv_tokens: int, num_expanded_tokens: int,
                 num_recv_tokens_per_expert_list: Optional[list], psum_num_recv_tokens_per_scaleup_rank: torch.Tensor,
                 psum_num_recv_tokens_per_expert: torch.Tensor, num_unaligned_recv_tokens_per_expert: torch.Tensor,
                 recv_src_metadata: torch.Tensor, dst_buffer_slot_idx: torch.Tensor, plan: torch.Tensor,
                 hidden: int, recv_slot: int, topk_weights: Optional[torch.Tensor] = None,
                 stamp: Optional[tuple] = None):
        self.do_expand = do_expand
        self.num_experts = num_experts
        self.expert_alignment = expert_alignment
        self.num_max_tokens_per_rank = num_max_tokens_per_rank
        self.num_sms = num_sms
        self.topk_idx = topk_idx
        self.num_recv_tokens = num_recv_tokens
        self.num_expanded_tokens = num_expanded_tokens
        self.num_recv_tokens_per_expert_list = num_recv_tokens_per_expert_list
        self.psum_num_recv_tokens_per_scaleup_rank = psum_num_recv_tokens_per_scaleup_rank
        self.psum_num_recv_tokens_per_expert = psum_num_recv_tokens_per_expert
        self.num_unaligned_recv_tokens_per_expert = num_unaligned_recv_tokens_per_expert
        self.recv_src_metadata = recv_src_metadata
        self.dst_buffer_slot_idx = dst_buffer_slot_idx
        self.plan = plan
        self.hidden = hidden
        self.recv_slot = recv_slot
        self.topk_weights = topk_weights
        # (buffer uid, buffer generation, num_ranks, num_tokens, num_topk): checked by every call that takes a handle
        # (the role of the reference's handle attestation, csrc/backends/ascend/elastic/dispatch_state.hpp:221-480)
        self.stamp = stamp
        self.token_metadata_at_forward = None      # multi-node only
        self.channel_linked_list = None            # multi-node only

    @property
    def num_tokens(self) -> int:
        return self.topk_idx.shape[0]

    @property
    def num_topk(self) -> int:
        return self.topk_idx.shape[1]

    @property
    def num_rows(self) -> int:
        """Rows the combine input must have."""
        return self.num_expanded_tokens if self.do_expand else self.num_recv_tokens


class _DispatchState:
    """Book-keeping between the three steps of a dispatch (prepare -> launch -> finish)."""
    __slots__ = ('call', 'T', 'H', 'K', 'E', 'fp8_out', 'do_expand', 'alignment', 'slot_idx', 'slot', 'handle_tensors',
                 'topk_idx', 'topk_weights', 'do_cpu_sync', 'num_sms', 'col_major_sf', 'cached_handle', 'x_dtype',
                 'keep_alive', 'do_handle_copy', 'side')


class ElasticBuffer(LowLatencyMixin, CollectivesMixin):
    """Symmetric communication buffer for one expert-parallel group (one process per GPU, or CPU ranks on gloo).

    Arguments follow deep_ep (deep_ep/buffers/elastic.py:331-349).  ``num_bytes`` overrides the size derived
    from the MoE shape; ``enable_expand`` / ``num_experts`` / ``expert_alignment`` size the receive regions for
    the expand layout; ``extra_bytes`` reserves room behind the MoE regions for all-gather sessions, pipeline
    FIFOs, Engram storage and the low-latency buffers.  ``num_cpu_bytes`` reserves pinned host memory, mapped into
    this GPU's address space, behind the device buffer: Engram storage that does not fit the GPU region goes there
    (deep_ep/buffers/elastic.py:511-516, csrc/kernels/backend/symmetric.hpp:145-186).  One NVLink domain has no NIC
    path, so the RDMA-only arguments must keep their defaults: ``num_allocated_qps=0`` and ``sl_idx=3`` (anything else
    raises ``ValueError`` instead of being silently dropped).  ``symmetric_memory`` selects how the buffer is allocated and
    shared with the peers: ``'ipc'`` = ``cudaMalloc`` + ``cudaIpc`` handles, ``'vmm'`` = ``cuMemCreate`` / ``cuMemMap`` with the
    allocation's POSIX file descriptor passed over a Unix-domain socket (csrc/kernels/backend/symmetric.hpp:22-87 of the reference).
    """

    def __init__(self, group: Optional[dist.ProcessGroup], num_bytes: Optional[int] = None, num_cpu_bytes: int = 0,
                 num_max_tokens_per_rank: int = 0, hidden: int = 0, num_topk: int = 0, use_fp8_dispatch: bool = False,
                 deterministic: bool = False, allow_hybrid_mode: bool = True, allow_multiple_reduction: bool = True,
                 prefer_overlap_with_compute: bool = True, sl_idx: int = 3, num_allocated_qps: int = 0,
                 num_cpu_timeout_secs: float = 300, num_gpu_timeout_secs: float = 100, explicitly_destroy: bool = False,
                 enable_expand: bool = False, num_experts: int = 0, expert_alignment: int = 1, num_recv_slots: int = 2,
                 extra_bytes: int = 0, zero_copy: bool = True, low_latency_shrink: bool = False,
                 symmetric_memory: str = 'ipc', _virtual: Optional[Tuple[int, int]] = None):
        if symmetric_memory not in ('ipc', 'vmm'):
            raise ValueError("symmetric_memory must be 'ipc' (cudaMalloc + cudaIpc handles) or 'vmm' (CUDA virtual memory "
                             "allocation shared as a POSIX file descriptor)")
        if num_allocated_qps != 0 or sl_idx != 3:
            raise ValueError('num_allocated_qps / sl_idx configure RDMA queue pairs; a single NVLink domain has none '
                             '(leave them at their defaults)')
        if num_cpu_bytes < 0:
            raise ValueError('num_cpu_bytes must not be negative')
        self.group = group
        self._virtual = _virtual
        self.low_latency_shrink = low_latency_shrink
        self._ll = None
        self._agrs = self._pp = self._engram = None
        self.profile = None
        self._kernel_timing = None
        self._tune = (0, 0)
        self._side_aligned = False
        if _virtual is not None:
            self.rank_idx, self.num_ranks = _virtual
        else:
            self.rank_idx = dist.get_rank(group) if group is not None else 0
            self.num_ranks = dist.get_world_size(group) if group is not None else 1
        self.num_max_tokens_per_rank = num_max_tokens_per_rank
        self.hidden = hidden
        self.num_topk = num_topk
        self.use_fp8_dispatch = use_fp8_dispatch
        self.deterministic = deterministic
        self.allow_hybrid_mode = allow_hybrid_mode
        self.allow_multiple_reduction = allow_multiple_reduction
        self.prefer_overlap_with_compute = prefer_overlap_with_compute
        self.explicitly_destroy = explicitly_destroy
        self.zero_copy = zero_copy
        self.enable_expand = enable_expand
        self.num_cpu_bytes = num_cpu_bytes
        self.num_scaleout_ranks, self.num_scaleup_ranks = 1, self.num_ranks
        self.num_rdma_ranks, self.num_nvlink_ranks = 1, self.num_ranks
        self._destroyed = False
        self._recv_slot_counter = 0
        self._combine_slot_counter = 0
        self._sm_cache = {}
        self._uid = next(_buffer_uids)

        backend = dist.get_backend(group) if (group is not None and _virtual is None) else None
        self.is_cpu = (backend == 'gloo') or not torch.cuda.is_available()
        if self.is_cpu:
            from ..backends.cpu import CpuBackend
            self._cpu = CpuBackend(group, self.rank_idx, self.num_ranks)
            from ..backends.cpu_collectives import CpuCollectives
            self._cpu_coll = CpuCollectives(group, self.rank_idx, self.num_ranks)
            self.low_latency_shrink = low_latency_shrink
            self.core = None
            self.regions = None
            return

        from .. import _native
        self._C = _native.load()
        shape = self._C.MoeShape()
        shape.num_ranks = self.num_ranks
        shape.num_max_tokens_per_rank = num_max_tokens_per_rank
        shape.hidden = hidden
        shape.num_topk = max(1, num_topk)
        shape.num_experts_hint = num_experts
        shape.expert_alignment = expert_alignment
        shape.use_fp8_dispatch = use_fp8_dispatch
        shape.enable_expand = enable_expand
        shape.num_recv_slots = num_recv_slots
        self.regions = self._C.plan_regions(shape)
        alignment = self._C.get_elastic_buffer_alignment()
        moe_bytes = self.regions.moe_bytes
        total = align(max(value_or(num_bytes, 0) + self._C.get_workspace_bytes(), moe_bytes) + extra_bytes, alignment)
        self.num_bytes = total
        self.extra_offset = align(self.regions.extra, 1024)
        self.extra_bytes = total - self.extra_offset
        self._extra_cursor = self.extra_offset
        if os.environ.get('EP_BUFFER_DEBUG'):
            print(f'[EP rank {self.rank_idx}] symmetric buffer {total / 2**20:.1f} MiB '
                  f'(MoE regions {moe_bytes / 2**20:.1f} MiB, capacity {self.regions.capacity_rows} rows, '
                  f'{num_recv_slots} receive slots, {num_cpu_bytes / 2**20:.1f} MiB mapped host memory)', flush=True)
        extra_args = (int(num_cpu_bytes), True) if symmetric_memory == 'vmm' else ((int(num_cpu_bytes),) if num_cpu_bytes else ())
        self.core = self._C.ElasticBuffer(self.rank_idx, self.num_ranks, total, float(num_gpu_timeout_secs),
                                          float(num_cpu_timeout_secs), *extra_args)
        self.symmetric_memory = symmetric_memory
        if _virtual is None:
            if self.num_ranks > 1:
                handles = all_gather_object(group, bytes(self.core.get_local_ipc_handle()))
                self.core.open_peers(handles)
                if num_cpu_bytes > 0:
                    self.core.open_cpu_peers(all_gather_object(group, self.core.get_local_cpu_segment_name()))
            torch.cuda.synchronize()
            if group is not None and self.num_ranks > 1:
                dist.barrier(group=group)
            if num_cpu_bytes > 0:
                self.core.unlink_cpu_segment_name()      # every rank has mapped it; the mappings keep it alive
            if symmetric_memory == 'vmm':
                self.core.finish_export()                # every peer has fetched the descriptor
        self.comm_stream = _get_comm_stream()
        # combine launches on this stream; it is the communication stream unless a caller that overlaps dispatches of one
        # batch with combines of another (a pipelined MoE layer) gives combine a stream of its own
        self.combine_stream = self.comm_stream

    # ------------------------------------------------------------------------------------------ extra region
    def reserve(self, num_bytes: int, alignment: int = 1024) -> int:
        """Carve ``num_bytes`` out of the region behind the MoE buffers (``extra_bytes`` at construction) and
        return its byte offset.  Every rank must make the same sequence of calls."""
        off = align(self._extra_cursor, alignment)
        if off + num_bytes > self.num_bytes:
            raise RuntimeError(f'symmetric buffer too small: need {num_bytes} more bytes behind offset {off} of '
                               f'{self.num_bytes}; pass a larger `extra_bytes`')
        self._extra_cursor = off + num_bytes
        return off

    # ------------------------------------------------------------------------------------------ life cycle
    def destroy(self) -> None:
        """Release the symmetric buffer.  Collective when the group has more than one rank."""
        if self._destroyed:
            return
        if not self.is_cpu:
            torch.cuda.synchronize()
            if self.group is not None and self.num_ranks > 1 and dist.is_initialized():
                try:
                    dist.barrier(group=self.group)
                except Exception:
                    pass
            self.core.destroy()
        self._destroyed = True

    def __del__(self):
        try:
            if not self._destroyed and not self.is_cpu and self.core is not None:
                if self.explicitly_destroy:
                    print('WARNING: ElasticBuffer.destroy() was not called before the buffer was dropped', flush=True)
                self.core.destroy()
        except Exception:
            pass

    # ------------------------------------------------------------------------------------------ hints
    @staticmethod
    def get_buffer_size_hint(group: Optional[dist.ProcessGroup], num_max_tokens_per_rank: int, hidden: int,
                             num_topk: int = 0, use_fp8_dispatch: bool = False, allow_hybrid_mode: bool = True,
                             allow_multiple_reduction: bool = True, enable_expand: bool = False, num_experts: int = 0,
                             expert_alignment: int = 1, num_recv_slots: int = 2, num_ranks: Optional[int] = None) -> int:
        """Bytes (2 MiB aligned, workspace included) that a buffer for this MoE shape needs."""
        from .. import _native
        C = _native.load()
        shape = C.MoeShape()
        shape.num_ranks = num_ranks if num_ranks is not None else (dist.get_world_size(group) if group is not None else 1)
        shape.num_max_tokens_per_rank = num_max_tokens_per_rank
        shape.hidden = hidden
        shape.num_topk = max(1, num_topk)
        shape.num_experts_hint = num_experts
        shape.expert_alignment = expert_alignment
        shape.use_fp8_dispatch = use_fp8_dispatch
        shape.enable_expand = enable_expand
        shape.num_recv_slots = num_recv_slots
        return C.calculate_elastic_buffer_size(shape)

    @staticmethod
    def get_engram_storage_size_hint(num_entries: int, hidden: int, num_max_tokens_per_rank: int,
                                     dtype: torch.dtype = torch.bfloat16) -> Tuple[int, int]:
        a = 2 << 20
        per_entry = align(hidden * dtype.itemsize, 32)
        return align(per_entry * num_max_tokens_per_rank, a), align(per_entry * num_entries, a)

    @staticmethod
    def get_pp_buffer_size_hint(num_max_tensor_bytes: int, num_max_inflight_tensors: int) -> int:
        return align(align(num_max_tensor_bytes, 32) * num_max_inflight_tensors * 2 * 2, 2 << 20)

    @staticmethod
    def get_agrs_num_max_session_bytes(group: dist.ProcessGroup, shapes, dtype: torch.dtype) -> int:
        if not isinstance(shapes[0], (tuple, list, torch.Size)):
            shapes = (shapes,)
        n = dist.get_world_size(group) if group is not None else 1
        return sum(align(n * math.prod(s) * dtype.itemsize, 32) for s in shapes)

    @staticmethod
    def get_agrs_buffer_size_hint(group: dist.ProcessGroup, num_max_session_bytes: int) -> int:
        return align(num_max_session_bytes, 2 << 20)

    def get_comm_stream(self) -> 'torch.cuda.Stream':
        return self.comm_stream

    def get_physical_domain_size(self) -> Tuple[int, int]:
        return 1, self.num_ranks

    def get_logical_domain_size(self) -> Tuple[int, int]:
        return 1, self.num_ranks

    # ------------------------------------------------------------------------------------------ SM model
    def get_theoretical_num_sms(self, num_experts: int, num_topk: int, num_scaleout_topk: int = 0, rdma_gbs: float = 0,
                                nvlink_gbs: float = 0, sm_read_gbs: float = 0, sm_write_gbs: float = 0) -> int:
        """SM count for dispatch / combine from a bandwidth model: enough SMs that the per-SM NVLink issue rate
        is not the bottleneck, times 1.25 headroom, even, at least 4; at least 64 when the caller does not want
        to overlap with compute (same rule as deep_ep/buffers/elastic.py:1253-1369, constants re-measured on
        B200 in ``ops/sm_model.py``)."""
        from ..ops.sm_model import theoretical_num_sms
        key = (num_experts, num_topk, nvlink_gbs, sm_read_gbs, sm_write_gbs)
        if key not in self._sm_cache:
            device_sms = 148 if self.is_cpu else torch.cuda.get_device_properties('cuda').multi_processor_count
            self._sm_cache[key] = theoretical_num_sms(self.num_ranks, num_experts, num_topk, nvlink_gbs, sm_read_gbs,
                                                      sm_write_gbs, self.prefer_overlap_with_compute, device_sms)
        return self._sm_cache[key]

    def get_theoretical_num_qps(self, num_sms: int) -> int:
        """No RDMA queue pairs exist inside one NVLink domain: always 0 (pass that as ``num_qps``)."""
        return 0

    def set_dispatch_tuning(self, num_warps: int = 0, num_stages: int = 0, line_aligned_side: Optional[bool] = None) -> None:
        """Shape of the dispatch kernel: warps per CTA (1..12, each with its own staging ring) and, for the fused
        FP8 cast, staging buffers per warp (2..4; more buffers keep more tokens' stores in flight per warp but
        leave room for fewer warps).  0 selects the default (12 warps, 2 buffers).  ``line_aligned_side``: place every
        row's scales and tail record on 128-byte boundaries at the receiver (``recv_sf`` and ``recv_topk_idx`` /
        ``recv_topk_weights`` become row-strided views), so that each of these small stores is whole lines on the wire."""
        assert 0 <= num_warps <= 12 and num_stages in (0, 2, 3, 4)
        self._tune = (num_warps, num_stages)
        if line_aligned_side is not None:
            self._side_aligned = bool(line_aligned_side)

    # ------------------------------------------------------------------------------------------ barrier
    def barrier(self, use_comm_stream: bool = True, with_cpu_sync: bool = False, sequential: bool = True) -> None:
        """GPU-side barrier over all ranks (signals over NVLink), optionally followed by a host sync."""
        if self.is_cpu:
            dist.barrier(group=self.group)
            return
        stream = self.comm_stream if use_comm_stream else torch.cuda.current_stream()
        if use_comm_stream:
            stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            self.core.barrier()
        if use_comm_stream:
            torch.cuda.current_stream().wait_stream(stream)
        if with_cpu_sync:
            stream.synchronize()
            self.core.check_status()

    # ------------------------------------------------------------------------------------------ layout
    def get_dispatch_layout(self, topk_idx: torch.Tensor, num_experts: int, previous_event: Optional[EventHandle] = None,
                            async_finish: bool = False, allocate_on_comm_stream: bool = False):
        """Routing summary of ``topk_idx [T, K]`` (``-1`` = no selection), computed by one sm_100a kernel.

        Returns ``(num_tokens_per_rank int32 [ranks], num_tokens_per_rdma_rank (always None: one NVLink domain),
        num_tokens_per_expert int32 [num_experts], is_token_in_rank bool [T, ranks], event)``, the tuple of the
        reference's ``Buffer.get_dispatch_layout`` (deep_ep/buffers/legacy.py:293-319).  ``dispatch`` does not
        need it (it counts inside its kernel); it is for callers that size or balance work before dispatching.
        """
        assert num_experts % self.num_ranks == 0
        if self.is_cpu:
            lay = layout_ref.dispatch_layout(topk_idx, num_experts, self.num_ranks)
            return lay[0], None, lay[1], lay[2], EventOverlap(None)
        if previous_event is not None and not allocate_on_comm_stream:
            raise ValueError('`previous_event` requires `allocate_on_comm_stream=True`')
        self._stream_prologue(previous_event, None)
        with torch.cuda.stream(self.comm_stream):
            idx = topk_idx.contiguous()
            per_rank, per_expert, in_rank = self._C.get_dispatch_layout(idx, num_experts, self.num_ranks)
        event = self._stream_epilogue(async_finish, (per_rank, per_expert, in_rank), (idx, topk_idx))
        return per_rank, None, per_expert, in_rank, event

    # ------------------------------------------------------------------------------------------ handles
    def _stamp(self, T: int, K: int) -> tuple:
        gen = 0 if self.is_cpu else int(self.core.generation())
        return (self._uid, gen, self.num_ranks, T, K)

    def _attest(self, handle: EPHandle, what: str) -> None:
        """Reject a handle that this buffer did not make: another buffer's, one from before this buffer was destroyed
        or poisoned, or one whose recorded shape does not fit.  Raised on the host, before anything is launched."""
        stamp = getattr(handle, 'stamp', None)
        where = f'[EP rank {self.rank_idx}] {what}'
        if stamp is None:
            raise HandleError(f'{where}: the handle carries no buffer stamp (it was not returned by ElasticBuffer.dispatch)')
        uid, _gen, ranks, T, K = stamp
        if uid != self._uid:
            raise HandleError(f'{where}: the handle belongs to another buffer (buffer id {uid}, this buffer is {self._uid})')
        if self._destroyed:
            raise HandleError(f'{where}: the buffer that made this handle has been destroyed')
        if ranks != self.num_ranks or tuple(handle.plan.shape) != (T, K) or tuple(handle.dst_buffer_slot_idx.shape) != (T, K):
            raise HandleError(f'{where}: the handle was made for {ranks} ranks and [{T}, {K}] selections, which does not fit '
                              f'this call ({self.num_ranks} ranks, plan {tuple(handle.plan.shape)})')
        if not self.is_cpu and self.core.state() == 'poisoned':
            raise HandleError(f'{where}: the buffer is poisoned by an earlier failure; handles made by it are void')

    # ------------------------------------------------------------------------------------------ dispatch
    def dispatch(self, x: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]], topk_idx: Optional[torch.Tensor] = None,
                 topk_weights: Optional[torch.Tensor] = None,
                 cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None, num_experts: Optional[int] = None,
                 num_max_tokens_per_rank: Optional[int] = None, expert_alignment: Optional[int] = None,
                 num_sms: int = 0, num_qps: int = 0, previous_event: Optional[EventHandle] = None,
                 previous_event_before_epilogue: Optional[EventHandle] = None, async_with_compute_stream: bool = False,
                 allocate_on_comm_stream: bool = False, handle: Optional[EPHandle] = None, do_handle_copy: bool = True,
                 do_cpu_sync: Optional[bool] = None, do_expand: bool = False, do_zero_padding: bool = False,
                 use_tma_aligned_col_major_sf: bool = False, fused_fp8_cast: Optional[bool] = None):
        """Send every token to the ranks that own its selected experts.

        Returns ``(recv_x | (recv_x, recv_sf), recv_topk_idx, recv_topk_weights, handle, event)`` with the
        reference's meaning (deep_ep/buffers/elastic.py:1391-1603): non-expand layout gives one row per
        (token, destination rank) with expert ids localised to the receiver; ``do_expand`` gives one row per
        (token, local expert), grouped by expert with aligned group starts, ``recv_topk_idx`` is ``None`` and
        ``recv_topk_weights`` is 1-D; ``do_zero_padding`` makes the kernel zero the rows between an expert's last
        row and its aligned end.  With ``do_cpu_sync`` (default unless a cached ``handle`` is passed) the
        tensors have the exact number of rows; otherwise they have the worst-case size and
        ``handle.psum_num_recv_tokens_per_scaleup_rank[-1]`` holds the valid row count on the device.
        With ``use_fp8_dispatch`` (or ``fused_fp8_cast=True`` for this call) and bf16 input the e4m3 cast is fused into
        the kernel; ``fused_fp8_cast=False`` sends bf16 rows even on an FP8 buffer (backward passes).

        Streams (csrc/elastic/buffer.hpp:528-586 of the reference): the kernel runs on the communication stream, which
        first waits for ``previous_event`` (this needs ``allocate_on_comm_stream=True``) or else for the work the
        current stream has been given so far, and for ``previous_event_before_epilogue`` if given (the reference lets
        that event gate only its second kernel; here placement is part of the one kernel, so it gates the launch).
        Handle and output tensors are allocated with the communication stream current when
        ``allocate_on_comm_stream``, otherwise with the caller's stream current.  With ``async_with_compute_stream``
        the returned event must be waited for before the results are used; otherwise the current stream waits.
        ``num_qps`` must be 0 (there are no queue pairs inside one NVLink domain).
        """
        assert not self._destroyed
        if num_qps != 0:
            raise ValueError('num_qps must be 0: there are no RDMA queue pairs inside one NVLink domain')
        if previous_event is not None and not allocate_on_comm_stream:
            raise ValueError('`previous_event` requires `allocate_on_comm_stream=True`')
        if handle is not None:
            assert topk_idx is None, '`topk_idx` comes from the cached handle'
            self._attest(handle, 'cached dispatch')
            num_experts = handle.num_experts
            expert_alignment = handle.expert_alignment
            do_expand = handle.do_expand
            num_max_tokens_per_rank = handle.num_max_tokens_per_rank
            do_cpu_sync = False if do_cpu_sync is None else do_cpu_sync
            assert not do_cpu_sync, 'a cached dispatch already knows its sizes'
        do_cpu_sync = value_or(do_cpu_sync, True)
        assert not do_zero_padding or do_expand, '`do_zero_padding` requires `do_expand` (or a cached expand handle)'
        assert num_experts is not None and num_experts % self.num_ranks == 0
        num_max_tokens_per_rank = value_or(num_max_tokens_per_rank, self.num_max_tokens_per_rank)
        expert_alignment = value_or(expert_alignment, 1)

        if self.is_cpu:
            return self._cpu.dispatch(self, x, topk_idx, topk_weights, cumulative_local_expert_recv_stats, num_experts,
                                      num_max_tokens_per_rank, expert_alignment, handle, do_expand, do_zero_padding,
                                      do_handle_copy)

        K = (handle.topk_idx if topk_idx is None else topk_idx).shape[1]
        num_sms = self.get_theoretical_num_sms(num_experts, K) if num_sms == 0 else num_sms
        alloc_stream = self.comm_stream if allocate_on_comm_stream else torch.cuda.current_stream()
        if allocate_on_comm_stream:
            self._stream_prologue(previous_event, previous_event_before_epilogue)
        with torch.cuda.stream(alloc_stream):
            st = self._prepare_dispatch(x, topk_idx, topk_weights, cumulative_local_expert_recv_stats, num_experts,
                                        num_max_tokens_per_rank, expert_alignment, num_sms, handle, do_handle_copy,
                                        do_cpu_sync, do_expand, use_tma_aligned_col_major_sf, fused_fp8_cast,
                                        do_zero_padding)
        if not allocate_on_comm_stream:
            # input copies made while preparing ran on the caller's stream: wait for them too
            self._stream_prologue(previous_event, previous_event_before_epilogue)
        with torch.cuda.stream(self.comm_stream):
            self._timed('dispatch', lambda: self.core.dispatch(st.call, num_sms))
            out = self._finish_dispatch(st)
        inputs = (st.call.x, st.call.sf, st.call.topk_idx, st.call.topk_weights, st.call.stats, st.call.lane_src,
                  st.call.plan, st.call.psum_rank, st.call.psum_expert, st.call.recv_per_expert, x, topk_idx, topk_weights)
        event = self._stream_epilogue(async_with_compute_stream, out, inputs)
        return (*out, event)

    def _next_recv_slot(self) -> int:
        slot = self._recv_slot_counter % self.regions.num_recv_slots
        self._recv_slot_counter += 1
        return slot

    def _prepare_dispatch(self, x, topk_idx, topk_weights, stats, num_experts, num_max_tokens, alignment, num_sms, handle,
                          do_handle_copy, do_cpu_sync, do_expand, col_major_sf, fused_fp8_cast=None,
                          do_zero_padding=False) -> _DispatchState:
        C = self._C
        x_in, sf_in = x if isinstance(x, tuple) else (x, None)
        T, H = x_in.shape
        cached = handle is not None
        idx = handle.topk_idx if cached else topk_idx
        assert idx.dtype in (torch.int64, torch.int32)
        K = idx.shape[1]
        R, El = self.num_ranks, num_experts // self.num_ranks
        quantize = (self.use_fp8_dispatch if fused_fp8_cast is None else fused_fp8_cast) and x_in.dtype == torch.bfloat16
        assert H * (1 if quantize or x_in.dtype == torch.float8_e4m3fn else 2) <= self.regions.x_row_bytes, \
            'rows are wider than the receive regions: size the buffer with use_fp8_dispatch=False for bf16 rows'
        fp8_out = quantize or x_in.dtype == torch.float8_e4m3fn
        assert H <= self.hidden or self.hidden == 0, 'hidden exceeds what the buffer was sized for'
        assert not do_expand or self.enable_expand, 'construct the buffer with enable_expand=True for the expand layout'
        dev = x_in.device
        i32 = dict(dtype=torch.int32, device=dev)
        call = C.DispatchCall()
        call.x = x_in.contiguous()
        if sf_in is not None:
            call.sf = sf_in.contiguous().float() if sf_in.dtype != torch.float32 else sf_in.contiguous()
        call.topk_idx = idx.contiguous()
        if topk_weights is not None:
            call.topk_weights = topk_weights.contiguous()
        if stats is not None:
            call.stats = stats
        if cached:
            call.lane_src, call.plan = handle.dst_buffer_slot_idx, handle.plan
            call.psum_rank = handle.psum_num_recv_tokens_per_scaleup_rank
            call.psum_expert = handle.psum_num_recv_tokens_per_expert
            call.recv_per_expert = handle.num_unaligned_recv_tokens_per_expert
        else:
            call.lane_src = torch.empty((T, K), **i32)
            call.plan = torch.empty((T, K), **i32)
            call.psum_rank = torch.empty((R,), **i32)
            call.psum_expert = torch.empty((El,), **i32)
            call.recv_per_expert = torch.empty((El,), **i32)
        call.num_experts = num_experts
        call.expert_alignment = alignment
        call.num_max_tokens = num_max_tokens
        call.quantize = quantize
        call.do_expand = do_expand
        call.do_zero_padding = bool(do_zero_padding)
        call.cached = cached
        call.tune_warps, call.tune_stages = self._tune
        slot_idx = self._next_recv_slot()
        slot = self.regions.slot(slot_idx)
        cap = self.regions.capacity_rows
        call.off_recv_x, call.off_recv_sf, call.off_recv_idx = slot.x, slot.sf, slot.idx
        call.off_recv_w, call.off_recv_meta = slot.w, slot.meta
        G = (H + 127) // 128
        call.sf_stride_row, call.sf_stride_col = (1, cap) if col_major_sf else (G, 1)
        call.recv_capacity_rows = cap
        tail = None
        if not do_expand and not col_major_sf and (not fp8_out or (G * 4) % 16 == 0):
            # scales travel as one bulk store per row; expert ids (already relative to the receiver), weights and
            # source ids as one more: the tail record {ids | weights | metadata}
            off_w = K * idx.element_size()
            off_meta = align(off_w + K * 4, 8)
            tail_bytes = align(off_meta + 8, 16)
            tail_pitch = align(tail_bytes, 128) if self._side_aligned else tail_bytes
            sf_pitch = align(G * 4, 128) // 4 if self._side_aligned else G
            assert tail_pitch <= self.regions.tail_bytes and sf_pitch * 4 <= self.regions.sf_row_bytes, \
                'side records larger than the buffer was sized for'
            call.side_packed = True
            call.tail_bytes, call.tail_off_w, call.tail_off_meta, call.tail_pitch = tail_bytes, off_w, off_meta, tail_pitch
            call.sf_stride_row = sf_pitch
            call.off_recv_tail = slot.tail
            tail = (tail_pitch, off_w, off_meta, sf_pitch)
        if self.profile is not None:
            call.prof = self.profile['dispatch']

        st = _DispatchState()
        st.call, st.T, st.H, st.K, st.E = call, T, H, K, num_experts
        st.fp8_out, st.do_expand, st.alignment = fp8_out, do_expand, alignment
        st.slot_idx, st.slot = slot_idx, slot
        st.topk_idx, st.topk_weights = idx, topk_weights
        st.do_cpu_sync, st.num_sms, st.col_major_sf = do_cpu_sync, num_sms, col_major_sf
        st.cached_handle = handle
        st.x_dtype = x_in.dtype
        st.do_handle_copy = do_handle_copy
        st.side = tail
        return st

    def _finish_dispatch(self, st: _DispatchState):
        core, cap = self.core, self.regions.capacity_rows
        R, El = self.num_ranks, st.E // self.num_ranks
        K, H = st.K, st.H
        per_expert_list = None
        if st.cached_handle is not None:
            num_recv, num_expanded = st.cached_handle.num_recv_tokens, st.cached_handle.num_expanded_tokens
            per_expert_list = st.cached_handle.num_recv_tokens_per_expert_list
        elif st.do_cpu_sync:
            counts = core.wait_recv_counts(El)
            num_recv, num_expanded = counts[0], counts[1]
            per_expert_list = [align(c, st.alignment) for c in counts[2:]]
        else:
            num_recv = min(cap, R * st.call.num_max_tokens)
            num_expanded = cap if st.do_expand else 0
        rows = num_expanded if st.do_expand else num_recv
        G = (H + 127) // 128
        x_dtype = torch.float8_e4m3fn if st.fp8_out else torch.bfloat16
        recv_x = core.view(st.slot.x, [rows, H], [H, 1], x_dtype)
        recv_sf = recv_w = None
        if st.side is not None:
            # contiguous scales; strided views over the tail records
            tail_bytes, off_w, off_meta, sf_pitch = st.side      # tail_bytes: distance of two rows' records
            if st.fp8_out:
                recv_sf = core.view(st.slot.sf, [rows, G], [sf_pitch, 1], torch.float32)
            isz = st.topk_idx.element_size()
            recv_idx = core.view(st.slot.tail, [rows, K], [tail_bytes // isz, 1], st.topk_idx.dtype)
            if st.topk_weights is not None:
                recv_w = core.view(st.slot.tail + off_w, [rows, K], [tail_bytes // 4, 1], torch.float32)
            meta = core.view(st.slot.tail + off_meta, [rows, 2], [tail_bytes // 4, 1], torch.int32)
        else:
            if st.fp8_out:
                strides = [1, cap] if st.col_major_sf else [G, 1]
                recv_sf = core.view(st.slot.sf, [rows, G], strides, torch.float32)
            recv_idx = None if st.do_expand else core.view(st.slot.idx, [rows, K], [K, 1], st.topk_idx.dtype)
            if st.topk_weights is not None:
                recv_w = core.view(st.slot.w, [rows], [1], torch.float32) if st.do_expand else \
                    core.view(st.slot.w, [rows, K], [K, 1], torch.float32)
            meta = core.view(st.slot.meta, [rows, 2], [2, 1], torch.int32)
        if not self.zero_copy:
            recv_x = recv_x.clone()
            recv_sf = None if recv_sf is None else recv_sf.clone()
            recv_idx = None if recv_idx is None else recv_idx.clone()
            recv_w = None if recv_w is None else recv_w.clone()
            meta = meta.clone()
        if st.cached_handle is not None:
            handle = st.cached_handle
            handle.recv_slot = st.slot_idx
            handle.recv_src_metadata = meta
        else:
            idx_copy = st.topk_idx.clone() if st.do_handle_copy else st.topk_idx
            handle = EPHandle(st.do_expand, st.E, st.alignment, st.call.num_max_tokens, st.num_sms, idx_copy, num_recv,
                              num_expanded, per_expert_list, st.call.psum_rank, st.call.psum_expert,
                              st.call.recv_per_expert, meta, st.call.lane_src, st.call.plan, H, st.slot_idx,
                              st.topk_weights, stamp=self._stamp(st.T, K))
        x_out = (recv_x, recv_sf) if st.fp8_out else recv_x
        return x_out, recv_idx, recv_w, handle

    # ------------------------------------------------------------------------------------------ combine
    def get_combine_buffer(self, handle: EPHandle, hidden: Optional[int] = None) -> torch.Tensor:
        """bf16 ``[handle.num_rows, hidden]`` view of the input region that the NEXT ``combine`` call of this buffer
        reads.  Expert outputs written here are combined without the staging copy that a plain tensor needs.
        There are two such regions, used by alternate calls (peers may still be pulling from the previous call's
        region), so ask for the view after the previous ``combine`` has been issued."""
        assert not self.is_cpu
        H = value_or(hidden, handle.hidden)
        return self.core.view(self.regions.combine_x(self._combine_slot_counter), [handle.num_rows, H], [H, 1], torch.bfloat16)

    def combine(self, x: torch.Tensor, handle: EPHandle, topk_weights: Optional[torch.Tensor] = None,
                bias: Union[None, torch.Tensor, Tuple[torch.Tensor, torch.Tensor]] = None, num_sms: int = 0,
                num_qps: int = 0, previous_event: Optional[EventHandle] = None,
                previous_event_before_epilogue: Optional[EventHandle] = None, async_with_compute_stream: bool = False,
                allocate_on_comm_stream: bool = False, weighted: bool = False, out: Optional[torch.Tensor] = None):
        """Reduce the experts' output rows back onto the tokens' home ranks.

        ``x`` has one row per received row of the dispatch (``handle.num_rows``).  The result for token ``t`` is
        ``bias_0 + bias_1 + sum_k row(plan[t, k])`` accumulated in fp32 in top-k lane order and rounded once to
        bf16 (no weighting, as deep_ep/buffers/elastic.py:1616-1712); with ``weighted=True`` each row is first
        multiplied by the token's own ``topk_weights[t, k]`` (fused weighted reduce).  ``topk_weights`` given
        here are carried back to the home rank unchanged (``[rows, K]`` non-expand, ``[rows]`` expand) and
        returned as ``combined_topk_weights [T, K]``.  A plain ``x`` is first copied into the buffer's input region
        (one local pass over the rows); a tensor obtained from :meth:`get_combine_buffer` is read in place.
        Stream arguments behave as in :meth:`dispatch` (the kernel runs on ``self.combine_stream``).  ``out`` (contiguous
        bf16 ``[T, H]``) receives the result in place of a new tensor.
        Returns ``(combined_x, combined_topk_weights, event)``.
        """
        assert not self._destroyed
        if num_qps != 0:
            raise ValueError('num_qps must be 0: there are no RDMA queue pairs inside one NVLink domain')
        if previous_event is not None and not allocate_on_comm_stream:
            raise ValueError('`previous_event` requires `allocate_on_comm_stream=True`')
        self._attest(handle, 'combine')
        bias0, bias1 = (bias if isinstance(bias, (tuple, list)) else (bias, None)) if bias is not None else (None, None)
        if self.is_cpu:
            return self._cpu.combine(self, x, handle, topk_weights, bias0, bias1, weighted)
        num_sms = value_or(num_sms or None, handle.num_sms)
        stream = self.combine_stream
        alloc_stream = stream if allocate_on_comm_stream else torch.cuda.current_stream()
        if allocate_on_comm_stream:
            self._stream_prologue(previous_event, previous_event_before_epilogue, stream)
        with torch.cuda.stream(alloc_stream):
            call, out, out_w, staged = self._prepare_combine(x, handle, topk_weights, bias0, bias1, weighted, out)
        if not allocate_on_comm_stream:
            self._stream_prologue(previous_event, previous_event_before_epilogue, stream)
        with torch.cuda.stream(stream):
            for dst, src in staged:      # plain tensors go through the symmetric buffer
                dst.copy_(src)
            self._timed('combine', lambda: self.core.combine(call, num_sms), stream)
        inputs = (x, topk_weights, bias0, bias1, call.bias0, call.bias1, call.mul_weights, handle.plan,
                  handle.dst_buffer_slot_idx)
        event = self._stream_epilogue(async_with_compute_stream, (out, out_w), inputs, stream)
        return out, out_w, event

    def _prepare_combine(self, x, handle: EPHandle, topk_weights, bias0, bias1, weighted, out=None):
        C = self._C
        H = x.shape[1]
        rows = handle.num_rows
        assert x.dtype == torch.bfloat16 and x.shape[0] >= rows, 'combine input must be bf16 with one row per received row'
        region = self._combine_slot_counter & 1
        self._combine_slot_counter += 1
        off_x, off_w = self.regions.combine_x(region), self.regions.combine_w(region)
        staging = self.core.view(off_x, [rows, H], [H, 1], torch.bfloat16)
        staged = []
        if x.data_ptr() != staging.data_ptr():
            staged.append((staging, x[:rows]))
        call = C.CombineCall()
        call.off_x = off_x
        call.plan = handle.plan
        call.lane_src = handle.dst_buffer_slot_idx
        call.hidden = H
        if self.profile is not None:
            call.prof = self.profile['combine']
        T, K = handle.plan.shape
        if out is None:
            out = torch.empty((T, H), dtype=torch.bfloat16, device=x.device)
        assert out.shape == (T, H) and out.dtype == torch.bfloat16 and out.is_contiguous(), '`out` must be contiguous bf16 [T, H]'
        call.out = out
        out_w = None
        if topk_weights is not None:
            w_cols = 1 if handle.do_expand else K
            wview = self.core.view(off_w, [rows, w_cols], [w_cols, 1], torch.float32)
            staged.append((wview, topk_weights[:rows].reshape(rows, w_cols)))
            out_w = torch.empty((T, K), dtype=torch.float32, device=x.device)
            call.off_w, call.w_cols, call.out_w = off_w, w_cols, out_w
        if weighted:
            assert handle.do_expand, 'the fused weighted reduce needs the expand layout (one row per expert hit)'
            assert handle.topk_weights is not None, 'dispatch must have been given topk_weights'
            call.mul_weights = handle.topk_weights.contiguous()
        if bias0 is not None:
            call.bias0 = bias0.contiguous()
        if bias1 is not None:
            call.bias1 = bias1.contiguous()
        return call, out, out_w, staged

    # ------------------------------------------------------------------------------------------ streams
    def _stream_prologue(self, previous_event: Optional[EventHandle], before_epilogue: Optional[EventHandle], stream=None) -> None:
        """The communication stream waits for ``previous_event`` or for the current stream's work so far, and for
        ``before_epilogue`` (see :meth:`dispatch`)."""
        stream = self.comm_stream if stream is None else stream
        if previous_event is not None and previous_event.event is not None:
            stream.wait_event(previous_event.event)
        else:
            stream.wait_stream(torch.cuda.current_stream())
        if before_epilogue is not None and before_epilogue.event is not None:
            stream.wait_event(before_epilogue.event)

    def _stream_epilogue(self, async_with_compute_stream: bool, outputs, inputs=(), stream=None) -> EventOverlap:
        """Either hand back an event on the communication stream (async) or make the current stream wait.

        In the async case the caching allocator must not hand a block to someone else while the other stream still
        uses it: every tensor involved (inputs read by the kernel, handle tensors, outputs; the handle is walked
        too) is recorded on both streams, or, with ``EP_AVOID_RECORD_STREAM=1``, kept alive by the returned event
        instead (csrc/elastic/buffer.hpp:558-586, 1151-1164 of the reference)."""
        flat: List[torch.Tensor] = []

        def walk(o):
            if isinstance(o, torch.Tensor):
                flat.append(o)
            elif isinstance(o, (tuple, list)):
                for i in o:
                    walk(i)
            elif isinstance(o, EPHandle):
                for v in vars(o).values():
                    if isinstance(v, torch.Tensor):
                        flat.append(v)
        walk(outputs)
        walk(inputs)
        stream = self.comm_stream if stream is None else stream
        if async_with_compute_stream:
            if os.environ.get('EP_AVOID_RECORD_STREAM', '0') != '1':
                cur = torch.cuda.current_stream()
                for t in flat:
                    if t.is_cuda:
                        t.record_stream(cur)
                        t.record_stream(stream)
            return EventOverlap(EventHandle(stream, tuple(flat)))
        torch.cuda.current_stream().wait_stream(stream)
        return EventOverlap(None)

    def capture(self) -> EventHandle:
        """An event on the current stream, usable as ``previous_event``."""
        return EventHandle(torch.cuda.current_stream() if not self.is_cpu else None)

    # ------------------------------------------------------------------------------------------ kernel timing
    def enable_kernel_timing(self, enabled: bool = True) -> None:
        """Bracket every dispatch / combine kernel with CUDA events recorded on the communication stream right
        around the launch (what a per-kernel profiler reports), without the cross-stream hand-over on either side.
        Read the pairs with :meth:`kernel_times_ms`."""
        self._kernel_timing = {'dispatch': [], 'combine': []} if enabled else None

    def _timed(self, name: str, launch, stream=None) -> None:
        if self._kernel_timing is None:
            launch()
            return
        stream = self.comm_stream if stream is None else stream
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        launch()
        e1.record(stream)
        self._kernel_timing[name].append((e0, e1))

    def kernel_times_ms(self, name: str, clear: bool = True) -> List[float]:
        """Device time of every ``name`` ('dispatch' or 'combine') kernel launched since timing was enabled (or since
        the last call with ``clear``).  Synchronises the device."""
        torch.cuda.synchronize()
        out = [a.elapsed_time(b) for a, b in self._kernel_timing[name]]
        if clear:
            self._kernel_timing[name] = []
        return out

    # ------------------------------------------------------------------------------------------ profiling
    def enable_profiling(self, enabled: bool = True) -> None:
        """Make dispatch / combine record device-side phase timestamps (ns; CTA 0 of this rank, and the last CTA to
        finish for the closing phases); read them with :meth:`phase_times`."""
        keys = ('dispatch', 'combine', 'll_dispatch', 'll_combine')
        self.profile = {k: torch.zeros(8, dtype=torch.int64, device='cuda') for k in keys} if enabled else None

    def phase_times(self) -> dict:
        """Microseconds spent in each phase of the last dispatch and combine."""
        torch.cuda.synchronize()
        d, c = self.profile['dispatch'].tolist(), self.profile['combine'].tolist()
        names_d = ['layout_count', 'count_exchange', 'assign_rows', 'scatter', 'last_cta_drained', 'peers_done', 'close']
        names_c = ['entry_barrier', 'pull_reduce', 'last_cta_done']
        out = {'dispatch': {n: (d[i + 1] - d[i]) / 1e3 for i, n in enumerate(names_d) if d[i + 1] and d[i]},
               'combine': {n: (c[i + 1] - c[i]) / 1e3 for i, n in enumerate(names_c) if c[i + 1] and c[i]}}
        # low-latency kernels: microseconds since the start of the kernel at which each point was reached (CTA 0, except
        # "published", which the last CTA to finish its sends records)
        names = {'ll_dispatch': ['sends_issued', 'sends_complete', 'counts_published', 'counts_received', 'packed', 'end'],
                 'll_combine': ['stores_issued', 'stores_complete', 'flags_published', 'flags_received', 'reduced', 'end']}
        for key, ns in names.items():
            v = self.profile[key].tolist()
            out[key] = {n: (v[i + 1] - v[0]) / 1e3 for i, n in enumerate(ns) if v[i + 1] and v[0]}
        return out

    # ------------------------------------------------------------------------------------------ failures
    def check_status(self) -> None:
        """Raise (and poison the buffer) if a device wait reported a failure."""
        if not self.is_cpu:
            self.core.check_status()

    @property
    def state(self) -> str:
        return 'idle' if self.is_cpu else self.core.state()
