"""``Buffer`` / ``Config``: the first-generation API of the reference (deep_ep/buffers/legacy.py:14-713,
csrc/legacy/config.hpp:24-188) on top of the same runtime and kernels as ``ElasticBuffer``.

``get_dispatch_layout`` -> ``dispatch`` -> ``combine`` (tuple handles, explicit layout call, ``num_worst_tokens``
for the host-sync-free path) and the low-latency calls keep their signatures and return shapes.  There is no
RDMA path: one NVSwitch box is one NVLink domain, so the "internode" arguments are accepted and ignored.
"""
from typing import Optional, Tuple, Union

import torch
import torch.distributed as dist

from ..utils.event import EventHandle, EventOverlap
from .elastic import ElasticBuffer, EPHandle


class Config:
    """Per-call tuning knobs of the legacy API.  Only ``num_sms`` matters here; the chunk sizes described queue
    depths of the reference's ring buffers, which this implementation does not have."""

    def __init__(self, num_sms: int = 20, num_max_nvl_chunked_send_tokens: int = 6, num_max_nvl_chunked_recv_tokens: int = 256,
                 num_max_rdma_chunked_send_tokens: int = 6, num_max_rdma_chunked_recv_tokens: int = 256):
        self.num_sms = num_sms
        self.num_max_nvl_chunked_send_tokens = num_max_nvl_chunked_send_tokens
        self.num_max_nvl_chunked_recv_tokens = num_max_nvl_chunked_recv_tokens
        self.num_max_rdma_chunked_send_tokens = num_max_rdma_chunked_send_tokens
        self.num_max_rdma_chunked_recv_tokens = num_max_rdma_chunked_recv_tokens

    def get_nvl_buffer_size_hint(self, hidden_bytes: int, num_ranks: int, num_max_tokens_per_rank: int = 4096, num_topk: int = 8) -> int:
        """Bytes of symmetric memory for bf16 rows of ``hidden_bytes`` on ``num_ranks`` ranks."""
        return ElasticBuffer.get_buffer_size_hint(None, num_max_tokens_per_rank, hidden_bytes // 2, num_topk, num_ranks=num_ranks)

    def get_rdma_buffer_size_hint(self, hidden_bytes: int, num_ranks: int) -> int:
        return 0


def get_low_latency_rdma_size_hint(num_max_dispatch_tokens_per_rank: int, hidden: int, num_ranks: int, num_experts: int,
                                   num_topk: int = 8) -> int:
    return ElasticBuffer.get_low_latency_size_hint(num_max_dispatch_tokens_per_rank, hidden, num_ranks, num_experts, num_topk)


class Buffer:
    num_sms: int = 20

    def __init__(self, group: Optional[dist.ProcessGroup], num_nvl_bytes: int = 0, num_rdma_bytes: int = 0,
                 low_latency_mode: bool = False, num_qps_per_rank: int = 24, allow_nvlink_for_low_latency_mode: bool = True,
                 allow_mnnvl: bool = False, explicitly_destroy: bool = False, enable_shrink: bool = False,
                 num_max_tokens_per_rank: int = 0, hidden: int = 0, num_topk: int = 8, use_fp8_dispatch: bool = False):
        self.group = group
        self.rank = dist.get_rank(group) if group is not None else 0
        self.group_size = dist.get_world_size(group) if group is not None else 1
        self.num_nvl_bytes, self.num_rdma_bytes = num_nvl_bytes, num_rdma_bytes
        self.low_latency_mode = low_latency_mode
        self.explicitly_destroy = explicitly_destroy
        self.enable_shrink = enable_shrink
        self._shape = (num_max_tokens_per_rank, hidden, num_topk, use_fp8_dispatch)
        self._elastic: Optional[ElasticBuffer] = None
        if num_max_tokens_per_rank and hidden:
            self._ensure(num_max_tokens_per_rank, hidden, num_topk, use_fp8_dispatch)

    # ------------------------------------------------------------------------------------------ plumbing
    def _ensure(self, tokens: int, hidden: int, num_topk: int, fp8: bool) -> ElasticBuffer:
        if self._elastic is None:
            cap = torch.tensor([tokens], dtype=torch.int64, device='cuda' if torch.cuda.is_available() else 'cpu')
            if self.group is not None and self.group_size > 1:
                dist.all_reduce(cap, op=dist.ReduceOp.MAX, group=self.group)
            cap = max(int(cap.item()), self._shape[0])
            # the low-latency regions live behind the MoE regions; `num_rdma_bytes` is what the caller sized for them
            self._elastic = ElasticBuffer(self.group, num_max_tokens_per_rank=cap, hidden=hidden, num_topk=num_topk,
                                          use_fp8_dispatch=fp8, extra_bytes=self.num_rdma_bytes,
                                          explicitly_destroy=self.explicitly_destroy, low_latency_shrink=self.enable_shrink)
        e = self._elastic
        assert tokens <= e.num_max_tokens_per_rank and hidden <= e.hidden, \
            'this Buffer was created for smaller tensors; construct it with num_max_tokens_per_rank / hidden'
        return e

    def is_available(self) -> bool:
        return self._elastic is None or self._elastic.state == 'idle'

    def get_num_rdma_ranks(self) -> int:
        return 1

    def get_rdma_rank(self) -> int:
        return 0

    def get_root_rdma_rank(self, is_global: bool = True) -> int:
        return 0

    def get_local_device_id(self) -> int:
        return torch.cuda.current_device()

    def get_local_nvshmem_unique_id(self) -> bytes:
        """There is no NVSHMEM in this build (one NVLink domain, peers mapped directly): an empty id."""
        return b''

    def get_comm_stream(self):
        return self._elastic.get_comm_stream() if self._elastic is not None else torch.cuda.current_stream()

    def get_local_ipc_handle(self) -> bytes:
        """What a peer process needs to map this rank's buffer (a cudaIpc handle, or the descriptor socket of a VMM
        allocation).  The exchange itself happens when the buffer is built; this is for inspection and external set-ups
        (deep_ep/buffers/legacy.py:74-131 of the reference)."""
        assert self._elastic is not None and not self._elastic.is_cpu, 'the buffer is built on first use (or pass its shape to the constructor)'
        return bytes(self._elastic.core.get_local_ipc_handle())

    def get_local_buffer_tensor(self, dtype: torch.dtype = torch.uint8, offset: int = 0) -> torch.Tensor:
        """The data area of this rank's symmetric buffer (everything behind the workspace) as a flat tensor of ``dtype``,
        starting ``offset`` bytes in."""
        e = self._elastic
        assert e is not None and not e.is_cpu
        start = e._C.get_workspace_bytes() + offset
        n = (e.num_bytes - start) // dtype.itemsize
        return e.core.view(start, [n], [1], dtype)

    def sync(self, *args, **kwargs) -> None:
        """Peers are mapped when the buffer is built (a collective step of the constructor), so there is nothing left to
        synchronise; kept so that code written for the two-step set-up of the reference keeps working."""
        return None

    def destroy(self) -> None:
        if self._elastic is not None:
            self._elastic.destroy()
            self._elastic = None

    @staticmethod
    def set_num_sms(new_num_sms: int) -> None:
        assert new_num_sms % 2 == 0
        Buffer.num_sms = new_num_sms

    @staticmethod
    def capture() -> EventOverlap:
        return EventOverlap(EventHandle(torch.cuda.current_stream()))

    @staticmethod
    def get_low_latency_rdma_size_hint(num_max_dispatch_tokens_per_rank: int, hidden: int, num_ranks: int, num_experts: int) -> int:
        return get_low_latency_rdma_size_hint(num_max_dispatch_tokens_per_rank, hidden, num_ranks, num_experts)

    @staticmethod
    def get_dispatch_config(num_ranks: int) -> Config:
        return Config(Buffer.num_sms)

    @staticmethod
    def get_combine_config(num_ranks: int) -> Config:
        return Config(Buffer.num_sms)

    # ------------------------------------------------------------------------------------------ normal mode
    def get_dispatch_layout(self, topk_idx: torch.Tensor, num_experts: int, previous_event: Optional[EventOverlap] = None,
                            async_finish: bool = False, allocate_on_comm_stream: bool = False):
        """-> ``(num_tokens_per_rank [R] int32, None, num_tokens_per_expert [E] int32, is_token_in_rank [T, R] bool,
        event)``.  One sm_100a kernel; dispatch recomputes the same counts inside its own kernel, so calling this is
        optional."""
        if topk_idx.is_cuda:
            from .. import _native
            per_rank, per_expert, in_rank = _native.load().get_dispatch_layout(topk_idx.contiguous(), num_experts, self.group_size)
        else:
            from ..ops.layout_ref import get_dispatch_layout_ref
            per_rank, per_expert, in_rank = get_dispatch_layout_ref(topk_idx, num_experts, self.group_size)
        return per_rank, None, per_expert, in_rank, EventOverlap(EventHandle() if async_finish else None)

    def dispatch(self, x: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]], handle: Optional[tuple] = None,
                 num_tokens_per_rank: Optional[torch.Tensor] = None, num_tokens_per_rdma_rank: Optional[torch.Tensor] = None,
                 is_token_in_rank: Optional[torch.Tensor] = None, num_tokens_per_expert: Optional[torch.Tensor] = None,
                 topk_idx: Optional[torch.Tensor] = None, topk_weights: Optional[torch.Tensor] = None, expert_alignment: int = 1,
                 num_worst_tokens: int = 0, config: Optional[Config] = None, previous_event: Optional[EventOverlap] = None,
                 async_finish: bool = False, allocate_on_comm_stream: bool = False):
        """-> ``(recv_x, recv_topk_idx, recv_topk_weights, num_recv_tokens_per_expert_list, handle, event)``.
        ``num_worst_tokens > 0`` skips the host synchronisation (outputs get the worst-case size and the list is
        empty), which makes the call CUDA-graph friendly."""
        x0 = x[0] if isinstance(x, tuple) else x
        num_sms = (config or Config(Buffer.num_sms)).num_sms
        prev = previous_event.event if previous_event is not None else None
        if handle is not None:
            ep_handle: EPHandle = handle[-1]
            e = self._ensure(x0.shape[0], x0.shape[1], ep_handle.num_topk, x0.dtype == torch.float8_e4m3fn)
            recv_x, recv_idx, recv_w, ep_handle, event = e.dispatch(x, handle=ep_handle, topk_weights=topk_weights, num_sms=num_sms,
                                                                    previous_event=prev, async_with_compute_stream=async_finish)
            return recv_x, recv_idx, recv_w, None, handle, event
        assert topk_idx is not None and num_tokens_per_expert is not None
        num_experts = num_tokens_per_expert.numel()
        e = self._ensure(x0.shape[0], x0.shape[1], topk_idx.shape[1], x0.dtype == torch.float8_e4m3fn)
        recv_x, recv_idx, recv_w, ep_handle, event = e.dispatch(
            x, topk_idx, topk_weights, num_experts=num_experts, expert_alignment=expert_alignment, num_sms=num_sms,
            do_cpu_sync=(num_worst_tokens == 0), previous_event=prev, async_with_compute_stream=async_finish)
        per_expert = ep_handle.num_recv_tokens_per_expert_list if num_worst_tokens == 0 else []
        legacy_handle = (ep_handle.dst_buffer_slot_idx, ep_handle.plan, ep_handle.psum_num_recv_tokens_per_scaleup_rank,
                         ep_handle.psum_num_recv_tokens_per_expert, ep_handle.recv_src_metadata, ep_handle)
        return recv_x, recv_idx, recv_w, per_expert, legacy_handle, event

    def combine(self, x: torch.Tensor, handle: tuple, topk_weights: Optional[torch.Tensor] = None,
                bias: Union[None, torch.Tensor, Tuple[torch.Tensor, torch.Tensor]] = None, config: Optional[Config] = None,
                previous_event: Optional[EventOverlap] = None, async_finish: bool = False, allocate_on_comm_stream: bool = False):
        """Sum (no weighting) of the rows of every token back on its home rank -> ``(combined_x,
        combined_topk_weights, event)``."""
        ep_handle: EPHandle = handle[-1]
        num_sms = (config or Config(Buffer.num_sms)).num_sms
        prev = previous_event.event if previous_event is not None else None
        return self._elastic.combine(x, ep_handle, topk_weights=topk_weights, bias=bias, num_sms=num_sms, previous_event=prev,
                                     async_with_compute_stream=async_finish)

    # ------------------------------------------------------------------------------------------ low-latency mode
    # The reference's native Buffer has one entry point per transport (csrc/legacy/buffer.hpp intranode_* / internode_*); inside
    # one NVLink domain they are the same kernels, so the four names lead to the two methods above.
    def intranode_dispatch(self, *args, **kwargs):
        return self.dispatch(*args, **kwargs)

    def intranode_combine(self, *args, **kwargs):
        return self.combine(*args, **kwargs)

    def internode_dispatch(self, *args, **kwargs):
        return self.dispatch(*args, **kwargs)

    def internode_combine(self, *args, **kwargs):
        return self.combine(*args, **kwargs)

    def _ll_buffer(self, tokens: int, hidden: int, num_topk: int) -> ElasticBuffer:
        if self._elastic is None:
            self._elastic = ElasticBuffer(self.group, num_max_tokens_per_rank=max(tokens, self._shape[0]), hidden=hidden,
                                          num_topk=num_topk, extra_bytes=self.num_rdma_bytes,
                                          explicitly_destroy=self.explicitly_destroy, low_latency_shrink=self.enable_shrink)
        return self._elastic

    def clean_low_latency_buffer(self, num_max_dispatch_tokens_per_rank: int, hidden: int, num_experts: int) -> None:
        if self._elastic is not None:
            self._elastic.clean_low_latency_buffer(num_max_dispatch_tokens_per_rank, hidden, num_experts)

    def low_latency_dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, num_max_dispatch_tokens_per_rank: int, num_experts: int,
                             cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                             dispatch_wait_recv_cost_stats: Optional[torch.Tensor] = None, use_fp8: bool = True,
                             round_scale: bool = False, use_ue8m0: bool = False, async_finish: bool = False,
                             return_recv_hook: bool = False):
        e = self._ll_buffer(num_max_dispatch_tokens_per_rank, x.shape[1], topk_idx.shape[1])
        return e.low_latency_dispatch(x, topk_idx, num_max_dispatch_tokens_per_rank, num_experts, cumulative_local_expert_recv_stats,
                                      dispatch_wait_recv_cost_stats, use_fp8, round_scale, use_ue8m0, async_finish, return_recv_hook)

    def low_latency_combine(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, handle: tuple,
                            use_logfmt: bool = False, zero_copy: bool = False, async_finish: bool = False,
                            return_recv_hook: bool = False, out: Optional[torch.Tensor] = None,
                            combine_wait_recv_cost_stats: Optional[torch.Tensor] = None):
        return self._elastic.low_latency_combine(x, topk_idx, topk_weights, handle, use_logfmt, zero_copy, async_finish,
                                                 return_recv_hook, out, combine_wait_recv_cost_stats)

    def low_latency_update_mask_buffer(self, rank_to_mask: int, mask: bool = False) -> None:
        self._elastic.low_latency_update_mask_buffer(rank_to_mask, mask)

    def low_latency_query_mask_buffer(self, mask_status: torch.Tensor) -> torch.Tensor:
        return self._elastic.low_latency_query_mask_buffer(mask_status)

    def low_latency_clean_mask_buffer(self) -> None:
        self._elastic.low_latency_clean_mask_buffer()

    def get_next_low_latency_combine_buffer(self, handle: tuple) -> torch.Tensor:
        return self._elastic.get_next_low_latency_combine_buffer(handle)
