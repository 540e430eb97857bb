"""The non-MoE collectives of ``ElasticBuffer``: all-gather / reduce-scatter sessions on the copy engines,
pipeline-parallel send / recv, context-parallel KV gather and Engram remote fetch.

* AG / RS sessions (parity: csrc/elastic/buffer.hpp:379-526, deep_ep/buffers/elastic.py:1154-1251; reduce-scatter
  has no counterpart in the reference, whose README lists it as on-going): data moves with peer
  ``cudaMemcpyAsync`` on the copy engines, one per peer; completion is a 32-thread signal kernel over NVLink (bounded
  wait), or, with ``use_stream_memops``, stream memory operations, so no SM is busy while the bytes move.
* PP (parity: csrc/elastic/buffer.hpp:329-377): ring-neighbour send / recv on NCCL point-to-point, on a side
  stream so that it overlaps with compute.
* Engram (parity: csrc/elastic/buffer.hpp:212-327): every rank publishes a table of fixed-size entries in its
  symmetric buffer; ``engram_fetch`` pulls arbitrary entries from their owners with TMA loads over NVLink.
"""
import math
from typing import Callable, List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist

from ..utils.math import align


class CollectivesMixin:
    """Mixed into ``ElasticBuffer``; uses ``self.core``, ``self.reserve``, ``self.comm_stream``."""

    _agrs = None
    _pp = None
    _engram = None

    # ------------------------------------------------------------------------------------------ AG / RS sessions
    def agrs_set_config(self, num_max_session_bytes: int, num_max_agrs_per_session: int = 32,
                        use_stream_memops: bool = False) -> None:
        """Reserve the gather region: ``num_max_session_bytes`` is the sum over the tensors of one session of
        ``align(num_ranks * tensor_bytes, 32)``.

        ``use_stream_memops``: signal completion with stream memory operations (a 64-bit write into every peer's buffer
        and a wait on the local words, queued on the stream by the driver) instead of the 32-thread signal kernel, so
        that a whole all-gather uses no SM at all, as the reference does (csrc/kernels/backend/cuda_driver.cu:12-52).
        Unlike the kernel, such a wait has no time limit: a peer that never arrives stalls the stream.  Off by default."""
        if self.is_cpu:
            return self._cpu_coll.agrs_set_config(num_max_session_bytes, num_max_agrs_per_session, use_stream_memops)
        assert num_max_agrs_per_session <= 32
        assert self._agrs is None or not self._agrs['open'], 'destroy the open session first'
        self._agrs = {'offset': self.reserve(align(num_max_session_bytes, 1024)), 'bytes': num_max_session_bytes,
                      'cursor': 0, 'open': False, 'count': 0, 'max': num_max_agrs_per_session, 'inplace': {},
                      'memops': bool(use_stream_memops) and self._virtual is None}

    def _agrs_signal(self) -> None:
        """All ranks' copies queued so far have landed everywhere (on the current stream)."""
        if self._agrs.get('memops') and self.core.signal_and_wait_memops(self._C.CH_AGRS):
            return
        self.core.barrier(self._C.CH_AGRS)

    def create_agrs_session(self) -> None:
        if self.is_cpu:
            return self._cpu_coll.create_agrs_session()
        assert self._agrs is not None, 'call agrs_set_config first'
        assert not self._agrs['open'], 'one session at a time'
        self._agrs.update(open=True, cursor=0, count=0, inplace={})

    def destroy_agrs_session(self) -> None:
        """All ranks must be done reading the gathered tensors before the region is recycled."""
        if self.is_cpu:
            return self._cpu_coll.destroy_agrs_session()
        assert self._agrs is not None and self._agrs['open']
        self.comm_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.comm_stream):
            self._agrs_signal()
        torch.cuda.current_stream().wait_stream(self.comm_stream)
        self._agrs['open'] = False

    def _agrs_alloc(self, shape: Sequence[int], dtype: torch.dtype) -> Tuple[int, int]:
        a = self._agrs
        assert a is not None and a['open'], 'no open AG/RS session'
        assert a['count'] < a['max'], 'too many collectives in this session'
        nbytes = math.prod(shape) * dtype.itemsize
        total = align(self.num_ranks * nbytes, 32)
        assert a['cursor'] + total <= a['bytes'], 'session region exhausted: raise num_max_session_bytes'
        off = a['offset'] + a['cursor']
        a['cursor'] += total
        a['count'] += 1
        return off, nbytes

    def agrs_get_inplace_tensor(self, shape: Sequence[int], dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """This rank's slice inside the next gather slot: a producer that writes its result here saves the
        local copy of ``all_gather``."""
        if self.is_cpu:
            return self._cpu_coll.agrs_get_inplace_tensor(shape, dtype)
        off, nbytes = self._agrs_alloc(shape, dtype)
        t = self.core.view(off + self.rank_idx * nbytes, list(shape), list(_contiguous_strides(shape)), dtype)
        self._agrs['inplace'][t.data_ptr()] = (off, nbytes)
        return t

    def all_gather(self, tensors: Union[torch.Tensor, Sequence[torch.Tensor]]) -> Tuple[Union[torch.Tensor, List[torch.Tensor]], Callable]:
        """Gather ``t`` (or each tensor of a list) from all ranks -> ``([num_ranks, *shape] view(s), wait)``.
        ``wait()`` makes the current stream wait for the gathered data."""
        if self.is_cpu:
            return self._cpu_coll.all_gather(tensors)
        single = isinstance(tensors, torch.Tensor)
        ts = [tensors] if single else list(tensors)
        self.comm_stream.wait_stream(torch.cuda.current_stream())
        outs = []
        with torch.cuda.stream(self.comm_stream):
            for t in ts:
                t = t.contiguous()
                if t.data_ptr() in self._agrs['inplace']:
                    off, nbytes = self._agrs['inplace'].pop(t.data_ptr())
                    skip_local = True
                else:
                    off, nbytes = self._agrs_alloc(t.shape, t.dtype)
                    skip_local = False
                for step in range(self.num_ranks):
                    peer = (self.rank_idx + step) % self.num_ranks     # stagger the destinations
                    if peer == self.rank_idx and skip_local:
                        continue
                    self.core.peer_copy(peer, off + self.rank_idx * nbytes, t)
                shape = [self.num_ranks] + list(t.shape)
                outs.append(self.core.view(off, shape, list(_contiguous_strides(shape)), t.dtype))
            self._agrs_signal()
        event = torch.cuda.Event()
        event.record(self.comm_stream)

        def wait() -> None:
            torch.cuda.current_stream().wait_event(event)
        return (outs[0] if single else outs), wait

    def reduce_scatter(self, tensor: torch.Tensor) -> Tuple[torch.Tensor, Callable]:
        """``tensor [num_ranks, *shape]`` (bf16 or fp32): rank ``r`` receives ``sum over ranks of tensor[r]``
        accumulated in fp32 in rank order.  Slices travel on the copy engines; the sum is one local kernel.
        -> ``(out [*shape], wait)``."""
        if self.is_cpu:
            return self._cpu_coll.reduce_scatter(tensor)
        assert tensor.shape[0] == self.num_ranks and tensor.dtype in (torch.bfloat16, torch.float32)
        tensor = tensor.contiguous()
        shape = list(tensor.shape[1:])
        self.comm_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.comm_stream):
            off, nbytes = self._agrs_alloc(shape, tensor.dtype)
            for step in range(self.num_ranks):
                peer = (self.rank_idx + step) % self.num_ranks
                self.core.peer_copy(peer, off + self.rank_idx * nbytes, tensor[peer])
            self._agrs_signal()
            slots_shape = [self.num_ranks] + shape
            slots = self.core.view(off, slots_shape, list(_contiguous_strides(slots_shape)), tensor.dtype)
            out = torch.empty(shape, dtype=tensor.dtype, device=tensor.device)
            self._C.reduce_slots(slots, out)
        event = torch.cuda.Event()
        event.record(self.comm_stream)

        def wait() -> None:
            torch.cuda.current_stream().wait_event(event)
        return out, wait

    def cp_all_gather_kv(self, k: torch.Tensor, v: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, Callable]:
        """Context parallelism helper: gather the K and V shards of every rank with zero SMs (inside an open
        AG/RS session).  -> ``(k_all [ranks, ...], v_all [ranks, ...], wait)``."""
        (k_all, v_all), wait = self.all_gather([k, v])
        return k_all, v_all, wait

    # ------------------------------------------------------------------------------------------ pipeline parallel
    def pp_set_config(self, num_max_tensor_bytes: int, num_max_inflight_tensors: int) -> None:
        """Ring neighbours and the side stream for pipeline send / recv."""
        if self.is_cpu:
            return self._cpu_coll.pp_set_config(num_max_tensor_bytes, num_max_inflight_tensors)
        self._pp = {'prev': (self.rank_idx - 1) % self.num_ranks, 'next': (self.rank_idx + 1) % self.num_ranks,
                    'max_bytes': num_max_tensor_bytes, 'inflight': num_max_inflight_tensors,
                    'stream': torch.cuda.Stream(), 'pending': []}

    def _pp_check(self, t: torch.Tensor, peer: int) -> None:
        assert self._pp is not None, 'call pp_set_config first'
        assert peer in (self._pp['prev'], self._pp['next']), 'pipeline peers are the ring neighbours'
        assert t.numel() * t.element_size() <= self._pp['max_bytes'], 'tensor exceeds num_max_tensor_bytes'
        if len(self._pp['pending']) >= 2 * self._pp['inflight']:
            self._pp['pending'].pop(0).wait()

    def pp_send(self, t: torch.Tensor, dst_rank_idx: int) -> None:
        """Send ``t`` to a ring neighbour; ordered after the current stream's work, executed on the side stream."""
        if self.is_cpu:
            return self._cpu_coll.pp_send(t, dst_rank_idx)
        self._pp_check(t, dst_rank_idx)
        s = self._pp['stream']
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            t.record_stream(s)
            self._pp['pending'].append(dist.isend(t.contiguous(), dist.get_global_rank(self.group, dst_rank_idx), group=self.group))

    def pp_recv(self, t: torch.Tensor, src_rank_idx: int) -> None:
        """Receive into ``t`` from a ring neighbour; the current stream waits for the data."""
        if self.is_cpu:
            return self._cpu_coll.pp_recv(t, src_rank_idx)
        self._pp_check(t, src_rank_idx)
        s = self._pp['stream']
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            work = dist.irecv(t, dist.get_global_rank(self.group, src_rank_idx), group=self.group)
            work.wait()
        torch.cuda.current_stream().wait_stream(s)

    # ------------------------------------------------------------------------------------------ Engram
    def _engram_place(self, N: int, H: int, dtype: torch.dtype) -> dict:
        """Where this buffer keeps its Engram table: the CPU segment (``num_cpu_bytes`` at construction) when there is
        one and the table fits it, else a region of the symmetric device buffer.  Every rank decides alike."""
        entry = H * dtype.itemsize
        assert entry % 16 == 0, 'an entry must be a multiple of 16 bytes'
        if self._engram is None:
            in_cpu = 0 < N * entry <= self.num_cpu_bytes
            off = 0 if in_cpu else self.reserve(align(N * entry, 1024))
            self._engram = {'offset': off, 'N': N, 'H': H, 'dtype': dtype, 'entry': entry, 'cpu': in_cpu, 'sf': None}
        e = self._engram
        assert (N, H, dtype) == (e['N'], e['H'], e['dtype']), 'the Engram table shape is fixed per buffer'
        return e

    def _engram_store(self, e: dict, storage: torch.Tensor) -> None:
        if e['cpu']:
            self.core.cpu_segment_write(e['offset'], storage)
        else:
            self.core.view(e['offset'], [e['N'], e['H']], [e['H'], 1], e['dtype']).copy_(storage)

    def engram_write(self, storage: torch.Tensor, sf: Optional[torch.Tensor] = None) -> None:
        """Publish this rank's table ``storage [N, H]`` (bf16, or e4m3 with ``sf``).  ``sf [num_ranks * N, packs]`` is
        the scale table of ALL ranks' entries (4-byte packs: fp32, or four UE8M0 bytes), replicated on every rank; it
        stays local and is gathered with every fetch (csrc/elastic/buffer.hpp:212-242 of the reference).  The table
        goes to the CPU segment when the buffer has one that is large enough, else into the device buffer."""
        if self.is_cpu:
            return self._cpu_coll.engram_write(storage, sf)
        storage = storage.contiguous()
        N, H = storage.shape
        e = self._engram_place(N, H, storage.dtype)
        if sf is not None:
            assert sf.dim() == 2 and sf.is_contiguous() and sf.element_size() == 4 and sf.shape[0] == N * self.num_ranks, \
                '`sf` must be a contiguous [num_ranks * N, packs] table of 4-byte packs'
        e['sf'] = sf
        self.comm_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.comm_stream):
            self.core.barrier(self._C.CH_ENGRAM)       # nobody is still fetching the old table
            self._engram_store(e, storage)
            self.core.barrier(self._C.CH_ENGRAM)       # every table is in place
        torch.cuda.current_stream().wait_stream(self.comm_stream)

    def _engram_fetch_outputs(self, idx: torch.Tensor, col_major_sf: bool):
        e = self._engram
        T, n = idx.shape
        out = torch.empty((T, n * e['H']), dtype=e['dtype'], device=idx.device)
        fetched_sf = None
        if e['sf'] is not None:
            packs = e['sf'].shape[1]
            if col_major_sf:     # strides (1, align(T, 4)): the layout a TMA-fed GEMM wants for its scale operand
                fetched_sf = torch.empty_strided((T, n * packs), (1, align(T, 4)), dtype=e['sf'].dtype, device=idx.device)
            else:
                fetched_sf = torch.empty((T, n * packs), dtype=e['sf'].dtype, device=idx.device)
        return out, fetched_sf

    def engram_fetch(self, indices: torch.Tensor, num_qps: int = 0, use_tma_aligned_col_major_sf: bool = False, num_sms: int = 16):
        """``indices int32 [T, n]`` of global entry ids (owner = id // N) -> hook; ``hook()`` waits and returns
        ``(fetched [T, n * H], fetched_sf [T, n * packs] | None)``; the scales are column-major with
        ``use_tma_aligned_col_major_sf`` (csrc/elastic/buffer.hpp:244-327).  ``num_qps`` must be 0."""
        if num_qps != 0:
            raise ValueError('num_qps must be 0: there are no RDMA queue pairs inside one NVLink domain')
        if self.is_cpu:
            return self._cpu_coll.engram_fetch(indices, use_tma_aligned_col_major_sf)
        e = self._engram
        assert e is not None, 'call engram_write first'
        idx = indices.contiguous().to(torch.int32)
        n = idx.shape[1]
        self.comm_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.comm_stream):
            out, fetched_sf = self._engram_fetch_outputs(idx, use_tma_aligned_col_major_sf)
            tabs = [] if fetched_sf is None else [e['sf']]
            fsfs = [] if fetched_sf is None else [fetched_sf]
            self._C.ElasticBuffer.engram_fetch_group([self.core], [idx.view(-1)], [out], e['N'], e['entry'], e['offset'],
                                                     e['cpu'], tabs, fsfs, n, num_sms)
        event = torch.cuda.Event()
        event.record(self.comm_stream)

        def hook():
            torch.cuda.current_stream().wait_event(event)
            return out, fetched_sf
        return hook


def _contiguous_strides(shape: Sequence[int]) -> Tuple[int, ...]:
    strides, acc = [], 1
    for s in reversed(list(shape)):
        strides.append(acc)
        acc *= max(1, s)
    return tuple(reversed(strides))
