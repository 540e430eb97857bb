"""Tensor-parallel GEMMs fused with their collective in ONE kernel (no counterpart in the reference, which has no
GEMM and only a copy-engine all-gather).

* ``ag_gemm``: ``all_gather(x_shard) @ w^T``.  Every rank writes its ``[M / R, K]`` shard into its slice of a gathered
  matrix in the symmetric buffer; a few "copier" CTAs of the tcgen05 GEMM kernel pull the other slices over NVLink
  (TMA bulk loads from peer memory, no multicast), tile by tile, and flag each landed 128-row tile; the tensor-core
  CTAs start on the local rows and pick up remote tiles as their flags arrive.  A remote tile crosses NVLink once.
* ``gemm_rs``: ``reduce_scatter(x @ w^T)``.  The GEMM epilogue bulk-stores every row of the partial result straight
  into the owner rank's slot for this source; after a cross-GPU barrier the same kernel sums the R slots in fp32.
"""

import torch

from ..buffers.elastic import ElasticBuffer
from ..utils.math import align


class TensorParallelGemm:
    """Holds the symmetric regions for one (M, K, N) problem size on an ``ElasticBuffer``.

    ``extra_bytes`` of the buffer must cover ``size_hint(M, K, N)``."""

    def __init__(self, buffer: ElasticBuffer, M: int, K: int, N: int, num_sms: int = 0, num_copy_ctas: int = 0):
        R = buffer.num_ranks
        assert M % (128 * R) == 0 and N % 128 == 0 and K % 64 == 0
        self.buffer, self.M, self.K, self.N, self.R = buffer, M, K, N, R
        self.num_sms = num_sms or torch.cuda.get_device_properties('cuda').multi_processor_count
        self.num_copy_ctas = num_copy_ctas      # 0 = default (see `_copiers`)
        self.off_full = buffer.reserve(align(M * K * 2, 1024))
        self.slot_set_bytes = align(M * N * 2, 1024)
        self.off_slots = buffer.reserve(2 * self.slot_set_bytes)

    @staticmethod
    def size_hint(M: int, K: int, N: int) -> int:
        return align(M * K * 2, 1024) + 2 * align(M * N * 2, 1024) + (2 << 20)

    def shard_view(self) -> torch.Tensor:
        """This rank's ``[M / R, K]`` slice of the gathered matrix: write the activation shard here."""
        rows = self.M // self.R
        return self.buffer.core.view(self.off_full + self.buffer.rank_idx * rows * self.K * 2, [rows, self.K], [self.K, 1], torch.bfloat16)

    def _copiers(self, n_local: int) -> int:
        """CTAs that pull the remote shards (the rest run the tensor cores): 4 per rank and at least 16 unless the caller says otherwise.
        Measured at M 8192, K 7168: on 4 GPUs (N_local 1792, gather and GEMM take about as long) 16 copiers 0.253 ms, 32: 0.278 ms,
        48: 0.351 ms (NCCL all-gather + cuBLAS: 0.345 ms); on 8 GPUs (N_local 896, the gather of 103 MB is twice as long as the
        GEMM) 16 copiers 0.290 ms, 32: 0.243 ms, 48: 0.290 ms (NCCL + cuBLAS: 0.281 ms).  More copiers than that pull more slowly
        (the loads of all CTAs queue in front of the same links) and take SMs from the GEMM."""
        n = self.num_copy_ctas if self.num_copy_ctas > 0 else max(16, 4 * self.R)
        return max(1, min(n, self.num_sms - 1))

    def ag_gemm(self, x_shard: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """``x_shard [M / R, K]``, ``w [N_local, K]`` -> ``all_gather(x) @ w^T`` as bf16 ``[M, N_local]``."""
        view = self.shard_view()
        if x_shard.data_ptr() != view.data_ptr():
            view.copy_(x_shard)
        return self.buffer._C.ag_gemm(self.buffer.core, self.off_full, self.M, self.K, w.contiguous(), self.num_sms, self._copiers(w.shape[0]))

    def gemm_rs(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """``x [M, K_local]``, ``w [N, K_local]`` -> ``reduce_scatter(x @ w^T)`` as bf16 ``[M / R, N]``."""
        return self.buffer._C.gemm_rs(self.buffer.core, x.contiguous(), w.contiguous(), self.off_slots, self.slot_set_bytes, self.num_sms)
