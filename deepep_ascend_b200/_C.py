"""The native-module surface of the reference (``deep_ep._C`` / ``deep_ep_cpp``; names listed in its
tests/platform/api_contract.py:1-42), for code that reaches below the Python classes.

This build keeps part of that surface in C++ (``get_platform``, ``ElasticBuffer``, ``calculate_elastic_buffer_size``,
``get_low_latency_rdma_size_hint``, ``get_elastic_buffer_alignment`` and the kernels' entry points) and part in Python
(``EventHandle``, ``Config``, ``Buffer``, ``topk_idx_t``, the domain-size helpers).  Kernels are compiled ahead of time for
sm_100a, so the JIT hooks are accepted and do nothing, and there is no NCCL communicator behind the buffers: peers are reached
through mapped symmetric memory, so the communicator helpers return inert handles.  Every other attribute is forwarded to the
compiled module.
"""
import os
from typing import Optional

from . import _native
from .buffers.elastic import topk_idx_t  # noqa: F401
from .utils.envs import get_logical_domain_size, get_physical_domain_size  # noqa: F401
from .utils.event import EventHandle  # noqa: F401


def is_sm90_compiled() -> bool:
    """The reference asks this before it uses Hopper-only paths; this build holds sm_100a code only."""
    return False


def init_jit(library_root_path: Optional[str] = None, cuda_home: Optional[str] = None, *args, **kwargs) -> None:
    """Nothing to initialise: there is no run-time compiler (csrc/jit/compiler.hpp:22-267 of the reference)."""
    return None


def create_cpu_handle(num_bytes: int = 0) -> bytes:
    """Name of the POSIX shared-memory object a CPU segment of that size would use in this process (the real segment
    is created by ``ElasticBuffer(..., num_cpu_bytes=...)``)."""
    return f'/deepep_b200_cpu_{os.getpid()}_{int(num_bytes)}'.encode()


def get_local_nccl_unique_id() -> bytes:
    """No NCCL communicator is created by the buffers (bootstrap goes through the caller's process group): an empty id."""
    return b''


def create_nccl_comm(unique_id: bytes = b'', rank: int = 0, num_ranks: int = 1) -> int:
    """Returns an inert handle (0): peers are addressed through mapped symmetric memory, not through NCCL windows."""
    return 0


def destroy_nccl_comm(comm: int = 0) -> None:
    return None


def __getattr__(name):
    if name in ('Buffer', 'Config'):
        from .buffers import legacy
        return getattr(legacy, name)
    return getattr(_native.load(), name)
