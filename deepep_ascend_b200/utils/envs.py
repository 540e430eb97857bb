"""Process-group bring-up and topology probes (parity: deep_ep/utils/envs.py:185-446)."""
import os
import random
import re
import subprocess
from typing import Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

_global_seed = 0


def init_seed(seed: int = 0) -> None:
    global _global_seed
    _global_seed = seed
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)


def get_global_seed() -> int:
    return _global_seed


def init_dist(local_rank: Optional[int] = None, num_local_ranks: Optional[int] = None,
              backend: Optional[str] = None) -> Tuple[int, int, dist.ProcessGroup]:
    """Initialise ``torch.distributed`` from the usual environment (RANK / WORLD_SIZE / MASTER_*; rendezvous
    address defaults to 127.0.0.1) with one process per GPU, and return ``(rank, world_size, group)``."""
    rank = int(os.environ.get('RANK', local_rank if local_rank is not None else 0))
    world = int(os.environ.get('WORLD_SIZE', num_local_ranks if num_local_ranks is not None else 1))
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29533')
    if backend is None:
        backend = 'nccl' if torch.cuda.is_available() else 'gloo'
    if backend == 'nccl':
        dev = int(os.environ.get('LOCAL_RANK', local_rank if local_rank is not None else rank % max(1, torch.cuda.device_count())))
        torch.cuda.set_device(dev)
    if not dist.is_initialized():
        kwargs = {}
        if backend == 'nccl':
            kwargs['device_id'] = torch.device('cuda', torch.cuda.current_device())
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kwargs)
    return dist.get_rank(), dist.get_world_size(), dist.new_group(list(range(world)))


def dist_print(*args, once_in_node: bool = False, **kwargs) -> None:
    """Print rank by rank in order (or only on rank 0 with ``once_in_node``)."""
    if not dist.is_initialized():
        print(*args, **kwargs, flush=True)
        return
    for r in range(dist.get_world_size()):
        if r == dist.get_rank() and (not once_in_node or r == 0):
            print(*args, **kwargs, flush=True)
        dist.barrier()


def get_physical_domain_size(group: Optional[dist.ProcessGroup] = None) -> Tuple[int, int]:
    """(number of RDMA domains, NVLink ranks per domain).  One NVSwitch box is one NVLink domain."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    return 1, world


def get_logical_domain_size(group: Optional[dist.ProcessGroup] = None, allow_hybrid_mode: bool = True) -> Tuple[int, int]:
    """(scale-out ranks, scale-up ranks) used by the kernels: always one flat scale-up domain."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    return 1, world


def check_nvlink_connections(group: Optional[dist.ProcessGroup] = None) -> bool:
    """True when every pair of visible GPUs reports peer access (queried, never changed)."""
    if not torch.cuda.is_available():
        return False
    n = torch.cuda.device_count()
    return all(torch.cuda.can_device_access_peer(i, j) for i in range(n) for j in range(n) if i != j)


def check_torch_deterministic() -> bool:
    """Whether PyTorch's deterministic mode is on.  The reference uses this to force its slower sorted layout
    (deep_ep/utils/envs.py:361-367); here the row layout is a pure function of the routing (prefix sums, no arrival-order
    slot claims), so results are bit-reproducible in either mode and nothing has to change: the call only reports the mode."""
    return bool(torch.are_deterministic_algorithms_enabled())


def parse_nvlink_status(text: str) -> float:
    """Sum of the per-link GB/s figures in ``nvidia-smi nvlink -s`` output."""
    return sum(float(m) for m in re.findall(r'Link\s+\d+:\s*([0-9.]+)\s*GB/s', text))


def get_nvlink_gbs(default: float = 900.0) -> float:
    """Per-direction NVLink bandwidth of GPU 0 in GB/s: 0.9 x the sum over links that nvidia-smi reports
    (each link is listed with its per-direction rate), or ``default`` when the tool is unavailable."""
    try:
        out = subprocess.run(['nvidia-smi', 'nvlink', '-s', '-i', '0'], capture_output=True, text=True, timeout=10).stdout
        total = parse_nvlink_status(out)
        return total * 0.9 if total > 0 else default
    except Exception:
        return default


def get_rdma_gbs(default: float = 50.0) -> float:
    """No NIC path exists in a single-box build; kept for API parity."""
    return default
