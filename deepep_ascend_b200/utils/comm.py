"""Exchange of symmetric-memory handles over a process group (parity: deep_ep/utils/comm.py:11-83; this build
maps peers with its own cudaIpc handles instead of NCCL windows, so no NCCL communicator is needed)."""
from typing import Any, List

import torch.distributed as dist


def all_gather_object(group: dist.ProcessGroup, obj: Any) -> List[Any]:
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, obj, group=group)
    return out
