"""One process per GPU over NCCL + cudaIpc-mapped symmetric buffers; needs at least 2 GPUs.
Dispatch / combine are checked bitwise against the all_to_all_single oracle."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        import deepep_ascend_b200 as ep
        from deepep_ascend_b200.utils import refs
        from deepep_ascend_b200.utils.math import per_token_cast_to_fp8
        group = dist.new_group(list(range(world)))
        T, H, E, K = 512, 2048, 8 * world, 4
        buf = ep.ElasticBuffer(group, num_max_tokens_per_rank=T, hidden=H, num_topk=K, use_fp8_dispatch=True,
                               num_gpu_timeout_secs=10, num_cpu_timeout_secs=30)
        for seed in range(3):
            torch.manual_seed(seed * 10 + rank)
            t = T - 17 * rank - seed
            x = torch.randn(t, H, device='cuda').bfloat16()
            w, idx = torch.softmax(torch.randn(t, E, device='cuda'), -1).topk(K, -1)
            idx[torch.rand(idx.shape, device='cuda') < 0.05] = -1
            (rx, rsf), ridx, rw, handle, _ = buf.dispatch(x, idx, w, num_experts=E, num_sms=8)
            q, sf = per_token_cast_to_fp8(x.cpu())
            (ox, osf), oidx, ow, osrc, _ = refs.dispatch_nccl((q.cuda(), sf.cuda()), idx, w, T, E, group)
            assert rx.shape[0] == ox.shape[0] == handle.num_recv_tokens
            assert torch.equal(rx.view(torch.uint8), ox.view(torch.uint8)) and torch.equal(rsf, osf)
            assert torch.equal(ridx, oidx) and torch.equal(rw, ow)
            assert torch.equal(handle.recv_src_metadata[:, 0], osrc)
            # combine: rows regenerated from the source token id, so every rank can rebuild the expected sum
            y = refs.generate_pre_combine_data(handle.recv_src_metadata[:, 0] * world + rank, world * world * T, H, seed)
            out, back_w, _ = buf.combine(y, handle, topk_weights=rw)
            src = torch.arange(t, device='cuda') + rank * T
            acc = torch.zeros(t, H, device='cuda')
            from deepep_ascend_b200.ops import layout_ref
            prank, _ = layout_ref.unpack_lane(handle.plan)
            for k in range(K):
                m = prank[:, k] >= 0
                rows = refs.generate_pre_combine_data(src[m] * world + prank[m, k], world * world * T, H, seed)
                acc[m] += rows.float()
            assert torch.equal(out.view(torch.int16), acc.bfloat16().view(torch.int16))
            valid = idx >= 0
            assert torch.equal(back_w[valid], w[valid])
        buf.barrier(with_cpu_sync=True)
        buf.destroy()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('world', [2, 4, 8])
def test_multi_process_dispatch_combine(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f'needs {world} GPUs')
    mp.spawn(_worker, args=(world, _free_port()), nprocs=world, join=True)
