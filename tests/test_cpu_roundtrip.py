"""CPU / gloo world_size=2 round trip: 128 tokens per rank, hidden 256, fp32-valued activations,
8 experts (4 per rank), top-2 of softmax(logits) renormalised; the expert is the identity, so
combine(dispatch(x)) weighted by the routing weights must return sum_k w_k * x = x."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, do_expand: bool, use_fp8: bool):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        import deepep_ascend_b200 as ep
        from deepep_ascend_b200.ops import layout_ref
        from deepep_ascend_b200.utils.math import per_token_cast_back
        torch.manual_seed(rank)
        T, H, E, K = 128, 256, 8, 2
        x = torch.randn(T, H).bfloat16()
        logits = torch.randn(T, E)
        w, idx = torch.softmax(logits, dim=-1).topk(K, dim=-1)
        w = w / w.sum(dim=-1, keepdim=True)
        group = dist.new_group(list(range(world)))
        buf = ep.ElasticBuffer(group, num_max_tokens_per_rank=T, hidden=H, num_topk=K, use_fp8_dispatch=use_fp8,
                               enable_expand=do_expand, num_experts=E)
        stats = torch.zeros(E // world, dtype=torch.int32)
        recv_x, recv_idx, recv_w, handle, _ = buf.dispatch(x, idx, w, cumulative_local_expert_recv_stats=stats,
                                                           num_experts=E, do_expand=do_expand, expert_alignment=4 if do_expand else 1)
        # layout counts against a direct count
        per_rank, per_expert, _ = layout_ref.get_dispatch_layout_ref(idx, E, world)
        all_per_expert = [torch.zeros_like(per_expert) for _ in range(world)]
        dist.all_gather(all_per_expert, per_expert)
        El = E // world
        expect = torch.stack(all_per_expert).sum(0)[rank * El:(rank + 1) * El]
        assert handle.num_unaligned_recv_tokens_per_expert.tolist() == expect.tolist()
        assert stats.tolist() == expect.tolist()
        if use_fp8:
            recv_x = per_token_cast_back(*recv_x)
        if do_expand:
            assert recv_idx is None and recv_w.dim() == 1
            y = recv_x
            out, _, _ = buf.combine(y, handle, weighted=True)
            ref = x.float() if not use_fp8 else None
        else:
            assert int(handle.psum_num_recv_tokens_per_scaleup_rank[-1]) == recv_x.shape[0] == handle.num_recv_tokens
            # identity expert with per-row weighting done by the "expert" side: y_row = sum_{k local} w_k * x
            local = (recv_idx >= 0)
            y = (recv_x.float() * (recv_w * local).sum(dim=1, keepdim=True)).bfloat16()
            out, back_w, _ = buf.combine(y, handle, topk_weights=recv_w)
            assert torch.equal(back_w, w), 'weights carried back must be bit-identical'
            ref = x.float() if not use_fp8 else None
        if ref is not None:
            assert (out.float() - ref).abs().max() < 0.06, float((out.float() - ref).abs().max())
        else:
            assert (out.float() - x.float()).abs().max() < 0.35
        # cached re-dispatch returns the same rows
        recv_x2, _, _, _, _ = buf.dispatch(x, handle=handle, topk_weights=w)
        a = recv_x2[0] if use_fp8 else recv_x2
        b = buf.dispatch(x, idx, w, num_experts=E, do_expand=do_expand, expert_alignment=4 if do_expand else 1)[0]
        b = b[0] if use_fp8 else b
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
        buf.destroy()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('do_expand,use_fp8', [(False, False), (True, False), (False, True)])
def test_gloo_roundtrip(do_expand, use_fp8):
    mp.spawn(_worker, args=(2, _free_port(), do_expand, use_fp8), nprocs=2, join=True)
