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


def _worker(rank: int, world: int, port: int, do_expand: bool, use_fp8: bool, dtype=torch.bfloat16):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        import deepep_ascend_b200 as ep
        from deepep_ascend_b200.ops import layout_ref
        from deepep_ascend_b200.utils.math import per_token_cast_back
        torch.manual_seed(rank)
        T, H, E, K = 128, 256, 8, 2
        x = torch.randn(T, H).to(dtype)
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
            y = (recv_x.float() * (recv_w * local).sum(dim=1, keepdim=True)).to(recv_x.dtype)
            out, back_w, _ = buf.combine(y, handle, topk_weights=recv_w)
            assert torch.equal(back_w, w), 'weights carried back must be bit-identical'
            ref = x.float() if not use_fp8 else None
        if ref is not None:
            assert out.dtype == (torch.bfloat16 if use_fp8 else dtype)
            tol = 0.06 if dtype == torch.bfloat16 else 1e-5
            assert (out.float() - ref).abs().max() < tol, float((out.float() - ref).abs().max())
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


@pytest.mark.parametrize('do_expand', [False, True])
def test_gloo_roundtrip_fp32_activations(do_expand):
    """The round trip with fp32 activations x ~ N(0, 1): sum_k w_k * x comes back to within fp32 rounding."""
    mp.spawn(_worker, args=(2, _free_port(), do_expand, False, torch.float32), nprocs=2, join=True)


def _failure_worker(rank: int, world: int, port: int, case: str):
    from datetime import timedelta
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world, timeout=timedelta(seconds=6))
    try:
        import deepep_ascend_b200 as ep
        from deepep_ascend_b200.backends.cpu import CollectiveMismatch
        from deepep_ascend_b200.buffers.elastic import HandleError
        torch.manual_seed(rank)
        T, H, E, K = 32, 64, 8, 2
        x = torch.randn(T, H)
        w, idx = torch.softmax(torch.randn(T, E), dim=-1).topk(K, dim=-1)
        group = dist.new_group(list(range(world)), timeout=timedelta(seconds=6))
        buf = ep.ElasticBuffer(group, num_max_tokens_per_rank=T, hidden=H, num_topk=K)
        if case == 'mismatched_num_experts':
            # rank 1 believes there are 16 experts: every rank gets an error that names the odd rank, nothing hangs
            with pytest.raises(CollectiveMismatch, match=r'ranks \[1\] disagree'):
                buf.dispatch(x, idx, w, num_experts=E if rank == 0 else 2 * E)
        elif case == 'rank_skips_call':
            # rank 1 never makes the call: rank 0 gets a rank-qualified error once the process group's limit runs out
            if rank == 0:
                with pytest.raises(CollectiveMismatch, match=r'\[EP rank 0\] dispatch number 1: not every rank joined'):
                    buf.dispatch(x, idx, w, num_experts=E)
        elif case == 'foreign_handle':
            other = ep.ElasticBuffer(group, num_max_tokens_per_rank=T, hidden=H, num_topk=K)
            rx, _, _, handle, _ = buf.dispatch(x, idx, w, num_experts=E)
            with pytest.raises(HandleError, match='another buffer'):
                other.combine(rx, handle)
            out, _, _ = buf.combine(rx, handle)          # the rightful buffer still works afterwards
            assert out.shape == x.shape
            buf.destroy()
            with pytest.raises(HandleError, match='destroyed'):
                buf._attest(handle, 'combine')
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize('case', ['mismatched_num_experts', 'rank_skips_call', 'foreign_handle'])
def test_gloo_failures_are_reported_not_hung(case):
    """Failures made on the host (a rank with other arguments, a rank that never joins, a handle of another buffer) end
    in an error that names the rank."""
    mp.spawn(_failure_worker, args=(2, _free_port(), case), nprocs=2, join=True)
