"""The non-MoE operations and the low-latency pair on the CPU / gloo backend (world size 2): all-gather / reduce-scatter
sessions, pipeline send / recv, Engram tables, low-latency dispatch / combine with their packed layout and handle."""
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


def _setup(rank, world, port):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    import deepep_ascend_b200 as ep
    group = dist.new_group(list(range(world)))
    return ep, group


def _worker_sessions(rank, world, port):
    ep, group = _setup(rank, world, port)
    try:
        buf = ep.ElasticBuffer(group, num_max_tokens_per_rank=16, hidden=64, num_topk=2)
        buf.agrs_set_config(1 << 20, 8)
        for session in range(2):                                   # the region is recycled by the second session
            buf.create_agrs_session()
            a = (torch.arange(6, dtype=torch.float32).reshape(2, 3) + 100 * rank + session)
            b = (torch.randn(5, 4, generator=torch.Generator().manual_seed(rank)) * 3).bfloat16()
            (ga, gb), wait = buf.all_gather([a, b])
            wait()
            for r in range(world):
                assert torch.equal(ga[r], torch.arange(6, dtype=torch.float32).reshape(2, 3) + 100 * r + session)
                assert torch.equal(gb[r], (torch.randn(5, 4, generator=torch.Generator().manual_seed(r)) * 3).bfloat16())
            # a producer writes straight into its slice of the gather slot
            mine = buf.agrs_get_inplace_tensor((3, 2), torch.float32)
            mine.fill_(7.0 + rank)
            g, wait = buf.all_gather(mine)
            wait()
            assert [float(g[r][0, 0]) for r in range(world)] == [7.0 + r for r in range(world)]
            # reduce-scatter: rank r receives the sum of everybody's slice r, accumulated in fp32
            t = torch.stack([torch.full((4,), float(10 * rank + p)) for p in range(world)]).bfloat16()
            out, wait = buf.reduce_scatter(t)
            wait()
            assert out.dtype == torch.bfloat16 and out.tolist() == [float(sum(10 * s + rank for s in range(world)))] * 4
            k_all, v_all, wait = buf.cp_all_gather_kv(torch.full((2, 2), float(rank)), torch.full((2, 2), float(-rank)))
            assert float(k_all[1 % world].sum()) == 4.0 * (1 % world) and float(v_all[1 % world].sum()) == -4.0 * (1 % world)
            buf.destroy_agrs_session()
        with pytest.raises(AssertionError, match='no open AG/RS session'):
            buf.all_gather(torch.zeros(2))
        # pipeline ring: everybody sends to the next rank and receives from the previous one
        buf.pp_set_config(1 << 16, 4)
        nxt, prv = (rank + 1) % world, (rank - 1) % world
        for step in range(3):
            payload = torch.full((8, 4), float(rank * 10 + step)).bfloat16()
            got = torch.empty_like(payload)
            buf.pp_send(payload, nxt)
            buf.pp_recv(got, prv)
            assert float(got[0, 0]) == float(prv * 10 + step)
        # Engram: every rank publishes a table; a fetch returns arbitrary rows of any rank, with their scales
        N, H = 6, 32
        table = (torch.arange(N * H, dtype=torch.float32).reshape(N, H) + 1000 * rank).bfloat16()
        sf_all = torch.arange(world * N * 2, dtype=torch.float32).reshape(world * N, 2)
        buf.engram_write(table, sf=sf_all)
        idx = torch.tensor([[0, N + 1], [N - 1, 2 * N - 1 if world > 1 else N - 1]], dtype=torch.int32)
        for col_major in (False, True):
            fetched, fsf = buf.engram_fetch(idx, use_tma_aligned_col_major_sf=col_major)()
            for t in range(2):
                for n in range(2):
                    gid = int(idx[t, n])
                    owner, row = gid // N, gid % N
                    want = (torch.arange(H, dtype=torch.float32) + row * H + 1000 * owner).bfloat16()
                    assert torch.equal(fetched[t, n * H:(n + 1) * H], want)
                    assert torch.equal(fsf[t, n * 2:(n + 1) * 2], sf_all[gid])
            assert fsf.stride() == ((1, 4) if col_major else (4, 1))
        buf.destroy()
    finally:
        dist.destroy_process_group()


def test_gloo_sessions_pipeline_and_engram():
    mp.spawn(_worker_sessions, args=(2, _free_port()), nprocs=2, join=True)


def _worker_low_latency(rank, world, port, mode):
    ep, group = _setup(rank, world, port)
    try:
        from deepep_ascend_b200.utils.math import logfmt10_roundtrip, per_token_cast_back, per_token_cast_to_fp8
        T, H, E, K, M = 20 - 3 * rank, 256, 8, 3, 24
        El = E // world
        g = torch.Generator().manual_seed(50 + rank)
        x = (torch.randn(T, H, generator=g) * (1 + rank)).bfloat16()
        idx = torch.rand(T, E, generator=g).topk(K, dim=-1).indices
        idx[torch.rand(idx.shape, generator=g) < 0.15] = -1
        w = torch.rand(T, K, generator=g)
        buf = ep.ElasticBuffer(group, num_max_tokens_per_rank=M, hidden=H, num_topk=K)
        use_fp8 = mode != 'bf16'
        stats = torch.zeros(El, dtype=torch.int32)
        recv, count, handle, _, hook = buf.low_latency_dispatch(x, idx, M, E, cumulative_local_expert_recv_stats=stats, use_fp8=use_fp8,
                                                                use_ue8m0=(mode == 'ue8m0'))
        assert hook is None and torch.equal(stats, count)
        src_info, layout_range = handle[0], handle[1]
        # what every rank sent, gathered for the check
        all_x, all_idx = [None] * world, [None] * world
        dist.all_gather_object(all_x, x, group=group)
        dist.all_gather_object(all_idx, idx, group=group)
        rx, rsf = recv if use_fp8 else (recv, None)
        assert rx.shape == (El, world * M, H)
        y = torch.zeros(El, world * M, H, dtype=torch.bfloat16)
        for j in range(El):
            e, total = rank * El + j, 0
            for s in range(world):
                n, begin = int(layout_range[j, s]) & 0xffffffff, int(layout_range[j, s]) >> 32
                want_t = sorted((all_idx[s] == e).any(dim=1).nonzero().flatten().tolist())
                info = src_info[j, begin:begin + n]
                got_t, got_k = (info & 0xfffff).tolist(), (info >> 20).tolist()
                assert sorted(got_t) == want_t and begin == total
                total += n
                ref = per_token_cast_to_fp8(all_x[s], round_scale=(mode == 'ue8m0'), use_ue8m0=(mode == 'ue8m0')) if use_fp8 else None
                for i, (t, k) in enumerate(zip(got_t, got_k)):
                    assert int(all_idx[s][t, k]) == e
                    if use_fp8:
                        assert torch.equal(rx[j, begin + i].view(torch.uint8), ref[0][t].view(torch.uint8))
                        assert torch.equal(rsf[j, begin + i], ref[1][t])
                        val = per_token_cast_back(ref[0][t:t + 1], ref[1][t:t + 1])[0]
                    else:
                        assert torch.equal(rx[j, begin + i], all_x[s][t])
                        val = all_x[s][t]
                    y[j, begin + i] = (val.float() * (1 + 0.5 * (e % 2))).bfloat16()
            assert int(count[j]) == total
        target = buf.get_next_low_latency_combine_buffer(handle)
        target.copy_(y)
        for use_logfmt in (False, True):
            out, _, _ = buf.low_latency_combine(target, idx, w, handle, use_logfmt=use_logfmt)
            xd = per_token_cast_back(*per_token_cast_to_fp8(x, round_scale=(mode == 'ue8m0'), use_ue8m0=(mode == 'ue8m0'))) if use_fp8 else x
            want = torch.zeros(T, H)
            for k in range(K):
                m = idx[:, k] >= 0
                yk = (xd[m].float() * (1 + 0.5 * (idx[m, k] % 2)).unsqueeze(1)).bfloat16()
                yk = logfmt10_roundtrip(yk) if use_logfmt else yk.float()
                want[m] += w[m, k].unsqueeze(1) * yk
            torch.testing.assert_close(out.float(), want.bfloat16().float(), atol=2e-2, rtol=2e-2)
        # a masked rank is skipped: nothing is sent to it and nothing of it is combined
        if world > 1:
            buf.low_latency_update_mask_buffer(1, True)
            assert buf.low_latency_query_mask_buffer().tolist() == [0, 1]
            recv2, count2, handle2, _, _ = buf.low_latency_dispatch(x, idx, M, E, use_fp8=False)
            # rank 1 is skipped as a destination and ignored as a source: rank 0 keeps its own pairs only, rank 1 gets nothing
            own_pairs = int(((idx >= 0) & (idx // El == rank)).sum())
            assert int(count2.sum()) == (own_pairs if rank == 0 else 0)
            buf.low_latency_clean_mask_buffer()
            assert buf.low_latency_query_mask_buffer().tolist() == [0, 0]
        buf.destroy()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('mode', ['bf16', 'fp8', 'ue8m0'])
def test_gloo_low_latency_roundtrip(mode):
    mp.spawn(_worker_low_latency, args=(2, _free_port(), mode), nprocs=2, join=True)


def _worker_legacy(rank, world, port):
    ep, group = _setup(rank, world, port)
    try:
        T, H, E, K = 24, 128, 8, 2
        g = torch.Generator().manual_seed(7 + rank)
        x = torch.randn(T, H, generator=g).bfloat16()
        w, idx = torch.softmax(torch.randn(T, E, generator=g), dim=-1).topk(K, dim=-1)
        buf = ep.Buffer(group, num_nvl_bytes=1 << 20, num_rdma_bytes=0)
        per_rank, per_rdma, per_expert, in_rank, _ = buf.get_dispatch_layout(idx, E)
        assert per_rdma is None and per_rank.tolist() == [int(((idx // (E // world)) == r).any(dim=1).sum()) for r in range(world)]
        recv_x, recv_idx, recv_w, per_expert_list, handle, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_tokens_per_rank=per_rank,
                                                                            is_token_in_rank=in_rank, num_tokens_per_expert=per_expert)
        assert sum(per_expert_list) == int((recv_idx >= 0).sum()) and recv_x.shape[0] == recv_idx.shape[0]
        # identity experts: every received row goes back once per rank, so a token comes home as (ranks it visited) * x
        out, out_w, _ = buf.intranode_combine(recv_x, handle, topk_weights=recv_w)
        visits = in_rank.sum(dim=1, keepdim=True).float()
        torch.testing.assert_close(out.float(), (x.float() * visits).bfloat16().float(), atol=2e-2, rtol=2e-2)
        assert torch.equal(out_w, w)
        # the cached form takes the handle tuple
        again = buf.dispatch(x, handle=handle)[0]
        assert torch.equal(again, recv_x)
        # low-latency pair through the same object
        M = 32
        recv, count, ll_handle, _, _ = buf.low_latency_dispatch(x, idx, M, E, use_fp8=False)
        y = buf.get_next_low_latency_combine_buffer(ll_handle)
        y.copy_(recv)
        res, _, _ = buf.low_latency_combine(y, idx, w, ll_handle)
        torch.testing.assert_close(res.float(), (x.float() * w.sum(dim=1, keepdim=True)).bfloat16().float(), atol=3e-2, rtol=3e-2)
        assert buf.is_available() and buf.get_num_rdma_ranks() == 1 and buf.get_local_nvshmem_unique_id() == b''
        buf.destroy()
    finally:
        dist.destroy_process_group()


def test_gloo_legacy_buffer():
    """The legacy ``Buffer`` surface on two gloo ranks: layout, dispatch / combine with the handle tuple, cached dispatch,
    the transport-named aliases and the low-latency pair."""
    mp.spawn(_worker_legacy, args=(2, _free_port()), nprocs=2, join=True)
