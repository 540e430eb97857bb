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
        # ---- back to back without any host synchronisation: ten dispatch -> combine rounds with different data in flight
        # behind one another (receive slots and the two combine input regions are recycled while peers may still be busy
        # with the previous round); everything is checked at the end
        t = T - rank
        rounds = []
        for rnd in range(10):
            torch.manual_seed(1000 + rnd * 10 + rank)
            x = torch.randn(t, H, device='cuda').bfloat16()
            w, idx = torch.softmax(torch.randn(t, E, device='cuda'), -1).topk(K, -1)
            (rx, rsf), ridx, rw, handle, _ = buf.dispatch(x, idx, w, num_experts=E, num_sms=8, do_cpu_sync=False)
            n = handle.psum_num_recv_tokens_per_scaleup_rank[-1:]
            y = buf.get_combine_buffer(handle)
            # "expert": dequantise the received row and scale it by (1 + local expert hits); rows past the valid count are unused
            hits = (ridx >= 0).sum(dim=1, keepdim=True).float()
            y.copy_((rx.float().view(rx.shape[0], -1, 128) * rsf.unsqueeze(-1)).view(rx.shape[0], H) * hits)
            out, _, _ = buf.combine(y, handle, num_sms=8)
            rounds.append((x, idx, out))
        torch.cuda.synchronize()
        buf.check_status()
        from deepep_ascend_b200.utils.math import per_token_cast_back
        for x, idx, out in rounds:
            xq = per_token_cast_back(*per_token_cast_to_fp8(x.cpu())).cuda()
            valid = (idx >= 0).sum(dim=1, keepdim=True).float()          # every valid selection contributes its row once
            torch.testing.assert_close(out.float(), xq.float() * valid, atol=0.13, rtol=0.02)
        buf.barrier(with_cpu_sync=True)
        buf.destroy()
        # ---- the same exchange over buffers allocated with CUDA virtual memory and shared as file descriptors
        vbuf = ep.ElasticBuffer(group, num_max_tokens_per_rank=T, hidden=H, num_topk=K, use_fp8_dispatch=True, symmetric_memory='vmm',
                                num_gpu_timeout_secs=10, num_cpu_timeout_secs=30)
        assert vbuf.core.uses_vmm()
        torch.manual_seed(500 + rank)
        x = torch.randn(T - rank, H, device='cuda').bfloat16()
        w, idx = torch.softmax(torch.randn(T - rank, E, device='cuda'), -1).topk(K, -1)
        (rx, rsf), ridx, rw, handle, _ = vbuf.dispatch(x, idx, w, num_experts=E, num_sms=8)
        q, sf = per_token_cast_to_fp8(x.cpu())
        (ox, osf), oidx, ow, osrc, _ = refs.dispatch_nccl((q.cuda(), sf.cuda()), idx, w, T, E, group)
        assert torch.equal(rx.view(torch.uint8), ox.view(torch.uint8)) and torch.equal(rsf, osf) and torch.equal(ridx, oidx)
        out, _, _ = vbuf.combine(per_token_cast_back(rx, rsf).bfloat16(), handle, num_sms=8)
        hits = torch.zeros(x.shape[0], device='cuda')
        prank, _ = layout_ref.unpack_lane(handle.plan)
        hits = (prank >= 0).sum(dim=1, keepdim=True).float()
        torch.testing.assert_close(out.float(), per_token_cast_back(q, sf).cuda().float() * hits, atol=0.07, rtol=0.02)
        vbuf.check_status()
        vbuf.destroy()
        # ---- expand layout with aligned, zero-padded expert segments and the fused weighted reduce
        A = 16
        buf = ep.ElasticBuffer(group, num_max_tokens_per_rank=T, hidden=H, num_topk=K, use_fp8_dispatch=False, enable_expand=True,
                               num_experts=E, expert_alignment=A, num_gpu_timeout_secs=10, num_cpu_timeout_secs=30)
        torch.manual_seed(77 + rank)
        x = torch.randn(T - rank, H, device='cuda').bfloat16()
        w, idx = torch.softmax(torch.randn(T - rank, E, device='cuda'), -1).topk(K, -1)
        rx, ridx, rw, handle, _ = buf.dispatch(x, idx, w, num_experts=E, num_sms=8, do_expand=True, expert_alignment=A, do_zero_padding=True)
        assert ridx is None and rw.dim() == 1 and rx.shape[0] == handle.num_expanded_tokens
        ends = handle.psum_num_recv_tokens_per_expert.long().cpu()
        starts = torch.cat([torch.zeros(1, dtype=torch.long), (ends[:-1] + A - 1) // A * A])
        for j in range(E // world):
            assert handle.num_recv_tokens_per_expert_list[j] % A == 0
            pad = rx[int(ends[j]):int((ends[j] + A - 1) // A * A)]
            assert bool((pad == 0).all()), 'alignment padding must be zeroed by the kernel'
            assert int(ends[j] - starts[j]) == int(handle.num_unaligned_recv_tokens_per_expert[j])
        out, _, _ = buf.combine(rx, handle, weighted=True, num_sms=8)      # identity experts: sum_k w_k x
        torch.testing.assert_close(out.float(), x.float() * w.sum(-1, keepdim=True), atol=3e-2, rtol=2e-2)
        buf.check_status()
        buf.destroy()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('world', [2, 4, 8])
def test_multi_process_dispatch_combine(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f'needs {world} GPUs')
    mp.spawn(_worker, args=(world, _free_port()), nprocs=world, join=True)


def _worker_misc(rank: int, world: int, port: int):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        import deepep_ascend_b200 as ep
        from deepep_ascend_b200.utils.math import per_token_cast_back
        group = dist.new_group(list(range(world)))
        M, H, E, K = 64, 2048, 8 * world, 4
        extra = ep.ElasticBuffer.get_low_latency_size_hint(M, H, world, E, K) + (96 << 20)
        buf = ep.ElasticBuffer(group, num_max_tokens_per_rank=256, hidden=H, num_topk=K, extra_bytes=extra,
                               num_gpu_timeout_secs=10, num_cpu_timeout_secs=30, num_cpu_bytes=1 << 20)
        # ---- all-gather / reduce-scatter session
        buf.agrs_set_config(64 << 20)
        buf.create_agrs_session()
        x = torch.full((300, 40), float(rank + 1), device='cuda', dtype=torch.bfloat16)
        inplace = buf.agrs_get_inplace_tensor((16, 8), torch.float32)
        inplace.fill_(rank + 0.5)
        (g1, g2), wait = buf.all_gather([x, inplace])
        wait()
        for r in range(world):
            assert bool((g1[r] == r + 1).all()) and bool((g2[r] == r + 0.5).all())
        rs_in = torch.randn(world, 1000, device='cuda', generator=torch.Generator('cuda').manual_seed(rank)).bfloat16()
        out, wait = buf.reduce_scatter(rs_in)
        wait()
        gathered = [torch.empty_like(rs_in) for _ in range(world)]
        dist.all_gather(gathered, rs_in, group=group)
        acc = torch.zeros(1000, device='cuda')
        for s in range(world):
            acc += gathered[s][rank].float()
        assert torch.equal(out, acc.bfloat16())
        buf.destroy_agrs_session()
        # ---- the same session with completion signalled by stream memory operations (no SM at all)
        if buf.core.signal_and_wait_memops(buf._C.CH_AGRS):      # the driver accepts them on this machine
            buf._agrs['memops'] = True
            for it in range(3):
                buf.create_agrs_session()
                xs_ = torch.full((257, 16), float(10 * it + rank), device='cuda', dtype=torch.bfloat16)
                gathered, wait = buf.all_gather(xs_)
                wait()
                for r in range(world):
                    assert bool((gathered[r] == 10 * it + r).all()), (it, r)
                out, wait = buf.reduce_scatter(rs_in)
                wait()
                assert torch.equal(out, acc.bfloat16())
                buf.destroy_agrs_session()
            buf._agrs['memops'] = False
        # ---- pipeline send / recv around the ring
        buf.pp_set_config(1 << 20, 4)
        nxt, prv = (rank + 1) % world, (rank - 1) % world
        send = torch.full((1024,), float(rank), device='cuda')
        recv = torch.empty_like(send)
        if rank % 2 == 0:
            buf.pp_send(send, nxt)
            buf.pp_recv(recv, prv)
        else:
            buf.pp_recv(recv, prv)
            buf.pp_send(send, nxt)
        torch.cuda.synchronize()
        assert bool((recv == prv).all())
        # ---- pipeline: a random schedule (same on every rank) of directions and sizes, with random GPU-side skew in
        # front of the calls; every received tensor must hold what the neighbour sent in that step
        import random
        rng = random.Random(4242)
        for step in range(12):
            forward, n = rng.random() < 0.5, rng.choice([1, 257, 4096, 65536])
            skew = [rng.randint(0, 3) * 200_000 for _ in range(world)]
            dst, src = (nxt, prv) if forward else (prv, nxt)
            send = torch.full((n,), float(rank * 100 + step), device='cuda')
            recv = torch.empty_like(send)
            if skew[rank]:
                torch.cuda._sleep(skew[rank])
            if rank % 2 == 0:
                buf.pp_send(send, dst)
                buf.pp_recv(recv, src)
            else:
                buf.pp_recv(recv, src)
                buf.pp_send(send, dst)
            torch.cuda.synchronize()
            assert bool((recv == src * 100 + step).all()), (step, forward, n)
        # ---- Engram: the tables live in the CPU segments (pinned host memory that every rank's GPU maps); scales come from
        # a table replicated on every rank
        table = torch.full((100, 256), float(rank), device='cuda', dtype=torch.bfloat16) + torch.arange(100, device='cuda').unsqueeze(1).bfloat16()
        sf_table = (torch.arange(100 * world * 2, device='cuda', dtype=torch.float32) * 0.5).view(100 * world, 2)
        buf.engram_write(table, sf_table)
        assert buf._engram['cpu']
        idx = torch.randint(0, 100 * world, (50, 2), device='cuda', dtype=torch.int32)
        for col_major in (False, True):
            fetched, fetched_sf = buf.engram_fetch(idx, use_tma_aligned_col_major_sf=col_major)()
            want = (idx // 100).float().unsqueeze(-1) + (idx % 100).float().unsqueeze(-1)
            assert torch.equal(fetched.view(50, 2, 256).float(), want.expand(50, 2, 256).bfloat16().float())
            assert torch.equal(fetched_sf, sf_table[idx.long().view(-1)].view(50, 4))
            assert fetched_sf.stride() == ((1, 52) if col_major else (4, 1))
        # ---- low latency (also in hook mode) and its use through the legacy API names
        torch.manual_seed(rank)
        xt = torch.randn(M - rank, H, device='cuda').bfloat16()
        w, idx2 = torch.softmax(torch.randn(M - rank, E, device='cuda'), -1).topk(K, -1)
        for hook_mode in (False, True):
            (rx, rsf), count, handle, _, hook = buf.low_latency_dispatch(xt, idx2, M, E, return_recv_hook=hook_mode)
            if hook_mode:
                hook()
            y = torch.zeros(rx.shape, dtype=torch.bfloat16, device='cuda')
            for j in range(E // world):
                n = int(count[j])
                y[j, :n] = per_token_cast_back(rx[j, :n], rsf[j, :n])
            out, _, hook = buf.low_latency_combine(y, idx2, w, handle, return_recv_hook=hook_mode)
            if hook_mode:
                hook()
            torch.cuda.synchronize()
            want = xt.float() * w.sum(-1, keepdim=True)
            assert float((out.float() - want).abs().max()) < 0.3
        buf.check_status()
        buf.destroy()
        # ---- first-generation API
        legacy = ep.Buffer(group, num_nvl_bytes=0)
        xt = torch.randn(128, 1024, device='cuda').bfloat16()
        w, idx3 = torch.softmax(torch.randn(128, E, device='cuda'), -1).topk(K, -1)
        per_rank, _, per_expert, in_rank, _ = legacy.get_dispatch_layout(idx3, E)
        rx, ridx, rw, per_expert_list, h, _ = legacy.dispatch(xt, topk_idx=idx3, topk_weights=w, num_tokens_per_rank=per_rank,
                                                              is_token_in_rank=in_rank, num_tokens_per_expert=per_expert)
        assert sum(per_expert_list) == int((ridx >= 0).sum())
        cx, cw, _ = legacy.combine(rx, h, topk_weights=rw)
        hits = in_rank.sum(dim=1, keepdim=True).float()
        assert float((cx.float() - xt.float() * hits).abs().max()) < 0.13 and torch.equal(cw, w)
        legacy.destroy()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('world', [2, 8])
def test_multi_process_collectives_ll_legacy(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f'needs {world} GPUs')
    mp.spawn(_worker_misc, args=(world, _free_port()), nprocs=world, join=True)


def _worker_tp(rank: int, world: int, port: int):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        import deepep_ascend_b200 as ep
        from deepep_ascend_b200.parallel.tp import TensorParallelGemm
        group = dist.new_group(list(range(world)))
        M, K, N = 128 * world * 3, 1024, 512
        buf = ep.ElasticBuffer(group, num_max_tokens_per_rank=16, hidden=256, num_topk=2, extra_bytes=TensorParallelGemm.size_hint(M, K, N),
                               num_gpu_timeout_secs=10)
        tp = TensorParallelGemm(buf, M, K, N, num_sms=32, num_copy_ctas=4)
        for it in range(3):
            g = torch.Generator('cuda').manual_seed(100 * it + rank)
            x_shard = torch.randn(M // world, K, device='cuda', generator=g).bfloat16()
            w = torch.randn(N, K, device='cuda', generator=g).bfloat16() * 0.1
            c = tp.ag_gemm(x_shard, w)
            gathered = [torch.empty_like(x_shard) for _ in range(world)]
            dist.all_gather(gathered, x_shard, group=group)
            ref = torch.cat(gathered).float() @ w.float().t()
            assert float((c.float() - ref).abs().max()) <= 2e-2 * float(ref.abs().max()) + 1e-2
            # reduce-scatter of the partial products
            x = torch.randn(M, K, device='cuda', generator=g).bfloat16()
            out = tp.gemm_rs(x, w)
            partial = (x.float() @ w.float().t()).bfloat16()
            parts = [torch.empty_like(partial) for _ in range(world)]
            dist.all_gather(parts, partial, group=group)
            rows = slice(rank * (M // world), (rank + 1) * (M // world))
            acc = torch.zeros(M // world, N, device='cuda')
            for p in parts:
                acc += p[rows].float()
            assert float((out.float() - acc).abs().max()) <= 2e-2 * float(acc.abs().max()) + 1e-2
        torch.cuda.synchronize()
        buf.check_status()
        assert buf._C.gemm_error(rank) == 0
        buf.destroy()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('world', [2, 8])
def test_multi_process_fused_tp_gemm(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f'needs {world} GPUs')
    mp.spawn(_worker_tp, args=(world, _free_port()), nprocs=world, join=True)


def _worker_moe(rank: int, world: int, port: int):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        import deepep_ascend_b200 as ep
        from deepep_ascend_b200.models.moe import FusedMoE, moe_reference
        from deepep_ascend_b200.utils.math import calc_diff
        group = dist.new_group(list(range(world)))
        T, H, I, K = 384, 512, 256, 4
        E = 4 * world
        buf = ep.ElasticBuffer(group, num_max_tokens_per_rank=T, hidden=H, num_topk=K, enable_expand=True, num_experts=E,
                               expert_alignment=128, num_gpu_timeout_secs=10, num_cpu_timeout_secs=30)
        torch.manual_seed(5 + rank)
        layer = FusedMoE(buf, E, H, I, init_std=0.05, num_sms=8)
        # every rank needs all experts' weights for the reference
        def gather(p):
            parts = [torch.empty_like(p.data) for _ in range(world)]
            dist.all_gather(parts, p.data.contiguous(), group=group)
            return torch.cat(parts).float()
        w13_all, w2_all = gather(layer.w13), gather(layer.w2)
        for chunks, local_expand in ((1, True), (3, True), (1, False)):
            layer.num_chunks, layer.local_expand = chunks, local_expand
            layer.zero_grad()
            x = torch.randn(T - 5 * rank, H, device='cuda').bfloat16().requires_grad_(True)
            wts, idx = torch.softmax(torch.randn(x.shape[0], E, device='cuda'), dim=-1).topk(K, dim=-1)
            idx[::9, 1] = -1
            wts = wts.clone().requires_grad_(True)
            out = layer(x, idx, wts)
            g = torch.randn_like(out)
            out.backward(g)
            torch.cuda.synchronize()
            buf.check_status()
            xr, wr = x.detach().float().requires_grad_(True), wts.detach().clone().requires_grad_(True)
            w13r, w2r = w13_all.clone().requires_grad_(True), w2_all.clone().requires_grad_(True)
            ref = moe_reference(xr, idx, wr, w13r, w2r)
            ref.backward(g.float())
            # weight gradients: every rank's tokens contribute to every expert
            dist.all_reduce(w13r.grad, group=group)
            dist.all_reduce(w2r.grad, group=group)
            El = E // world
            sl = slice(rank * El, (rank + 1) * El)
            for name, got, want in (('out', out.float(), ref), ('dx', x.grad.float(), xr.grad), ('dw', wts.grad, wr.grad),
                                    ('d_w2', layer.w2.grad.float(), w2r.grad[sl]), ('d_w13', layer.w13.grad.float(), w13r.grad[sl])):
                d = calc_diff(got, want)
                assert d < 3e-3, (chunks, local_expand, name, d)
        buf.destroy()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('world', [2, 8])
def test_multi_process_fused_moe(world):
    """The fused MoE layer on several GPUs, as one pass and as a three-chunk pipeline: output and all four gradients against
    the plain PyTorch layer that holds every expert's weights."""
    if torch.cuda.device_count() < world:
        pytest.skip(f'needs {world} GPUs')
    mp.spawn(_worker_moe, args=(world, _free_port()), nprocs=world, join=True)
