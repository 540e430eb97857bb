"""Secondary benchmarks (one JSON line per measurement, rank 0): low-latency decode in a CUDA graph, fused MoE layer
forward+backward, skewed (Zipf) routing, fused tensor-parallel GEMMs, the NCCL all-to-all baseline, the plain
tcgen05 GEMM, and a per-phase breakdown of dispatch / combine.

    python bench_extras.py --gpus 1 --what gemm,ll
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench_extras.py --gpus 8 --what all

All multi-GPU numbers are device times (CUDA events behind a GPU spin that hides launch latency), max over ranks.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import numpy as np
import torch
import torch.distributed as dist

from deepep_ascend_b200 import ElasticBuffer
from deepep_ascend_b200.utils import gate
from deepep_ascend_b200.utils.testing import flush_l2_cache

SLEEP = 6_000_000


def main():
    p = argparse.ArgumentParser()
    p.add_argument('--gpus', type=int, default=1)
    p.add_argument('--what', default='all')
    p.add_argument('--iters', type=int, default=20)
    p.add_argument('--phase-sms', default='24,64', help='SM counts of the dispatch / combine phase breakdown and tuning sweep')
    p.add_argument('--moe-tokens', type=int, default=4096, help='tokens per rank of the fused MoE benchmark')
    p.add_argument('--moe-experts', type=int, default=0, help='experts of the fused MoE benchmark (default 256, or 32 on one GPU)')
    args = p.parse_args()
    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    lr = int(os.environ.get('LOCAL_RANK', '0'))
    assert world == args.gpus
    torch.cuda.set_device(lr)
    group = None
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', lr))
        group = dist.new_group(list(range(world)))
    what = set(args.what.split(','))
    want = lambda k: 'all' in what or k in what

    def emit(**kw):
        if rank == 0:
            print(json.dumps(kw), flush=True)

    def reduce_max(ts):
        t = torch.tensor(ts, dtype=torch.float64, device='cuda')
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return t.cpu().numpy()

    def timeit(fn, buf=None, iters=args.iters, warm=3, flush=True):
        evs = []
        for i in range(warm + iters):
            if flush:
                flush_l2_cache()
            torch.cuda._sleep(SLEEP)        # the host runs ahead; the barrier after it lines the ranks up (the spin counts SM cycles)
            if buf is not None and world > 1:
                buf.barrier(use_comm_stream=False)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            if i >= warm:
                evs.append((a, b))
        torch.cuda.synchronize()
        return reduce_max([a.elapsed_time(b) for a, b in evs])

    # ------------------------------------------------------------------ plain tcgen05 GEMM (single GPU view)
    if want('gemm'):
        from deepep_ascend_b200.ops import gemm as G
        for (M, N, K) in [(8192, 7168, 7168), (8192, 4096, 7168)]:
            a = torch.randn(M, K, device='cuda').bfloat16()
            b = torch.randn(N, K, device='cuda').bfloat16()
            t = timeit(lambda: G.gemm_nt(a, b), flush=False)
            t_ref = timeit(lambda: torch.matmul(a, b.t()), flush=False)
            emit(bench='gemm_bf16_tcgen05', M=M, N=N, K=K, ms=float(np.median(t)), tflops=2 * M * N * K / np.median(t) / 1e9,
                 cublas_ms=float(np.median(t_ref)), cublas_tflops=2 * M * N * K / np.median(t_ref) / 1e9)

    T, H, E, K = 8192, 7168, 256, 8
    # ------------------------------------------------------------------ dispatch / combine phase breakdown + variants
    if want('phases'):
        buf = ElasticBuffer(group, num_max_tokens_per_rank=T, hidden=H, num_topk=K, use_fp8_dispatch=True, num_gpu_timeout_secs=20)
        gen = torch.Generator().manual_seed(1234 + rank)
        x = torch.randn(T, H, generator=gen).bfloat16().cuda()
        w, idx = torch.softmax(torch.randn(T, E, generator=gen), -1).topk(K, -1)
        w, idx = w.cuda(), idx.cuda()
        st = {}

        def disp(sms, **kw):
            def f():
                st['h'] = buf.dispatch(x, idx, w, num_experts=E, num_sms=sms, do_cpu_sync=False, **kw)[3]
            return f
        disp(64)()
        torch.cuda.synchronize()
        rows = float(st['h'].psum_num_recv_tokens_per_scaleup_rank[-1])
        buf.enable_kernel_timing(True)

        def kernel_ms(name, fn, iters=args.iters):
            """median over steps of the per-step maximum over ranks of the kernel's own events"""
            buf.kernel_times_ms(name)
            timeit(fn, buf, iters=iters)
            return float(np.median(reduce_max(buf.kernel_times_ms(name)[-iters:])))
        for sms in [int(v) for v in args.phase_sms.split(',') if v]:
            for warps, stages in ((0, 0), (8, 3), (6, 4), (8, 2), (10, 2)):
                buf.set_dispatch_tuning(warps, stages)
                t = kernel_ms('dispatch', disp(sms))
                emit(bench='dispatch', num_sms=sms, warps=warps or 12, stages=stages or 2, ms=t, gbs=rows * 7488 / t / 1e6)
            for aligned in (True, False):
                buf.set_dispatch_tuning(0, 0, line_aligned_side=aligned)
                t = kernel_ms('dispatch', disp(sms))
                emit(bench='dispatch_side_layout', num_sms=sms, line_aligned_side=aligned, ms=t, gbs=rows * 7488 / t / 1e6)
            buf.set_dispatch_tuning(0, 0)
            buf.enable_profiling(True)
            for _ in range(3):
                if world > 1:
                    buf.barrier(use_comm_stream=False)
                disp(sms)()
                buf.combine(buf.get_combine_buffer(st['h']), st['h'], num_sms=sms)
                emit(bench='phase_times_us', num_sms=sms, **buf.phase_times())
            buf.enable_profiling(False)
            h0 = st['h']
            t3 = kernel_ms('dispatch', lambda: buf.dispatch(x, handle=h0, topk_weights=w, num_sms=sms))
            emit(bench='dispatch_cached_layout', num_sms=sms, ms=t3, gbs=rows * 7488 / t3 / 1e6)
            q = buf._C.per_token_cast_to_fp8(x, False, False)
            t4 = kernel_ms('dispatch', lambda: buf.dispatch((q[0], q[1]), idx, w, num_experts=E, num_sms=sms, do_cpu_sync=False))
            emit(bench='dispatch_prequantized_fp8', num_sms=sms, ms=t4, gbs=rows * 7488 / t4 / 1e6)
            t5 = kernel_ms('combine', lambda: buf.combine(buf.get_combine_buffer(st['h']), st['h'], num_sms=sms))
            emit(bench='combine', num_sms=sms, ms=t5, gbs=rows * 14336 / t5 / 1e6)
        buf.destroy()

    # ------------------------------------------------------------------ NCCL all_to_all_single baseline (same bytes)
    if want('nccl') and world > 1:
        from deepep_ascend_b200.utils import refs
        gen = torch.Generator().manual_seed(1234 + rank)
        x = torch.randn(T, H, generator=gen).bfloat16().cuda()
        w, idx = torch.softmax(torch.randn(T, E, generator=gen), -1).topk(K, -1)
        w, idx = w.cuda(), idx.cuda()
        q = torch.empty(T, H, device='cuda', dtype=torch.float8_e4m3fn)
        sf = torch.rand(T, H // 128, device='cuda')
        out = refs.dispatch_nccl((q, sf), idx, w, T, E, group)
        rows = float(out[0][0].shape[0])
        t = np.median(timeit(lambda: refs.dispatch_nccl((q, sf), idx, w, T, E, group)))
        emit(bench='nccl_all_to_all_dispatch_baseline', ms=float(t), gbs=rows * 7488 / t / 1e6, note='torch gather + 6 all_to_all_single calls')
        send = torch.empty(int(rows), H, device='cuda', dtype=torch.bfloat16)
        recv = torch.empty_like(send)
        splits = [int(rows) // world] * world
        splits[-1] += int(rows) - sum(splits)
        t = np.median(timeit(lambda: dist.all_to_all_single(recv, send, splits, splits, group=group)))
        emit(bench='nccl_all_to_all_single_bf16_rows', ms=float(t), gbs=rows * H * 2 / t / 1e6)

    # ------------------------------------------------------------------ low-latency decode in a CUDA graph
    if want('ll'):
        M, Tll = 128, 128
        extra = ElasticBuffer.get_low_latency_size_hint(M, H, world, E, K)
        buf = ElasticBuffer(group, num_max_tokens_per_rank=M, hidden=H, num_topk=K, extra_bytes=extra, num_gpu_timeout_secs=20)
        gen = torch.Generator().manual_seed(77 + rank)
        x = torch.randn(Tll, H, generator=gen).bfloat16().cuda()
        idx = torch.rand(Tll, E, generator=gen).topk(K, -1).indices.cuda()     # uniform random logits
        w = torch.rand(Tll, K, generator=gen).cuda()
        El = E // world
        y = torch.randn(El, world * M, H, device='cuda').bfloat16()
        cur = torch.cuda.current_stream()
        for sms, hooked in ((32, False), (64, False), (132, False), (132, True)):
            # hooked = the send and the receive phase are separate launches (no SM is held while data is in flight)
            def d():
                return buf.low_latency_dispatch(x, idx, M, E, use_fp8=True, return_recv_hook=hooked, num_sms=sms)
            def run_pair():
                recv, cnt, handle, _, hook = d()
                if hooked:
                    hook()
                out, _, hook2 = buf.low_latency_combine(y, idx, w, handle, return_recv_hook=hooked, num_sms=sms)
                if hooked:
                    hook2()
                return handle
            handle = run_pair()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier(group=group)
            # one graph holds a dispatch, another a combine, so that each can be timed by itself
            gd, gc = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                with torch.cuda.graph(gd, stream=side):
                    recv, cnt, handle, _, hook = d()
                    if hooked:
                        hook()
                with torch.cuda.graph(gc, stream=side):
                    out, _, hook2 = buf.low_latency_combine(y, idx, w, handle, return_recv_hook=hooked, num_sms=sms)
                    if hooked:
                        hook2()
            torch.cuda.synchronize()
            td, tc = [], []
            for i in range(5 + 100):
                torch.cuda._sleep(1_000_000)
                if world > 1:
                    buf.barrier(use_comm_stream=False)
                e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
                e[0].record()
                gd.replay()
                e[1].record()
                gc.replay()
                e[2].record()
                if i >= 5:
                    td.append((e[0], e[1]))
                    tc.append((e[1], e[2]))
            torch.cuda.synchronize()
            td = reduce_max([a.elapsed_time(b) * 1e3 for a, b in td])
            tc = reduce_max([a.elapsed_time(b) * 1e3 for a, b in tc])
            emit(bench='low_latency_cuda_graph', num_sms=sms, send_recv_split=hooked, tokens=Tll, dispatch_p50_us=float(np.percentile(td, 50)),
                 dispatch_p99_us=float(np.percentile(td, 99)), combine_p50_us=float(np.percentile(tc, 50)),
                 combine_p99_us=float(np.percentile(tc, 99)), reference='77 / 114 us (H800 + CX7 RDMA, published)')
            buf.check_status()
            if not hooked and sms == 132:
                # where the time goes: device timestamps of one eager call per kernel (us since kernel start, this rank)
                buf.enable_profiling(True)
                for _ in range(3):
                    if world > 1:
                        buf.barrier(use_comm_stream=False)
                    run_pair()
                pt = buf.phase_times()
                buf.enable_profiling(False)
                emit(bench='low_latency_phase_us', num_sms=sms, dispatch=pt['ll_dispatch'], combine=pt['ll_combine'])
        buf.destroy()

    # ------------------------------------------------------------------ fused MoE layer forward + backward
    if want('moe'):
        from deepep_ascend_b200.models.moe import FusedMoE
        Tm, I = args.moe_tokens, 2048
        bi, bw = min(5, args.iters), (2 if args.iters > 1 else 0)     # iterations / warm-up of every piece of the breakdown
        # 32 experts per rank, as at EP8 with 256 experts (a single GPU would otherwise hold all 256 and stream 22 GB of weights)
        Em = args.moe_experts or (E if world > 1 else 32)
        buf = ElasticBuffer(group, num_max_tokens_per_rank=Tm, hidden=H, num_topk=K, enable_expand=True, num_experts=Em,
                            expert_alignment=128, num_gpu_timeout_secs=30)
        layer = FusedMoE(buf, Em, H, I, init_std=0.02, num_sms=64)
        gen = torch.Generator().manual_seed(5 + rank)
        x = torch.randn(Tm, H, generator=gen).bfloat16().cuda().requires_grad_(True)
        w, idx = torch.softmax(torch.randn(Tm, Em, generator=gen), -1).topk(K, -1)
        w, idx = w.cuda().requires_grad_(True), idx.cuda()
        g = torch.randn(Tm, H, device='cuda').bfloat16()

        def fwd():
            return layer(x, idx, w)

        def fwd_bwd():
            layer.zero_grad(set_to_none=True)      # as a training loop does: gradients are assigned, not accumulated
            x.grad = w.grad = None
            layer(x, idx, w).backward(g)
        # breakdown of the forward pass
        from deepep_ascend_b200.ops import gemm as G
        st = {}

        def d_only():
            st['o'] = buf.dispatch(x.detach(), idx, w.detach(), num_experts=Em, do_expand=True, expert_alignment=G.BLOCK_M,
                                   fused_fp8_cast=True, num_sms=64)
        d_only()
        (rx, rsf), _, rw, hd, _ = st['o']
        tile_group, valid_row = G.expert_tile_groups(hd.psum_num_recv_tokens_per_expert, hd.num_rows)
        q13, s13, q2, s2 = layer.fp8_weights()
        t_disp = np.median(timeit(d_only, buf, iters=bi, warm=bw))
        hbuf = {}

        def g1():
            hbuf['h'] = G.grouped_gemm_nt(rx, q13, tile_group, sfa=rsf, sfb=s13)
        t_g1 = np.median(timeit(g1, None, iters=bi, warm=bw))

        def sw():
            hbuf['a'] = G.swiglu_quant(hbuf['h'])
        t_sw = np.median(timeit(sw, None, iters=bi, warm=bw))
        ybuf = buf.get_combine_buffer(hd)
        t_g2 = np.median(timeit(lambda: G.grouped_gemm_nt(hbuf['a'][0], q2, tile_group, out=ybuf, sfa=hbuf['a'][1], sfb=s2), None, iters=bi, warm=bw))
        t_comb = np.median(timeit(lambda: buf.combine(ybuf, hd, weighted=True, num_sms=64), buf, iters=bi, warm=bw))
        emit(bench='fused_moe_forward_breakdown_ms', rows=hd.num_rows, dispatch_expand_fp8=float(t_disp), gemm1_fp8=float(t_g1),
             swiglu_cast=float(t_sw), gemm2_fp8=float(t_g2), combine_weighted=float(t_comb),
             gemm1_tflops=2 * hd.num_rows * H * 2 * I / t_g1 / 1e9, gemm2_tflops=2 * hd.num_rows * H * I / t_g2 / 1e9)
        # the pieces that replace the expand-layout dispatch / combine when the expansion happens on the expert rank
        def d_loc():
            st['l'] = buf.dispatch(x.detach(), idx, w.detach(), num_experts=Em, do_expand=False, expert_alignment=G.BLOCK_M,
                                   fused_fp8_cast=True, num_sms=64)
        d_loc()
        t_dl = np.median(timeit(d_loc, buf, iters=bi, warm=bw))
        (rx_r, rsf_r), ridx, rw_r, hl, _ = st['l']
        rows_l = sum(hl.num_recv_tokens_per_expert_list)
        t_plan = np.median(timeit(lambda: G.local_expand_plan(ridx, hl.psum_num_recv_tokens_per_expert), None, iters=bi, warm=bw))
        pos, seg_end = G.local_expand_plan(ridx, hl.psum_num_recv_tokens_per_expert)
        t_copy = np.median(timeit(lambda: G.local_expand_copy(pos, rx_r, rows_l, sf=rsf_r, w=rw_r), None, iters=bi, warm=bw))
        w_e = G.local_expand_copy(pos, rx_r, rows_l, sf=rsf_r, w=rw_r)[2]
        y_exp = torch.randn(rows_l, H, device='cuda').bfloat16()
        t_red = np.median(timeit(lambda: G.local_reduce(pos, y_exp, w=w_e, out=buf.get_combine_buffer(hl)), None, iters=bi, warm=bw))
        t_cl = np.median(timeit(lambda: buf.combine(buf.get_combine_buffer(hl), hl, num_sms=64), buf, iters=bi, warm=bw))
        emit(bench='fused_moe_local_expand_breakdown_ms', received_rows=hl.num_rows, expert_rows=rows_l, dispatch_fp8=float(t_dl),
             plan=float(t_plan), expand_copy=float(t_copy), local_reduce=float(t_red), combine=float(t_cl))
        del y_exp, w_e
        # backward pieces, timed one by one on this rank's rows
        g_rows = torch.randn(hd.num_rows, H, device='cuda').bfloat16()
        rwc = rw.contiguous()
        seg_off = G.segment_offsets(hd.psum_num_recv_tokens_per_expert)
        w2_t, w13_t = layer.transposed_weights()
        bb = {}

        def prep():
            bb['dy_t'] = G.weighted_transpose(g_rows, rwc, valid_row)
        t_prep = np.median(timeit(prep, None, iters=bi, warm=bw))

        def dgrad2():
            bb['d_act'] = G.grouped_gemm_nt(g_rows, w2_t, tile_group)
        t_dg2 = np.median(timeit(dgrad2, None, iters=bi, warm=bw))

        def swb():
            bb['dh'], bb['dh_t'], bb['act_t'], bb['dot'] = G.swiglu_bwd(bb['d_act'], hbuf['h'], valid_row, row_weight=rwc)
        t_swb = np.median(timeit(swb, None, iters=bi, warm=bw))
        t_dg1 = np.median(timeit(lambda: G.grouped_gemm_nt(bb['dh'], w13_t, tile_group, out=ybuf), None, iters=bi, warm=bw))

        def xt():
            bb['x_t'] = G.dequant_transpose(rx, rsf, valid_row)
        t_xt = np.median(timeit(xt, None, iters=bi, warm=bw))
        t_wg2 = np.median(timeit(lambda: G.gemm_kgrouped(bb['dy_t'], bb['act_t'], seg_off), None, iters=bi, warm=bw))
        t_wg1 = np.median(timeit(lambda: G.gemm_kgrouped(bb['dh_t'], bb['x_t'], seg_off), None, iters=bi, warm=bw))
        emit(bench='fused_moe_backward_breakdown_ms', rows=hd.num_rows, weighted_transpose=float(t_prep), dgrad_down_bf16=float(t_dg2),
             swiglu_bwd=float(t_swb), dgrad_up_bf16=float(t_dg1), dequant_transpose=float(t_xt), wgrad_down=float(t_wg2),
             wgrad_up=float(t_wg1), dgrad_down_tflops=2 * hd.num_rows * H * I / t_dg2 / 1e9,
             dgrad_up_tflops=2 * hd.num_rows * H * 2 * I / t_dg1 / 1e9, wgrad_down_tflops=2 * hd.num_rows * H * I / t_wg2 / 1e9,
             wgrad_up_tflops=2 * hd.num_rows * H * 2 * I / t_wg1 / 1e9)
        del bb, g_rows
        tf = np.median(timeit(fwd, buf, iters=bi, warm=bw))
        tfb_all = timeit(fwd_bwd, buf, iters=bi, warm=bw)
        tfb = np.median(tfb_all)
        rows = float(idx.numel())
        flops_fwd = rows * (2 * H * 2 * I + 2 * I * H)
        emit(bench='fused_moe_layer', tokens_per_rank=Tm, hidden=H, intermediate=I, experts_per_rank=Em // world, fwd_ms=float(tf), fwd_bwd_ms=float(tfb), fwd_bwd_ms_all=[round(float(v), 3) for v in tfb_all],
             fwd_expert_tflops_per_gpu=flops_fwd / tf / 1e9, note='includes the host sync of dispatch (exact sizes)')
        # the same layer with the buffer's expand layout: one row per (token, expert) over NVLink instead of one per (token, rank)
        layer.local_expand = False
        tf_x = np.median(timeit(fwd, buf, iters=bi, warm=bw))
        tfb_x = np.median(timeit(fwd_bwd, buf, iters=bi, warm=bw))
        layer.local_expand = True
        emit(bench='fused_moe_layer_expand_over_nvlink', fwd_ms=float(tf_x), fwd_bwd_ms=float(tfb_x))
        # the same layer with the data-gradient GEMMs (and the dispatch of the output gradient) in e4m3
        layer.fp8_backward = True
        tfb8 = np.median(timeit(fwd_bwd, buf, iters=bi, warm=bw))
        layer.fp8_backward = False
        emit(bench='fused_moe_layer_fp8_backward', fwd_bwd_ms=float(tfb8), note='dgrad GEMMs and gradient dispatch in e4m3; weight gradients bf16')
        # the same layer as a pipeline of chunks: communication of one chunk under the GEMMs of its neighbours
        with torch.no_grad():
            for chunks, comm_sms in ((1, 64), (2, 24), (4, 24), (4, 16), (8, 24)):
                layer.num_chunks, layer.num_sms = chunks, comm_sms
                t = np.median(timeit(lambda: layer(x, idx, w), buf, iters=bi, warm=bw))
                emit(bench='fused_moe_forward_pipelined', chunks=chunks, comm_sms=comm_sms, fwd_ms=float(t),
                     fwd_expert_tflops_per_gpu=flops_fwd / t / 1e9)
        layer.num_chunks, layer.num_sms = 4, 24
        tfb4 = np.median(timeit(fwd_bwd, buf, iters=bi, warm=bw))
        emit(bench='fused_moe_layer_pipelined_forward', chunks=4, comm_sms=24, fwd_bwd_ms=float(tfb4))
        buf.check_status()
        buf.destroy()

    # ------------------------------------------------------------------ Zipf-skewed routing
    if want('zipf'):
        Tz, Hz, Ez, Kz = 4096, 4096, 64, 6
        buf = ElasticBuffer(group, num_max_tokens_per_rank=Tz, hidden=Hz, num_topk=Kz, num_gpu_timeout_secs=20)
        x = torch.randn(Tz, Hz, device='cuda').bfloat16()
        scores = gate.get_zipf_scores(Tz, Ez, 1.2, device='cuda')
        w, idx = torch.softmax(scores, -1).topk(Kz, -1)
        st = {}

        def dz():
            st['h'] = buf.dispatch(x, idx, w.contiguous(), num_experts=Ez, num_sms=64, do_cpu_sync=False)[3]
        dz()
        torch.cuda.synchronize()
        rows = torch.tensor([float(st['h'].psum_num_recv_tokens_per_scaleup_rank[-1])], device='cuda')
        rows_max = rows.clone()
        if world > 1:
            dist.all_reduce(rows_max, op=dist.ReduceOp.MAX, group=group)
        td = np.median(timeit(dz, buf))
        tc = np.median(timeit(lambda: buf.combine(buf.get_combine_buffer(st['h']), st['h'], num_sms=64), buf))
        row_d, row_c = Hz * 2 + Kz * 12, Hz * 2 + Kz * 4
        emit(bench='zipf_routing_bf16', s=1.2, experts=Ez, topk=Kz, hidden=Hz, hottest_rank_rows=float(rows_max), dispatch_ms=float(td),
             combine_ms=float(tc), dispatch_gbs_hottest=float(rows_max) * row_d / td / 1e6, combine_gbs_hottest=float(rows_max) * row_c / tc / 1e6)
        buf.destroy()

    # ------------------------------------------------------------------ fused tensor-parallel GEMMs
    if want('tp') and world > 1:
        from deepep_ascend_b200.parallel.tp import TensorParallelGemm
        M, Kt, N = 8192, 7168, 7168
        buf = ElasticBuffer(group, num_max_tokens_per_rank=16, hidden=256, num_topk=2, extra_bytes=TensorParallelGemm.size_hint(M, Kt, N),
                            num_gpu_timeout_secs=20)
        tp = TensorParallelGemm(buf, M, Kt, N)
        xs = torch.randn(M // world, Kt, device='cuda').bfloat16()
        w_col = torch.randn(N // world, Kt, device='cuda').bfloat16()          # column-parallel weight
        auto_copiers = tp._copiers(N // world)
        for copiers in sorted({16, 32, 48, auto_copiers}):
            tp.num_copy_ctas = copiers
            t = np.median(timeit(lambda: tp.ag_gemm(xs, w_col), buf, iters=10))
            emit(bench='ag_gemm_fused', M=M, K=Kt, N_local=N // world, copier_ctas=copiers, default=copiers == auto_copiers, ms=float(t),
                 tflops_per_gpu=2 * M * Kt * (N // world) / t / 1e9, nvlink_gbs_in=(world - 1) / world * M * Kt * 2 / t / 1e6)
        tp.num_copy_ctas = 0
        xk = torch.randn(M, Kt // world, device='cuda').bfloat16()             # row-parallel: K is sharded
        w_row = torch.randn(N, Kt // world, device='cuda').bfloat16()
        t = np.median(timeit(lambda: tp.gemm_rs(xk, w_row), buf, iters=10))
        emit(bench='gemm_rs_fused', M=M, K_local=Kt // world, N=N, ms=float(t), tflops_per_gpu=2 * M * (Kt // world) * N / t / 1e9,
             nvlink_gbs_out=(world - 1) / world * M * N * 2 / t / 1e6)
        # unfused baseline: NCCL all-gather then cuBLAS, cuBLAS then NCCL reduce-scatter
        full = torch.empty(M, Kt, device='cuda', dtype=torch.bfloat16)
        t = np.median(timeit(lambda: (dist.all_gather_into_tensor(full, xs, group=group), torch.matmul(full, w_col.t())), buf, iters=10))
        emit(bench='ag_gemm_nccl_cublas_baseline', ms=float(t))
        outrs = torch.empty(M // world, N, device='cuda', dtype=torch.bfloat16)
        t = np.median(timeit(lambda: dist.reduce_scatter_tensor(outrs, torch.matmul(xk, w_row.t()), group=group), buf, iters=10))
        emit(bench='gemm_rs_nccl_cublas_baseline', ms=float(t))
        buf.check_status()
        emit(bench='gemm_error_flag', value=buf._C.gemm_error(lr))
        buf.destroy()

    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
