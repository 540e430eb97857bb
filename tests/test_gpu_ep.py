"""Dispatch / combine kernels on one GPU with several virtual ranks (one cooperative launch per call),
checked bitwise against the all-ranks oracle in plain PyTorch."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _make_inputs(R, T, H, E, K, seed=0, drop=0.05):
    g = torch.Generator(device='cpu').manual_seed(seed)
    xs, idxs, ws = [], [], []
    for r in range(R):
        t = max(0, T - 3 * r)
        xs.append(torch.randn(t, H, generator=g).bfloat16().cuda())
        idx = torch.rand(t, E, generator=g).topk(K, dim=-1).indices
        idx[torch.rand(idx.shape, generator=g) < drop] = -1
        idxs.append(idx.cuda())
        ws.append(torch.rand(t, K, generator=g).cuda())
    return xs, idxs, ws


def _check_dispatch(outs, expect, fp8, do_expand):
    for r, (o, e) in enumerate(zip(outs, expect)):
        x, idx, w, handle = o
        gl = e['layout']
        rows = gl.num_expanded_tokens if do_expand else gl.num_recv_tokens
        assert handle.num_rows == rows, (r, handle.num_rows, rows)
        valid = e['valid']
        xv, sf = x if fp8 else (x, None)
        assert xv.shape[0] == rows
        assert torch.equal(xv.cpu().view(torch.uint8)[valid], e['x'].view(torch.uint8)[valid]), f'rank {r} payload'
        if fp8:
            assert torch.equal(sf.cpu()[valid], e['sf'][valid]), f'rank {r} scales'
        if not do_expand:
            assert torch.equal(idx.cpu(), e['idx'])
        assert torch.equal(w.cpu()[valid], e['w'][valid])
        assert torch.equal(handle.recv_src_metadata.cpu()[valid], e['meta'][valid])
        assert torch.equal(handle.dst_buffer_slot_idx.cpu(), gl.lane_src)
        assert torch.equal(handle.plan.cpu(), gl.plan)
        assert torch.equal(handle.psum_num_recv_tokens_per_scaleup_rank.cpu(), gl.psum_recv_per_rank)
        assert torch.equal(handle.psum_num_recv_tokens_per_expert.cpu(), gl.psum_recv_per_expert)
        assert torch.equal(handle.num_unaligned_recv_tokens_per_expert.cpu(), gl.recv_per_expert)


@pytest.mark.parametrize('R,T,H,E,K', [(2, 128, 256, 8, 2), (4, 200, 1024, 32, 4), (8, 96, 7168, 256, 8), (1, 64, 512, 4, 2),
                                       (8, 77, 2048, 64, 6), (8, 16, 128, 8, 2)])
@pytest.mark.parametrize('mode', ['bf16', 'fp8_in', 'quant'])
@pytest.mark.parametrize('do_expand', [False, True])
def test_dispatch_combine(R, T, H, E, K, mode, do_expand):
    _run_dispatch_combine(R, T, H, E, K, mode, do_expand)


@pytest.mark.parametrize('R,T,H,E,K', [(4, 200, 1024, 32, 4), (8, 96, 7168, 256, 8), (8, 77, 2048, 64, 6)])
@pytest.mark.parametrize('mode', ['bf16', 'fp8_in', 'quant'])
def test_dispatch_combine_line_aligned_side_records(R, T, H, E, K, mode):
    """The same checks with ``set_dispatch_tuning(line_aligned_side=True)``: scale rows and tail records sit on 128-byte lines
    at the receiver, so ``recv_sf`` / ``recv_topk_idx`` / ``recv_topk_weights`` are strided views with the same contents."""
    _run_dispatch_combine(R, T, H, E, K, mode, False, aligned=True)


def _run_dispatch_combine(R, T, H, E, K, mode, do_expand, aligned=False):
    from deepep_ascend_b200.backends.emulated import EmulatedWorld
    from deepep_ascend_b200.utils import refs
    from deepep_ascend_b200.utils.math import per_token_cast_to_fp8
    A = 8 if do_expand else 1
    world = EmulatedWorld(R, num_max_tokens_per_rank=T, hidden=H, num_topk=K, use_fp8_dispatch=(mode != 'bf16'),
                          enable_expand=do_expand, num_experts=E, expert_alignment=A)
    try:
        if aligned:
            for b in world.buffers:
                b.set_dispatch_tuning(0, 0, line_aligned_side=True)
        xs, idxs, ws = _make_inputs(R, T, H, E, K, seed=R + K)
        fp8 = mode != 'bf16'
        if fp8:
            q = [per_token_cast_to_fp8(x.cpu()) for x in xs]
            ref_x, ref_sf = [a for a, _ in q], [b for _, b in q]
        else:
            ref_x, ref_sf = xs, None
        if mode == 'fp8_in':
            ins = [(a.cuda(), b.cuda()) for a, b in zip(ref_x, ref_sf)]
        else:
            ins = xs
        stats = [torch.zeros(E // R, dtype=torch.int32, device='cuda') for _ in range(R)]
        outs = world.dispatch(ins, idxs, ws, E, num_sms=6, expert_alignment=A, do_expand=do_expand, stats=stats)
        torch.cuda.synchronize()
        for b in world.buffers:
            b.check_status()
        expect = refs.dispatch_all(ref_x, ref_sf, idxs, ws, E, T, do_expand, A)
        _check_dispatch(outs, expect, fp8, do_expand)
        for r in range(R):
            assert torch.equal(stats[r].cpu(), expect[r]['layout'].recv_per_expert)

        # combine: random expert outputs, two biases, weights carried back
        g = torch.Generator(device='cpu').manual_seed(5)
        ys = [torch.randn(o[3].num_rows, H, generator=g).bfloat16().cuda() for o in outs]
        b0 = [torch.randn(x.shape[0], H, generator=g).bfloat16().cuda() for x in xs]
        b1 = [torch.randn(x.shape[0], H, generator=g).bfloat16().cuda() for x in xs]
        handles = [o[3] for o in outs]
        recv_ws = [o[2] for o in outs]
        res = world.combine(ys, handles, topk_weights=recv_ws, bias0=b0, bias1=b1, num_sms=5)
        torch.cuda.synchronize()
        for b in world.buffers:
            b.check_status()
        want = refs.combine_all(ys, [e['layout'] for e in expect], H, [b.cpu() for b in b0], [b.cpu() for b in b1])
        for r in range(R):
            assert torch.equal(res[r][0].cpu().view(torch.int16), want[r].view(torch.int16)), f'rank {r} combine'
            valid = (idxs[r] >= 0).cpu()
            assert torch.equal(res[r][1].cpu()[valid], ws[r].cpu()[valid]), 'weights must come back unchanged'

        # cached re-dispatch lands in the next receive slot with identical contents
        outs2 = world.dispatch(ins, [None] * R, ws, E, num_sms=6, handles=handles)
        torch.cuda.synchronize()
        for r in range(R):
            a = outs2[r][0][0] if fp8 else outs2[r][0]
            valid = expect[r]['valid']
            assert torch.equal(a.cpu().view(torch.uint8)[valid], expect[r]['x'].view(torch.uint8)[valid])
        if do_expand:
            res = world.combine(ys, handles, weighted=True, num_sms=5)
            torch.cuda.synchronize()
            want = refs.combine_all(ys, [e['layout'] for e in expect], H, mul_weights=[w.cpu() for w in ws])
            for r in range(R):
                torch.testing.assert_close(res[r][0].cpu().float(), want[r].float(), atol=2e-2, rtol=2e-2)
    finally:
        world.destroy()


def test_no_cpu_sync_and_col_major_sf():
    from deepep_ascend_b200.backends.emulated import EmulatedWorld
    from deepep_ascend_b200.utils import refs
    from deepep_ascend_b200.utils.math import per_token_cast_to_fp8
    R, T, H, E, K = 4, 64, 1024, 16, 4
    world = EmulatedWorld(R, num_max_tokens_per_rank=T, hidden=H, num_topk=K, use_fp8_dispatch=True)
    try:
        xs, idxs, ws = _make_inputs(R, T, H, E, K, seed=3)
        outs = world.dispatch(xs, idxs, ws, E, num_sms=4, do_cpu_sync=False, use_tma_aligned_col_major_sf=True)
        torch.cuda.synchronize()
        q = [per_token_cast_to_fp8(x.cpu()) for x in xs]
        expect = refs.dispatch_all([a for a, _ in q], [b for _, b in q], idxs, ws, E, T)
        for r in range(R):
            (x, sf), idx, w, handle = outs[r]
            n = int(handle.psum_num_recv_tokens_per_scaleup_rank[-1])
            assert n == expect[r]['layout'].num_recv_tokens and x.shape[0] == world.buffers[r].regions.capacity_rows
            assert sf.stride(0) == 1 and sf.stride(1) % 4 == 0
            assert torch.equal(x[:n].cpu().view(torch.uint8), expect[r]['x'].view(torch.uint8))
            assert torch.equal(sf[:n].cpu(), expect[r]['sf'])
    finally:
        world.destroy()
