"""Stand-alone kernels and the failure path on one GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_native_extension_is_loaded():
    from deepep_ascend_b200 import _native
    C = _native.load()
    assert C.get_platform() == 'cuda-sm100a'


@pytest.mark.parametrize('dtype', [torch.int64, torch.int32])
def test_get_dispatch_layout(dtype):
    from deepep_ascend_b200 import _native
    from deepep_ascend_b200.ops import layout_ref
    C = _native.load()
    idx = torch.rand(777, 64).topk(6, dim=-1).indices.to(dtype)
    idx[torch.rand(idx.shape) < 0.1] = -1
    per_rank, per_expert, in_rank = C.get_dispatch_layout(idx.cuda(), 64, 8)
    r0, r1, r2 = layout_ref.get_dispatch_layout_ref(idx, 64, 8)
    assert torch.equal(per_rank.cpu(), r0) and torch.equal(per_expert.cpu(), r1) and torch.equal(in_rank.cpu(), r2)


@pytest.mark.parametrize('H', [128, 256, 2048, 7168, 400])
@pytest.mark.parametrize('mode', ['plain', 'round', 'ue8m0'])
def test_fp8_cast_kernel(H, mode):
    from deepep_ascend_b200 import _native
    from deepep_ascend_b200.utils.math import per_token_cast_to_fp8
    C = _native.load()
    x = (torch.randn(333, H) * torch.rand(333, 1) * 4).bfloat16()
    x[5] = 0
    q, sf = C.per_token_cast_to_fp8(x.cuda(), mode != 'plain', mode == 'ue8m0')
    rq, rsf = per_token_cast_to_fp8(x, round_scale=(mode != 'plain'), use_ue8m0=(mode == 'ue8m0'))
    assert torch.equal(sf.cpu(), rsf)
    assert torch.equal(q.cpu().view(torch.uint8), rq.view(torch.uint8))


def test_barrier_and_bounded_wait_reports_status():
    from deepep_ascend_b200.backends.emulated import EmulatedWorld
    world = EmulatedWorld(4, num_max_tokens_per_rank=16, hidden=256, num_topk=2, num_gpu_timeout_secs=0.2)
    try:
        for _ in range(3):
            world.barrier()
        torch.cuda.synchronize()
        for b in world.buffers:
            b.check_status()
            assert b.state == 'idle'
        # a wait on a flag that nothing sets must end by itself with a status record, not a trap or a hang
        C = world._C
        C.ElasticBuffer.wait_flag_test_group(world.cores, 7)
        torch.cuda.synchronize()
        for r, b in enumerate(world.buffers):
            code, phase, peer, expected, observed, rank = b.core.read_status()
            assert (code, expected, observed, rank) == (1, 7, 0, r)
            with pytest.raises(RuntimeError, match='timed out'):
                b.check_status()
            assert b.state == 'poisoned'
            with pytest.raises(RuntimeError, match='poisoned'):
                b.core.barrier()
        # the context is still usable
        assert float(torch.ones(4, device='cuda').sum()) == 4.0
    finally:
        world.destroy()


def test_poison_fill_no_stray_writes():
    """All MoE regions of every rank are filled with 0xFF before a dispatch; afterwards only the rows the layout assigns have
    changed: the tail of the used receive slot and the whole unused slot still hold the poison."""
    from deepep_ascend_b200.backends.emulated import EmulatedWorld
    R, T, H, E, K = 4, 64, 512, 16, 4
    world = EmulatedWorld(R, num_max_tokens_per_rank=T, hidden=H, num_topk=K, use_fp8_dispatch=True, num_experts=E)
    try:
        ws_bytes = world.buffers[0]._C.get_workspace_bytes()
        for b in world.buffers:
            b.core.view(ws_bytes, [b.regions.moe_bytes - ws_bytes], [1], torch.uint8).fill_(0xFF)
        g = torch.Generator().manual_seed(3)
        xs = [torch.randn(T, H, generator=g).bfloat16().cuda() for _ in range(R)]
        idxs = [torch.rand(T, E, generator=g).topk(K, -1).indices.cuda() for _ in range(R)]
        ws = [torch.rand(T, K, generator=g).cuda() for _ in range(R)]
        outs = world.dispatch(xs, idxs, ws, E, num_sms=6)
        torch.cuda.synchronize()
        for b, (x, idx, w, handle) in zip(world.buffers, outs):
            b.check_status()
            q, sf = x
            rows, cap, reg = handle.num_rows, b.regions.capacity_rows, b.regions
            assert 0 < rows < cap
            used, other = reg.slot(handle.recv_slot), reg.slot((handle.recv_slot + 1) % reg.num_recv_slots)
            x_tail = b.core.view(used.x + rows * H, [cap * reg.x_row_bytes - rows * H], [1], torch.uint8)
            assert bool((x_tail == 0xFF).all()), 'payload written behind the last received row'
            assert sf.is_contiguous()
            pitch = idx.stride(0) * idx.element_size()
            sf_tail = b.core.view(used.sf + rows * sf.shape[1] * 4, [(cap - rows) * sf.shape[1] * 4], [1], torch.uint8)
            assert bool((sf_tail == 0xFF).all()), 'scales written behind the last received row'
            rec_tail = b.core.view(used.tail + rows * pitch, [(cap - rows) * pitch], [1], torch.uint8)
            assert bool((rec_tail == 0xFF).all()), 'tail record written behind the last received row'
            assert bool((b.core.view(other.x, [cap * reg.x_row_bytes], [1], torch.uint8) == 0xFF).all()), 'the unused slot was touched'
            # every received row was written: e4m3 never produces the byte pattern 0xFF for finite inputs in all 512 channels
            assert not bool((q.view(torch.uint8) == 0xFF).all(dim=1).any())
            assert bool(torch.isfinite(sf).all()) and bool((idx >= -1).all())
    finally:
        world.destroy()
