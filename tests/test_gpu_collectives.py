"""All-gather / reduce-scatter sessions and Engram fetch on one GPU with virtual ranks."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_all_gather_reduce_scatter_sessions():
    from deepep_ascend_b200.backends.emulated import EmulatedWorld
    R = 4
    world = EmulatedWorld(R, num_max_tokens_per_rank=16, hidden=256, num_topk=2, extra_bytes=64 << 20)
    try:
        world.agrs_set_config(32 << 20)
        for session in range(2):
            world.create_agrs_session()
            for shape, dtype in [((1000, 33), torch.bfloat16), ((7,), torch.float32), ((128, 1024), torch.bfloat16)]:
                xs = [torch.randn(*shape, device='cuda').to(dtype) * (r + 1) for r in range(R)]
                outs = world.all_gather(xs)
                torch.cuda.synchronize()
                want = torch.stack(xs)
                for r in range(R):
                    assert torch.equal(outs[r], want)
            ins = [torch.randn(R, 513, 40, device='cuda').bfloat16() for _ in range(R)]
            outs = world.reduce_scatter(ins)
            torch.cuda.synchronize()
            for r in range(R):
                acc = torch.zeros(513, 40, device='cuda')
                for s in range(R):
                    acc += ins[s][r].float()
                assert torch.equal(outs[r], acc.bfloat16())
            world.destroy_agrs_session()
        for b in world.buffers:
            b.check_status()
    finally:
        world.destroy()


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float8_e4m3fn])
@pytest.mark.parametrize('in_cpu_segment', [False, True])
def test_engram_fetch(dtype, in_cpu_segment):
    """Entries are pulled from their owners' tables (device region, or the CPU segment behind the buffer); with a
    replicated scale table the scales of every fetched entry come back too, row- or column-major."""
    from deepep_ascend_b200.backends.emulated import EmulatedWorld
    R, N, H = 4, 300, 512
    fp8 = dtype == torch.float8_e4m3fn
    world = EmulatedWorld(R, num_max_tokens_per_rank=16, hidden=256, num_topk=2, extra_bytes=16 << 20,
                          num_cpu_bytes=(1 << 20) if in_cpu_segment else 0)
    try:
        tables = [(torch.randn(N, H, device='cuda') * (r + 1)).to(dtype) for r in range(R)]
        packs = H // 128
        sf_table = torch.rand(R * N, packs, device='cuda') if fp8 else None
        world.engram_write(tables, [sf_table] * R if fp8 else None)
        assert all(b._engram['cpu'] == in_cpu_segment for b in world.buffers)
        everything = torch.cat([t.view(torch.uint8) for t in tables])
        idx = [torch.randint(0, R * N, (37 + r, 3), device='cuda', dtype=torch.int32) for r in range(R)]
        for col_major in ([False, True] if fp8 else [False]):
            outs = world.engram_fetch(idx, use_tma_aligned_col_major_sf=col_major)
            torch.cuda.synchronize()
            for r in range(R):
                fetched, fetched_sf = outs[r]
                want = everything[idx[r].long().view(-1)].view(idx[r].shape[0], -1)
                assert torch.equal(fetched.view(torch.uint8), want)
                if fp8:
                    T = idx[r].shape[0]
                    assert fetched_sf.shape == (T, 3 * packs)
                    assert fetched_sf.stride() == ((1, (T + 3) // 4 * 4) if col_major else (3 * packs, 1))
                    assert torch.equal(fetched_sf, sf_table[idx[r].long().view(-1)].view(T, 3 * packs))
                else:
                    assert fetched_sf is None
                world.buffers[r].check_status()
    finally:
        world.destroy()
