"""Low-latency dispatch / combine on one GPU with virtual ranks, against a plain PyTorch statement of the result."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(R, T, H, E, K, seed):
    g = torch.Generator().manual_seed(seed)
    xs = [(torch.randn(T - r, H, generator=g) * (1 + r)).bfloat16().cuda() for r in range(R)]
    idxs = []
    for r in range(R):
        idx = torch.rand(T - r, E, generator=g).topk(K, dim=-1).indices
        idx[torch.rand(idx.shape, generator=g) < 0.1] = -1
        idxs.append(idx.cuda())
    ws = [torch.rand(T - r, K, generator=g).cuda() for r in range(R)]
    return xs, idxs, ws


@pytest.mark.parametrize('R,T,H,E,K', [(2, 16, 256, 8, 2), (4, 33, 2048, 32, 4), (8, 32, 7168, 64, 8)])
@pytest.mark.parametrize('mode', ['bf16', 'fp8', 'fp8_round', 'ue8m0'])
@pytest.mark.parametrize('split', [False, True])
def test_low_latency_roundtrip(R, T, H, E, K, mode, split):
    from deepep_ascend_b200.backends.emulated import EmulatedWorld
    from deepep_ascend_b200.buffers.elastic import ElasticBuffer
    from deepep_ascend_b200.utils.math import per_token_cast_back, per_token_cast_to_fp8
    M = T + 3
    extra = ElasticBuffer.get_low_latency_size_hint(M, H, R, E, K)
    world = EmulatedWorld(R, num_max_tokens_per_rank=M, hidden=H, num_topk=K, extra_bytes=extra, num_gpu_timeout_secs=5)
    try:
        El = E // R
        for it in range(3):     # several calls: both buffer sets and the epoch tags get exercised
            xs, idxs, ws = _inputs(R, T, H, E, K, seed=it)
            use_fp8 = mode != 'bf16'
            stats = [torch.zeros(El, dtype=torch.int32, device='cuda') for _ in range(R)]
            outs = world.low_latency_dispatch(xs, idxs, M, E, use_fp8=use_fp8, round_scale=(mode == 'fp8_round'),
                                              use_ue8m0=(mode == 'ue8m0'), stats=stats, split_phases=split)
            torch.cuda.synchronize()
            for b in world.buffers:
                b.check_status()
            if use_fp8:
                ref = [per_token_cast_to_fp8(x.cpu(), round_scale=(mode == 'fp8_round'), use_ue8m0=(mode == 'ue8m0')) for x in xs]
            ys = []
            for d in range(R):
                recv, count, handle = outs[d]
                src_info, layout_range = handle[0].cpu(), handle[1].cpu()
                rx, rsf = (recv[0].cpu(), recv[1].cpu()) if use_fp8 else (recv.cpu(), None)
                y = torch.zeros(El, R * M, H, dtype=torch.bfloat16)
                for j in range(El):
                    e = d * El + j
                    total = 0
                    for s in range(R):
                        n, begin = int(layout_range[j, s]) & 0xffffffff, int(layout_range[j, s]) >> 32
                        want = sorted((idxs[s].cpu() == e).any(dim=1).nonzero().flatten().tolist())
                        info = src_info[j, begin:begin + n]
                        got_t, got_k = (info & 0xfffff).tolist(), (info >> 20).tolist()
                        assert sorted(got_t) == want, (d, j, s)
                        assert begin == total
                        total += n
                        for i, (t, k) in enumerate(zip(got_t, got_k)):
                            assert int(idxs[s][t, k]) == e
                            row = begin + i
                            if use_fp8:
                                assert torch.equal(rx[j, row].view(torch.uint8), ref[s][0][t].view(torch.uint8))
                                assert torch.equal(rsf[j, row], ref[s][1][t])
                                val = per_token_cast_back(ref[s][0][t:t + 1], ref[s][1][t:t + 1])[0]
                            else:
                                assert torch.equal(rx[j, row], xs[s][t].cpu())
                                val = xs[s][t].cpu()
                            y[j, row] = (val.float() * (1 + 0.25 * (e % 3))).bfloat16()
                    assert int(count[j]) == total and int(stats[d][j]) == total
                ys.append(y.cuda())
            res = world.low_latency_combine(ys, idxs, ws, [o[2] for o in outs], split_phases=split)
            torch.cuda.synchronize()
            for b in world.buffers:
                b.check_status()
            for s in range(R):
                x = xs[s].cpu()
                if use_fp8:
                    x = per_token_cast_back(*ref[s])
                idx, w = idxs[s].cpu(), ws[s].cpu()
                want = torch.zeros(x.shape[0], H)
                for k in range(K):
                    m = idx[:, k] >= 0
                    yk = (x[m].float() * (1 + 0.25 * (idx[m, k] % 3)).unsqueeze(1)).bfloat16().float()
                    want[m] += w[m, k].unsqueeze(1) * yk
                torch.testing.assert_close(res[s].cpu().float(), want.bfloat16().float(), atol=3e-2, rtol=2e-2)
    finally:
        world.destroy()


@pytest.mark.parametrize('R,T,H,E,K', [(2, 16, 256, 8, 2), (4, 33, 2048, 32, 4), (8, 32, 7168, 64, 8)])
@pytest.mark.parametrize('split', [False, True])
def test_low_latency_combine_logfmt(R, T, H, E, K, split):
    """Combine with LogFMT-10 rows on the wire: the result is the weighted sum of the CODED rows (stated in plain PyTorch by
    ``logfmt10_roundtrip``) and stays within the accuracy the reference asks of this mode (calc_diff against the exact
    sum, tests/legacy/test_low_latency.py:178-181).  Zero rows and rows of one repeated value are coded exactly."""
    from deepep_ascend_b200.backends.emulated import EmulatedWorld
    from deepep_ascend_b200.buffers.elastic import ElasticBuffer
    from deepep_ascend_b200.utils.math import calc_diff, logfmt10_roundtrip
    M = T + 1
    extra = ElasticBuffer.get_low_latency_size_hint(M, H, R, E, K)
    world = EmulatedWorld(R, num_max_tokens_per_rank=M, hidden=H, num_topk=K, extra_bytes=extra, num_gpu_timeout_secs=5)
    try:
        for it in range(3):
            xs, idxs, ws = _inputs(R, T, H, E, K, seed=40 + it)
            for x in xs:
                x[0] = 0                 # an all-zero row
                x[1, :128] = -1.5        # a group with a single magnitude
            outs = world.low_latency_dispatch(xs, idxs, M, E, use_fp8=False, split_phases=split)
            res = world.low_latency_combine([o[0] for o in outs], idxs, ws, [o[2] for o in outs], split_phases=split, use_logfmt=True)
            torch.cuda.synchronize()
            for r in range(R):
                world.buffers[r].check_status()
                wsum = (ws[r].cpu() * (idxs[r].cpu() >= 0)).sum(dim=1, keepdim=True)
                coded = logfmt10_roundtrip(xs[r].cpu()) * wsum
                exact = xs[r].cpu().float() * wsum
                got = res[r].cpu().float()
                assert bool(torch.isfinite(got).all())
                assert calc_diff(got, exact) < 2e-5, calc_diff(got, exact)
                torch.testing.assert_close(got, coded, atol=3e-2, rtol=3e-2)
                assert bool((got[0] == 0).all())
                torch.testing.assert_close(got[1, :128], (-1.5 * wsum[1]).expand(128).bfloat16().float(), atol=0, rtol=1e-2)
    finally:
        world.destroy()
