"""Host-only checks of the deterministic layout definition against brute-force Python loops."""
import pytest
import torch

from deepep_ascend_b200.ops import layout_ref
from deepep_ascend_b200.utils import gate, refs


def brute_force(idxs, E, R, do_expand, A):
    El = E // R
    rows = [dict() for _ in range(R)]     # dest -> {(src, t, k): row}
    if not do_expand:
        for d in range(R):
            n = 0
            for s in range(R):
                for t in range(idxs[s].shape[0]):
                    ks = [k for k in range(idxs[s].shape[1]) if idxs[s][t, k] >= 0 and idxs[s][t, k] // El == d]
                    if ks:
                        rows[d][(s, t)] = n
                        n += 1
    else:
        for d in range(R):
            end = 0
            for j in range(El):
                start = (end + A - 1) // A * A
                n = start
                for s in range(R):
                    for t in range(idxs[s].shape[0]):
                        for k in range(idxs[s].shape[1]):
                            if idxs[s][t, k] == d * El + j:
                                rows[d][(s, t, k)] = n
                                n += 1
                end = n
    return rows


@pytest.mark.parametrize('R,E,K,T', [(2, 8, 2, 37), (4, 16, 3, 50), (8, 64, 6, 40), (1, 4, 2, 9)])
@pytest.mark.parametrize('do_expand', [False, True])
def test_layout_matches_brute_force(R, E, K, T, do_expand):
    torch.manual_seed(R * 100 + K)
    A = 4 if do_expand else 1
    idxs = []
    for r in range(R):
        scores = gate.get_balanced_scores(T + r, E, device='cpu')
        idx = scores.topk(K, dim=-1).indices
        idx[torch.rand(idx.shape) < 0.1] = -1
        idxs.append(idx)
    xs = [torch.randn(i.shape[0], 16).bfloat16() for i in idxs]
    ws = [torch.rand(i.shape[0], K) for i in idxs]
    outs = refs.dispatch_all(xs, None, idxs, ws, E, 64, do_expand, A)
    expect = brute_force(idxs, E, R, do_expand, A)
    El = E // R
    for s in range(R):
        rank, row = layout_ref.unpack_lane(outs[s]['layout'].lane_src)
        for t in range(idxs[s].shape[0]):
            for k in range(K):
                e = int(idxs[s][t, k])
                if e < 0:
                    assert rank[t, k] == -1
                    continue
                d = e // El
                assert rank[t, k] == d
                key = (s, t, k) if do_expand else (s, t)
                assert row[t, k] == expect[d][key]
    for d in range(R):
        gl = outs[d]['layout']
        per_expert = [sum(int((idxs[s] == d * El + j).sum()) for s in range(R)) for j in range(El)]
        assert gl.recv_per_expert.tolist() == per_expert
        n_rows = len(expect[d])
        if do_expand:
            assert outs[d]['valid'].sum() == n_rows
            ends = gl.psum_recv_per_expert.tolist()
            start = 0
            for j in range(El):
                assert ends[j] - start == per_expert[j]
                start = (ends[j] + A - 1) // A * A
            assert gl.num_expanded_tokens == start
        else:
            assert gl.num_recv_tokens == n_rows and bool(outs[d]['valid'].all())
            src = outs[d]['meta'][:, 0]
            assert bool((src[1:] > src[:-1]).all()), 'rows must be ordered by (source rank, token)'
            assert gl.psum_recv_per_rank[-1] == n_rows


def test_get_dispatch_layout_ref():
    idx = torch.tensor([[0, 5, -1], [7, 6, 1]])
    per_rank, per_expert, in_rank = layout_ref.get_dispatch_layout_ref(idx, 8, 4)
    assert per_rank.tolist() == [2, 0, 1, 1]
    assert per_expert.tolist() == [1, 1, 0, 0, 0, 1, 1, 1]
    assert in_rank.tolist() == [[True, False, True, False], [True, False, False, True]]


def test_expert_tile_groups_and_segment_offsets():
    """Host-free helpers that map the expand layout's expert segments onto GEMM tiles (CPU tensors work as well)."""
    import torch
    from deepep_ascend_b200.ops import gemm as G
    torch.manual_seed(3)
    for _ in range(20):
        num_experts = int(torch.randint(1, 9, (1,)))
        counts = torch.randint(0, 400, (num_experts,))
        counts[torch.rand(num_experts) < 0.3] = 0
        ends, start = [], 0
        for c in counts.tolist():
            ends.append(start + c)
            start = (start + c + 127) // 128 * 128
        rows = max(start, 128)
        ends_t = torch.tensor(ends, dtype=torch.int32)
        tile_group, valid = G.expert_tile_groups(ends_t, rows)
        off = G.segment_offsets(ends_t)
        exp_group = torch.full((rows // 128,), -1, dtype=torch.int32)
        exp_valid = torch.zeros(rows, dtype=torch.bool)
        s = 0
        for e, c in enumerate(counts.tolist()):
            exp_valid[s:s + c] = True
            for t in range(s // 128, (s + c + 127) // 128):
                exp_group[t] = e
            assert off[e].item() == s
            s = (s + c + 127) // 128 * 128
        assert off[-1].item() == s
        assert torch.equal(tile_group[:rows // 128], exp_group), (counts, tile_group, exp_group)
        assert torch.equal(valid, exp_valid)


def test_local_expand_plan_statement():
    """Numbering of the (row, k) pairs of a non-expand dispatch inside their experts' 128-aligned segments: the PyTorch
    statement (which the kernels are checked against on a GPU) against brute-force loops."""
    import torch
    from deepep_ascend_b200.ops import gemm as G
    g = torch.Generator().manual_seed(9)
    for rows, K, El in ((1, 1, 1), (50, 2, 3), (333, 8, 16), (64, 4, 5)):
        idx = torch.full((rows, K), -1, dtype=torch.int64)
        for r in range(rows):
            n = int(torch.randint(0, min(K, El) + 1, (1,), generator=g))
            idx[r, torch.randperm(K, generator=g)[:n]] = torch.randperm(El, generator=g)[:n]
        counts = [int((idx == e).sum()) for e in range(El)]
        starts, psum, s0 = [], [], 0
        for c in counts:
            starts.append(s0)
            s0 += (c + 127) // 128 * 128
            psum.append(s0)
        want = torch.full((rows, K), -1, dtype=torch.int32)
        nxt = list(starts)
        for r in range(rows):
            for k in range(K):
                e = int(idx[r, k])
                if e >= 0:
                    want[r, k] = nxt[e]
                    nxt[e] += 1
        pos, seg_end = G.local_expand_plan(idx, torch.tensor(psum, dtype=torch.int32))
        assert torch.equal(pos, want)
        assert seg_end.tolist() == [s + c for s, c in zip(starts, counts)]
