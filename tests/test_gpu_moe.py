"""Fused MoE layer (dispatch -> FP8 grouped GEMM -> SwiGLU -> FP8 grouped GEMM -> weighted combine) and its
backward pass on one GPU (a group of one rank), against a plain fp32 PyTorch statement of the layer."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('copy_rows,chunks,local_expand', [(False, 1, True), (True, 1, True), (True, 2, True), (True, 4, True),
                                                          (False, 1, False), (True, 1, False), (True, 2, False)])
@pytest.mark.parametrize('T,H,I,E,K', [(200, 256, 128, 4, 2), (512, 1024, 512, 8, 4)])
def test_fused_moe_forward_backward(T, H, I, E, K, copy_rows, chunks, local_expand):
    from deepep_ascend_b200 import ElasticBuffer
    from deepep_ascend_b200.models.moe import FusedMoE, moe_reference
    from deepep_ascend_b200.utils.math import calc_diff
    torch.manual_seed(0)
    buf = ElasticBuffer(None, num_max_tokens_per_rank=T, hidden=H, num_topk=K, enable_expand=True, num_experts=E,
                        expert_alignment=128)
    try:
        layer = FusedMoE(buf, E, H, I, init_std=0.05, num_sms=16, copy_saved_rows=copy_rows, num_chunks=chunks, local_expand=local_expand)
        x = torch.randn(T, H, device='cuda').bfloat16().requires_grad_(True)
        scores = torch.softmax(torch.randn(T, E, device='cuda'), dim=-1)
        w, idx = scores.topk(K, dim=-1)
        idx[::7, 0] = -1
        w = w.clone().requires_grad_(True)
        out = layer(x, idx, w)
        g = torch.randn_like(out)
        out.backward(g)
        torch.cuda.synchronize()
        buf.check_status()

        xr = x.detach().float().requires_grad_(True)
        wr = w.detach().clone().requires_grad_(True)
        w13 = layer.w13.detach().float().requires_grad_(True)
        w2 = layer.w2.detach().float().requires_grad_(True)
        ref = moe_reference(xr, idx, wr, w13, w2)
        ref.backward(g.float())
        assert calc_diff(out.float(), ref) < 3e-3, calc_diff(out.float(), ref)
        assert calc_diff(x.grad.float(), xr.grad) < 3e-3, calc_diff(x.grad.float(), xr.grad)
        assert calc_diff(w.grad, wr.grad) < 3e-3, calc_diff(w.grad, wr.grad)
        assert calc_diff(layer.w2.grad.float(), w2.grad) < 3e-3, calc_diff(layer.w2.grad.float(), w2.grad)
        assert calc_diff(layer.w13.grad.float(), w13.grad) < 3e-3, calc_diff(layer.w13.grad.float(), w13.grad)
    finally:
        buf.destroy()


@pytest.mark.parametrize('T,H,I,E,K,chunks', [(200, 256, 128, 4, 2, 1), (512, 1024, 512, 8, 4, 2)])
def test_fused_moe_fp8_backward(T, H, I, E, K, chunks):
    """``fp8_backward=True``: the data-gradient GEMMs and the dispatch of the output gradient run in e4m3 with block scales.
    The gradients stay within the accuracy of an FP8 pipeline (calc_diff against the fp32 layer), and the forward
    result is the same as without the option."""
    from deepep_ascend_b200 import ElasticBuffer
    from deepep_ascend_b200.models.moe import FusedMoE, moe_reference
    from deepep_ascend_b200.utils.math import calc_diff
    torch.manual_seed(1)
    buf = ElasticBuffer(None, num_max_tokens_per_rank=T, hidden=H, num_topk=K, enable_expand=True, num_experts=E,
                        expert_alignment=128)
    try:
        layer = FusedMoE(buf, E, H, I, init_std=0.05, num_sms=16, num_chunks=chunks, fp8_backward=True)
        x = torch.randn(T, H, device='cuda').bfloat16().requires_grad_(True)
        w, idx = torch.softmax(torch.randn(T, E, device='cuda'), dim=-1).topk(K, dim=-1)
        idx[::5, 1] = -1
        w = w.clone().requires_grad_(True)
        out = layer(x, idx, w)
        g = torch.randn_like(out)
        out.backward(g)
        torch.cuda.synchronize()
        buf.check_status()
        layer.fp8_backward = False
        with torch.no_grad():
            assert torch.equal(layer(x, idx, w), out)
        xr, wr = x.detach().float().requires_grad_(True), w.detach().clone().requires_grad_(True)
        w13, w2 = layer.w13.detach().float().requires_grad_(True), layer.w2.detach().float().requires_grad_(True)
        moe_reference(xr, idx, wr, w13, w2).backward(g.float())
        diffs = dict(dx=calc_diff(x.grad.float(), xr.grad), dw=calc_diff(w.grad, wr.grad),
                     dw2=calc_diff(layer.w2.grad.float(), w2.grad), dw13=calc_diff(layer.w13.grad.float(), w13.grad))
        assert all(v < 5e-3 for v in diffs.values()), diffs
    finally:
        buf.destroy()


@pytest.mark.parametrize('rows,H,I', [(128, 256, 128), (640, 1024, 512)])
def test_backward_elementwise_kernels(rows, H, I):
    """The three element-wise kernels of the backward pass (row-major and transposed outputs) vs PyTorch."""
    from deepep_ascend_b200.ops import gemm as G
    from deepep_ascend_b200.utils.math import per_token_cast_to_fp8, per_token_cast_back
    torch.manual_seed(rows)
    valid = torch.rand(rows, device='cuda') > 0.2
    g = torch.randn(rows, H, device='cuda').bfloat16()
    y = torch.randn(rows, H, device='cuda').bfloat16()
    w = torch.rand(rows, device='cuda')
    dy, dy_t, dot = G.moe_bwd_prep(g, y, w, valid)
    vm = valid.unsqueeze(1)
    ref_dy = torch.where(vm, (g.float() * w.unsqueeze(1)).bfloat16(), torch.zeros_like(g))
    assert torch.equal(dy, ref_dy)
    assert torch.equal(dy_t, ref_dy.t().contiguous())
    ref_dot = torch.where(valid, (g.float() * y.float()).sum(1), torch.zeros_like(w))
    torch.testing.assert_close(dot, ref_dot, rtol=1e-4, atol=1e-3)

    d_act = torch.randn(rows, I, device='cuda').bfloat16()
    h = torch.randn(rows, 2 * I, device='cuda').bfloat16()
    dh, dh_t, act_t = G.swiglu_bwd(d_act, h, valid)
    gate, up, d = h[:, :I].float(), h[:, I:].float(), d_act.float()
    sig = torch.sigmoid(gate)
    ref_dh = torch.cat([d * up * sig * (1 + gate * (1 - sig)), d * gate * sig], dim=1)
    ref_dh = torch.where(vm, ref_dh, torch.zeros_like(ref_dh))
    ref_act = torch.where(vm, gate * sig * up, torch.zeros_like(gate))
    torch.testing.assert_close(dh.float(), ref_dh, rtol=2e-2, atol=2e-2)
    assert torch.equal(dh_t, dh.t().contiguous())
    torch.testing.assert_close(act_t.float(), ref_act.t(), rtol=2e-2, atol=2e-2)

    dh2, dh2_t, act2_t, dot2 = G.swiglu_bwd(d_act, h, valid, row_weight=w)
    ref_dh2 = torch.where(vm, ref_dh * w.unsqueeze(1), torch.zeros_like(ref_dh))
    torch.testing.assert_close(dh2.float(), ref_dh2, rtol=2e-2, atol=2e-2)
    assert torch.equal(dh2_t, dh2.t().contiguous()) and torch.equal(act2_t, act_t)
    ref_dot2 = torch.where(valid, (d * act_t.t().float()).sum(1), torch.zeros_like(w))
    torch.testing.assert_close(dot2, ref_dot2, rtol=1e-3, atol=1e-2)
    gw_t = G.weighted_transpose(g, w, valid)
    assert torch.equal(gw_t, ref_dy.t().contiguous())

    x = torch.randn(rows, H, device='cuda').bfloat16()
    q, sf = per_token_cast_to_fp8(x)
    x_t = G.dequant_transpose(q, sf, valid)
    ref_x = torch.where(vm, per_token_cast_back(q, sf).bfloat16(), torch.zeros_like(x))
    assert torch.equal(x_t, ref_x.t().contiguous())


def test_two_layers_share_one_buffer():
    """Two layers on ONE buffer, both forwards before any backward (what gradient accumulation and pipeline micro-batches
    do): the rows a layer keeps for its backward pass must survive the other layer's dispatches."""
    from deepep_ascend_b200 import ElasticBuffer
    from deepep_ascend_b200.models.moe import FusedMoE, moe_reference
    from deepep_ascend_b200.utils.math import calc_diff
    T, H, I, E, K = 256, 512, 256, 4, 2
    torch.manual_seed(3)
    buf = ElasticBuffer(None, num_max_tokens_per_rank=T, hidden=H, num_topk=K, enable_expand=True, num_experts=E, expert_alignment=128)
    try:
        layers = [FusedMoE(buf, E, H, I, init_std=0.05, num_sms=8) for _ in range(2)]
        xs, ws, idxs, outs, gs = [], [], [], [], []
        for layer in layers:
            x = torch.randn(T, H, device='cuda').bfloat16().requires_grad_(True)
            w, idx = torch.softmax(torch.randn(T, E, device='cuda'), dim=-1).topk(K, dim=-1)
            w = w.clone().requires_grad_(True)
            outs.append(layer(x, idx, w))
            xs.append(x), ws.append(w), idxs.append(idx), gs.append(torch.randn(T, H, device='cuda').bfloat16())
        for out, g in zip(outs, gs):
            out.backward(g)
        torch.cuda.synchronize()
        buf.check_status()
        for layer, x, w, idx, g in zip(layers, xs, ws, idxs, gs):
            xr, wr = x.detach().float().requires_grad_(True), w.detach().clone().requires_grad_(True)
            w13, w2 = layer.w13.detach().float().requires_grad_(True), layer.w2.detach().float().requires_grad_(True)
            moe_reference(xr, idx, wr, w13, w2).backward(g.float())
            assert calc_diff(x.grad.float(), xr.grad) < 3e-3 and calc_diff(w.grad, wr.grad) < 3e-3
            assert calc_diff(layer.w13.grad.float(), w13.grad) < 3e-3 and calc_diff(layer.w2.grad.float(), w2.grad) < 3e-3
    finally:
        buf.destroy()


@pytest.mark.parametrize('R', [2, 4])
def test_moe_forward_on_virtual_ranks(R):
    """The forward data flow of the layer across several ranks on one GPU (every collective of the virtual ranks is one
    cooperative launch): expand-layout FP8 dispatch -> grouped FP8 GEMMs with SwiGLU -> fused weighted combine, against the
    plain PyTorch layer that holds all experts."""
    from deepep_ascend_b200.backends.emulated import EmulatedWorld
    from deepep_ascend_b200.models.moe import moe_reference
    from deepep_ascend_b200.ops import gemm as G
    from deepep_ascend_b200.utils.math import calc_diff
    T, H, I, K = 160, 512, 256, 4
    E = 4 * R
    El = E // R
    torch.manual_seed(R)
    world = EmulatedWorld(R, num_max_tokens_per_rank=T, hidden=H, num_topk=K, use_fp8_dispatch=True, enable_expand=True,
                          num_experts=E, expert_alignment=128)
    try:
        w13 = (torch.randn(E, 2 * I, H, device='cuda') * 0.05).bfloat16()
        w2 = (torch.randn(E, H, I, device='cuda') * 0.05).bfloat16()
        xs = [torch.randn(T - r, H, device='cuda').bfloat16() for r in range(R)]
        tk = [torch.softmax(torch.randn(T - r, E, device='cuda'), dim=-1).topk(K, dim=-1) for r in range(R)]
        ws, idxs = [t[0].contiguous() for t in tk], [t[1].contiguous() for t in tk]
        outs = world.dispatch(xs, idxs, ws, E, num_sms=6, expert_alignment=128, do_expand=True)
        ys, handles = [], []
        for r, ((rx, rsf), _, recv_w, handle) in enumerate(outs):
            q13, s13 = G.quantize_weight_blocks(w13[r * El:(r + 1) * El].float())
            q2, s2 = G.quantize_weight_blocks(w2[r * El:(r + 1) * El].float())
            tile_group, _ = G.expert_tile_groups(handle.psum_num_recv_tokens_per_expert, handle.num_rows)
            h = G.grouped_gemm_nt(rx, q13, tile_group, sfa=rsf, sfb=s13, buffer=world.buffers[r])
            a2, sf2 = G.swiglu_quant(h)
            y = world.buffers[r].get_combine_buffer(handle)
            G.grouped_gemm_nt(a2, q2, tile_group, out=y, sfa=sf2, sfb=s2, buffer=world.buffers[r])
            ys.append(y)
            handles.append(handle)
        res = world.combine(ys, handles, weighted=True, num_sms=6)
        torch.cuda.synchronize()
        for r in range(R):
            world.buffers[r].check_status()
            ref = moe_reference(xs[r].float(), idxs[r], ws[r], w13.float(), w2.float())
            d = calc_diff(res[r][0].float(), ref)
            assert d < 3e-3, (r, d)
    finally:
        world.destroy()


def test_expert_segments_kernel_matches_its_pytorch_statement():
    """Tile groups, row validity and segment boundaries of the expand layout: the one-launch kernel against plain PyTorch."""
    from deepep_ascend_b200.ops import gemm as G
    torch.manual_seed(11)
    for trial in range(30):
        num_experts = int(torch.randint(1, 70, (1,)))
        alignment = 128 * int(torch.randint(1, 3, (1,)))
        counts = torch.randint(0, 700, (num_experts,))
        counts[torch.rand(num_experts) < 0.3] = 0
        ends, start = [], 0
        for c in counts.tolist():
            ends.append(start + c)
            start = (start + c + alignment - 1) // alignment * alignment
        rows = start + (64 if trial % 3 == 0 else 0)        # also a row count that is not a multiple of the tile
        ends_t = torch.tensor(ends, dtype=torch.int32, device='cuda')
        got = G.expert_segments(ends_t, rows, alignment)
        want = G.expert_segments_ref(ends_t, rows, alignment)
        for g, w in zip(got, want):
            assert g.dtype == w.dtype and torch.equal(g, w)
        assert torch.equal(G.segment_offsets(ends_t, alignment), want[2])


@pytest.mark.parametrize('rows,I', [(5, 128), (77, 384), (300, 2048), (40, 4352)])
def test_swiglu_quant_kernel(rows, I):
    """SwiGLU fused with the 1 x 128 e4m3 cast against plain PyTorch (I = 4352 takes more than 16 steps per row, I = 384
    ends in a half step)."""
    from deepep_ascend_b200.ops import gemm as G
    from deepep_ascend_b200.utils.math import calc_diff, per_token_cast_back
    torch.manual_seed(rows + I)
    h = (torch.randn(rows, 2 * I, device='cuda') * 2).bfloat16()
    h[0, :I] = -60.0                      # sigmoid underflows: the activation is 0 and the scale is clamped
    q, sf, act = G.swiglu_quant(h, keep_bf16=True)
    gate, up = h[:, :I].float(), h[:, I:].float()
    ref = (torch.nn.functional.silu(gate) * up)
    assert act.dtype == torch.bfloat16 and q.dtype == torch.float8_e4m3fn and sf.shape == (rows, I // 128)
    torch.testing.assert_close(act.float(), ref.bfloat16().float(), rtol=1.6e-2, atol=1e-6)
    # the scales are exactly amax / 448 of the bf16 activation the kernel produced, and the codes are its cast
    # (stated on the CPU: CUDA PyTorch turns a division by a constant into a multiplication by its reciprocal)
    act_c = act.float().cpu().view(rows, I // 128, 128)
    amax = act_c.abs().amax(dim=2).clamp(1e-4)
    assert torch.equal(sf.cpu(), amax / 448.0)
    want_q = (act_c * (448.0 / amax).unsqueeze(2)).view(rows, I).to(torch.float8_e4m3fn)
    assert torch.equal(q.cpu().view(torch.uint8), want_q.view(torch.uint8))
    assert calc_diff(per_token_cast_back(q, sf), ref) < 1e-3
    q2, sf2 = G.swiglu_quant(h)
    assert torch.equal(q2.view(torch.uint8), q.view(torch.uint8)) and torch.equal(sf2, sf)


@pytest.mark.parametrize('rows,K,El,H,idx_dtype', [(37, 2, 4, 256, torch.int64), (900, 8, 32, 1024, torch.int64), (513, 4, 7, 7168, torch.int32)])
def test_local_expand_and_reduce_kernels(rows, K, El, H, idx_dtype):
    """The (token, rank) -> (token, expert) expansion on the expert rank and its inverse, against plain PyTorch: positions
    ordered by received row inside 128-aligned expert segments, row / scale / weight copies, weighted and plain reductions."""
    from deepep_ascend_b200.ops import gemm as G
    g = torch.Generator().manual_seed(rows + K)
    # every row picks up to K distinct local experts; the other lanes (experts of other ranks) are -1
    idx = torch.full((rows, K), -1, dtype=torch.int64)
    for r in range(rows):
        n = int(torch.randint(0, min(K, El) + 1, (1,), generator=g))
        lanes = torch.randperm(K, generator=g)[:n]
        idx[r, lanes] = torch.randperm(El, generator=g)[:n]
    counts = torch.stack([(idx == e).sum() for e in range(El)])
    aligned = (counts + 127) // 128 * 128
    psum = aligned.cumsum(0).to(torch.int32)
    starts = psum - aligned.to(torch.int32)
    total = int(psum[-1])
    want_pos = torch.full((rows, K), -1, dtype=torch.int32)
    for e in range(El):
        rr, kk = torch.nonzero(idx == e, as_tuple=True)          # row-major order = received order
        want_pos[rr, kk] = starts[e] + torch.arange(len(rr), dtype=torch.int32)
    # the index tensor as dispatch returns it: rows with a pitch (a view into wider records)
    wide = torch.full((rows, K + 3), 77, dtype=idx_dtype, device='cuda')
    wide[:, :K] = idx.to(idx_dtype).cuda()
    pos, seg_end = G.local_expand_plan(wide[:, :K], psum.cuda())
    assert torch.equal(pos.cpu(), want_pos)
    assert torch.equal(seg_end.cpu(), (starts + counts.to(torch.int32)))

    x = torch.randn(rows, H, generator=g).bfloat16().cuda()
    sf = torch.rand(rows, H // 128, generator=g).cuda()
    w = torch.rand(rows, K, generator=g).cuda()
    x_e, sf_e, w_e = G.local_expand_copy(pos, x, total, sf=sf, w=w)
    valid = pos >= 0
    src_row = torch.nonzero(valid, as_tuple=True)[0]
    at = pos[valid].long()
    assert torch.equal(x_e[at], x[src_row]) and torch.equal(sf_e[at], sf[src_row]) and torch.equal(w_e[at], w[valid])
    q = x.view(torch.uint8)[:, :H].contiguous().view(torch.float8_e4m3fn)       # a one-byte element type takes the same path
    assert torch.equal(G.local_expand_copy(pos, q, total)[0][at].view(torch.uint8), q[src_row].view(torch.uint8))

    y = torch.zeros(total, H, dtype=torch.bfloat16, device='cuda')
    y[at] = torch.randn(len(at), H, device='cuda').bfloat16()
    for weights in (None, w_e):
        got = G.local_reduce(pos, y, w=weights)
        want = torch.zeros(rows, H, device='cuda')
        for k in range(K):
            m = valid[:, k]
            rowsel = y[pos[m, k].long()].float()
            want[m] += rowsel if weights is None else rowsel * weights[pos[m, k].long()].unsqueeze(1)
        torch.testing.assert_close(got.float(), want.bfloat16().float(), rtol=1.6e-2, atol=1e-3)
        assert bool((got[~valid.any(dim=1)] == 0).all())
    out = torch.empty(rows, H, dtype=torch.bfloat16, device='cuda')
    assert G.local_reduce(pos, y, w=w_e, out=out).data_ptr() == out.data_ptr()


def test_fused_moe_on_a_buffer_without_expand_regions():
    """With ``local_expand`` (the default) the layer only uses the (token, rank) layout of the buffer, so a buffer built without
    ``enable_expand`` serves it; without ``local_expand`` the constructor asks for the expand-capable buffer."""
    from deepep_ascend_b200 import ElasticBuffer
    from deepep_ascend_b200.models.moe import FusedMoE, moe_reference
    from deepep_ascend_b200.utils.math import calc_diff
    T, H, I, E, K = 300, 512, 256, 8, 4
    torch.manual_seed(21)
    buf = ElasticBuffer(None, num_max_tokens_per_rank=T, hidden=H, num_topk=K)      # rows sized for the bf16 gradients of the backward pass
    try:
        with pytest.raises(AssertionError, match='enable_expand'):
            FusedMoE(buf, E, H, I, local_expand=False)
        layer = FusedMoE(buf, E, H, I, init_std=0.05, num_sms=16)
        x = torch.randn(T, H, device='cuda').bfloat16().requires_grad_(True)
        w, idx = torch.softmax(torch.randn(T, E, device='cuda'), dim=-1).topk(K, dim=-1)
        w = w.clone().requires_grad_(True)
        out = layer(x, idx, w)
        g = torch.randn_like(out)
        out.backward(g)
        torch.cuda.synchronize()
        buf.check_status()
        xr, wr = x.detach().float().requires_grad_(True), w.detach().clone().requires_grad_(True)
        w13, w2 = layer.w13.detach().float().requires_grad_(True), layer.w2.detach().float().requires_grad_(True)
        ref = moe_reference(xr, idx, wr, w13, w2)
        ref.backward(g.float())
        assert calc_diff(out.float(), ref) < 3e-3 and calc_diff(x.grad.float(), xr.grad) < 3e-3
        assert calc_diff(layer.w13.grad.float(), w13.grad) < 3e-3 and calc_diff(w.grad, wr.grad) < 3e-3
    finally:
        buf.destroy()
