"""Expert-parallel MoE feed-forward layer built from this library's own kernels:

    dispatch (expand layout, bf16 -> e4m3 cast fused into the NVLink scatter)
      -> grouped block-scaled FP8 GEMM on tcgen05 (gate | up projection)
      -> SwiGLU fused with the e4m3 cast of the next GEMM's input
      -> grouped block-scaled FP8 GEMM (down projection) writing straight into the combine input region
      -> combine (pull + top-k-weighted fp32 reduction in one kernel)

and its backward pass, in which the gradients travel the same routes in reverse (the backward of combine is a
cached dispatch, the backward of dispatch is a combine).  The reference library stops at dispatch / combine and
leaves the layer to the caller (its README shows this data flow for DeepSeek-V3 style training, README.md:227-273).
"""
import torch
import torch.nn as nn

from ..buffers.elastic import ElasticBuffer
from ..ops import gemm as G


class _MoEFunction(torch.autograd.Function):
    """Forward and backward of the layer.  The token batch is cut into ``layer.num_chunks`` pieces that run as a software
    pipeline: while the tensor cores work on the experts of chunk c, the communication stream combines chunk c - 1 and
    dispatches chunk c + 1, each through one of the buffer's two receive slots / two combine input regions.  Every rank
    issues its communication kernels in the same order on ONE stream (d0, d1, c0, d2, c1, ...), and the GEMMs leave the
    communication kernels their SMs (``num_sms`` of them), so the kernels of different ranks can never wait for SMs that
    a kernel waiting for them holds."""

    @staticmethod
    def forward(ctx, x, topk_weights, w13, w2, layer, topk_idx):
        buf: ElasticBuffer = layer.buffer
        E = layer.num_experts
        T = x.shape[0]
        C = max(1, min(layer.num_chunks, T))
        bounds = [T * c // C for c in range(C + 1)]
        pipelined = C > 1
        need_grad = any(ctx.needs_input_grad)
        keep_copy = need_grad and (pipelined or layer.copy_saved_rows)
        comm_sms, gemm_sms = layer.sm_split(pipelined)
        q13, s13, q2, s2 = layer.fp8_weights()
        out = torch.empty((T, x.shape[1]), dtype=torch.bfloat16, device=x.device)
        slots = buf.regions.num_recv_slots
        start = buf.capture() if pipelined else None
        disp, g1_done, comb_done, saved, handles = {}, [], [], [], []
        local = layer.local_expand
        no_pos = torch.empty(0, dtype=torch.int32, device=x.device)

        def issue_dispatch(c):
            lo, hi = bounds[c], bounds[c + 1]
            kw = {}
            if pipelined:
                # the receive slot of chunk c was last read by the first GEMM (and the copies for backward) of chunk c - slots
                kw = dict(previous_event=g1_done[c - slots] if c >= slots else start, allocate_on_comm_stream=True,
                          async_with_compute_stream=True)
            disp[c] = buf.dispatch(x[lo:hi], topk_idx[lo:hi], topk_weights[lo:hi], num_experts=E, do_expand=not local,
                                   expert_alignment=G.BLOCK_M, fused_fp8_cast=True, num_sms=comm_sms, **kw)

        issue_dispatch(0)
        for c in range(C):
            lo, hi = bounds[c], bounds[c + 1]
            (rx, rsf), recv_idx, recv_w, handle, ev = disp.pop(c)
            ev.current_stream_wait()
            if local:
                # One row per (token, rank) came over NVLink; every local expert the token selected gets its copy here, in the
                # expert's 128-aligned segment (rows in received order).  The copies are private to this call.
                rows = sum(handle.num_recv_tokens_per_expert_list)
                pos, seg_end = G.local_expand_plan(recv_idx, handle.psum_num_recv_tokens_per_expert)
                rx, rsf, recv_w = G.local_expand_copy(pos, rx, rows, sf=rsf, w=recv_w)
                tile_group, valid_row, seg_off = G.expert_segments(seg_end, rows)
            else:
                rows, pos = handle.num_rows, no_pos
                tile_group, valid_row, seg_off = G.expert_segments(handle.psum_num_recv_tokens_per_expert, rows)
            h = G.grouped_gemm_nt(rx, q13, tile_group, sfa=rsf, sfb=s13, num_sms=gemm_sms, buffer=buf)    # [rows, 2I]
            if keep_copy and not local:
                # the received rows live in a receive slot of the buffer that later dispatches will reuse
                rx, rsf, recv_w = rx.clone(), rsf.clone(), recv_w.clone()
            if pipelined:
                g1_done.append(buf.capture())
                if c + 1 < C:
                    issue_dispatch(c + 1)      # runs while the tensor cores are busy with this chunk
            a2, sf2 = G.swiglu_quant(h)
            if pipelined and c >= 1:
                # the combine input region about to be written was read by the combine of chunk c - 2, which every rank
                # has finished once this rank's combine of chunk c - 1 has completed
                comb_done[c - 1].current_stream_wait()
            if local:
                # the weighted sum over a token's local experts happens here, so one row per (token, rank) travels home
                y_exp = G.grouped_gemm_nt(a2, q2, tile_group, sfa=sf2, sfb=s2, num_sms=gemm_sms, buffer=buf)      # [rows, H]
                y = G.local_reduce(pos, y_exp, w=recv_w, out=buf.get_combine_buffer(handle))
            else:
                y = buf.get_combine_buffer(handle)
                G.grouped_gemm_nt(a2, q2, tile_group, out=y, sfa=sf2, sfb=s2, num_sms=gemm_sms, buffer=buf)    # [rows, H] in the combine region
            kw = dict(previous_event=buf.capture(), allocate_on_comm_stream=True, async_with_compute_stream=True) if pipelined else {}
            _, _, cev = buf.combine(y, handle, weighted=not local, num_sms=comm_sms, out=out[lo:hi], **kw)
            comb_done.append(cev)
            handles.append(handle)
            saved += [rx, rsf, recv_w, h, tile_group, valid_row, seg_off, pos]
        for cev in comb_done[-2:]:
            cev.current_stream_wait()
        ctx.layer, ctx.handles, ctx.bounds = layer, handles, bounds
        ctx.save_for_backward(*saved)
        return out

    @staticmethod
    def backward(ctx, d_out):
        layer, bounds = ctx.layer, ctx.bounds
        buf: ElasticBuffer = layer.buffer
        w2_t, w13_t = (None, None) if layer.fp8_backward else layer.transposed_weights()
        d_out = d_out.contiguous()
        dxs, dws, d_w2, d_w13 = [], [], None, None
        for c, handle in enumerate(ctx.handles):
            rx, rsf, recv_w, h, tile_group, valid_row, seg_off, pos = ctx.saved_tensors[8 * c:8 * c + 8]
            rw = recv_w.contiguous()
            local, rows = layer.local_expand, h.shape[0]

            def send_home(d_rows_exp, d_w_rows):
                """Backward of dispatch: the gradient rows (and the gradient of every routing weight) travel to the tokens' ranks."""
                if not local:
                    return buf.combine(d_rows_exp, handle, topk_weights=d_w_rows, num_sms=layer.num_sms)[:2]
                d_recv = G.local_reduce(pos, d_rows_exp, out=buf.get_combine_buffer(handle))
                d_w = torch.where(pos >= 0, d_w_rows[pos.clamp(min=0).long()], torch.zeros((), device=pos.device))
                return buf.combine(d_recv, handle, topk_weights=d_w, num_sms=layer.num_sms)[:2]
            if layer.fp8_backward:
                # Data gradients on the e4m3 tensor cores, as the forward GEMMs: the gradient rows are cast (1 x 128 scales)
                # inside the dispatch kernel, the weights are the forward e4m3 weights transposed (128 x 128 blocks stay
                # 128 x 128 blocks), and the SwiGLU gradient is cast once more before the up projection.
                q2_t, s2_t, q13_t, s13_t = layer.fp8_transposed_weights()
                (g_q, g_sf), _, _, _, _ = buf.dispatch(d_out[bounds[c]:bounds[c + 1]], handle=handle, fused_fp8_cast=True, num_sms=layer.num_sms)
                if local:
                    g_q, g_sf = G.local_expand_copy(pos, g_q, rows, sf=g_sf)
                d_act_u = G.grouped_gemm_nt(g_q, q2_t, tile_group, sfa=g_sf, sfb=s2_t, buffer=buf)             # [rows, I]
                dh, dh_t, act_t, d_w_rows = G.swiglu_bwd(d_act_u, h, valid_row, row_weight=rw)
                dh_q, dh_sf = G.per_token_cast_to_fp8(dh)
                d_recv = None if local else buf.get_combine_buffer(handle)
                d_recv = G.grouped_gemm_nt(dh_q, q13_t, tile_group, out=d_recv, sfa=dh_sf, sfb=s13_t, buffer=buf)
                dx, d_topk_w = send_home(d_recv, d_w_rows)
                # (g * w)^T for the weight gradient: the routing weight rides on the scales of the dequantisation
                dy_t = G.dequant_transpose(g_q, g_sf * rw.unsqueeze(1), valid_row)
            else:
                # backward of the weighted combine: every expert row receives its token's gradient g (cached dispatch)
                g_rows, _, _, _, _ = buf.dispatch(d_out[bounds[c]:bounds[c + 1]], handle=handle, fused_fp8_cast=False, num_sms=layer.num_sms)
                if local:
                    g_rows = G.local_expand_copy(pos, g_rows, rows)[0]
                # down projection on the UNWEIGHTED gradient: d loss / d weight of a row is <g W2, activation> (= <g, y>, so the
                # expert outputs need not be kept), and the weight is applied inside the SwiGLU backward kernel.  Padding rows of
                # g_rows hold stale data; every consumer masks them.
                d_act_u = G.grouped_gemm_nt(g_rows, w2_t, tile_group, buffer=buf)                    # [rows, I]
                dh, dh_t, act_t, d_w_rows = G.swiglu_bwd(d_act_u, h, valid_row, row_weight=rw)
                # up projection: the gradient rows go into the combine region and travel home (backward of dispatch)
                d_recv = None if local else buf.get_combine_buffer(handle)
                d_recv = G.grouped_gemm_nt(dh, w13_t, tile_group, out=d_recv, buffer=buf)
                dx, d_topk_w = send_home(d_recv, d_w_rows)
                dy_t = G.weighted_transpose(g_rows, rw, valid_row)                                  # (g * w)^T [H, rows]
            # weight gradients: one K-grouped GEMM per weight tensor, reduction over the rows of every expert segment
            x_t = G.dequant_transpose(rx, rsf, valid_row)
            g2 = G.gemm_kgrouped(dy_t, act_t, seg_off)                                          # [El, H, I]
            g13 = G.gemm_kgrouped(dh_t, x_t, seg_off)                                           # [El, 2I, H]
            d_w2 = g2 if d_w2 is None else d_w2 + g2
            d_w13 = g13 if d_w13 is None else d_w13 + g13
            dxs.append(dx)
            dws.append(d_topk_w)
        dx = dxs[0] if len(dxs) == 1 else torch.cat(dxs)
        d_topk_w = dws[0] if len(dws) == 1 else torch.cat(dws)
        return dx, d_topk_w, d_w13, d_w2, None, None


class FusedMoE(nn.Module):
    """SwiGLU expert FFN sharded over an expert-parallel group.

    ``w13 [E_local, 2 * intermediate, hidden]`` (gate rows then up rows) and ``w2 [E_local, hidden, intermediate]`` are
    bf16 master weights; the forward pass runs on e4m3 copies with 128 x 128 block scales that are refreshed
    whenever the master weights change.  ``num_chunks > 1`` cuts the batch into chunks whose dispatch / combine run under
    the GEMMs of the neighbouring chunks (see ``_MoEFunction``).  ``forward(x [T, hidden] bf16, topk_idx [T, K], topk_weights [T, K] fp32)``
    returns ``sum_k w_k * FFN_{e_k}(x)`` as bf16 ``[T, hidden]``.
    """

    def __init__(self, buffer: ElasticBuffer, num_experts: int, hidden: int, intermediate: int, init_std: float = 0.02,
                 num_sms: int = 0, device='cuda', copy_saved_rows: bool = True, num_chunks: int = 1, fp8_backward: bool = False,
                 local_expand: bool = True):
        super().__init__()
        assert num_experts % buffer.num_ranks == 0 and hidden % 128 == 0 and intermediate % 128 == 0
        assert buffer.enable_expand or local_expand, \
            'without local_expand the layer uses the expand layout: construct the buffer with enable_expand=True, expert_alignment=128'
        self.buffer, self.num_experts, self.hidden, self.intermediate = buffer, num_experts, hidden, intermediate
        self.num_sms = num_sms
        # True (default): the dispatched rows kept for the backward pass are copied out of the receive slot, which later
        # dispatches on the same buffer (other layers, micro-batches, gradient accumulation) overwrite.  False saves the copy
        # and is only valid while no dispatch but this layer's own backward one runs on the buffer in between.
        self.copy_saved_rows = copy_saved_rows
        # > 1: the batch is processed as that many pipelined chunks (communication of one chunk under the GEMMs of another)
        self.num_chunks = num_chunks
        # True: the data-gradient GEMMs (and the dispatch of the output gradient) run in e4m3 with block scales like the forward
        # pass; the weight gradients stay in bf16.  False: the whole backward pass is bf16.
        self.fp8_backward = fp8_backward
        # True: dispatch and combine move one row per (token, rank); the copies for the token's local experts and the weighted sum
        # over them are made on the expert rank (``ops.gemm.local_expand_*`` / ``local_reduce``).  False: the buffer's expand layout
        # moves one row per (token, expert) over NVLink.  With top-8 of 256 experts on 8 ranks that is 8 rows per token instead of 5.25.
        self.local_expand = local_expand
        el = num_experts // buffer.num_ranks
        self.w13 = nn.Parameter((torch.randn(el, 2 * intermediate, hidden, device=device) * init_std).bfloat16())
        self.w2 = nn.Parameter((torch.randn(el, hidden, intermediate, device=device) * init_std).bfloat16())
        self._fp8 = None
        self._fp8_t = None
        self._t = None

    def sm_split(self, pipelined: bool):
        """(SMs of the communication kernels, SMs of the GEMMs; 0 = all).  In the pipelined schedule the two run at the same
        time, so the GEMMs leave the communication kernels their SMs."""
        if not pipelined:
            return self.num_sms, 0
        total = torch.cuda.get_device_properties('cuda').multi_processor_count
        comm = self.num_sms if self.num_sms else 24
        return comm, max(1, total - comm)

    def _versions(self):
        return (self.w13._version, self.w2._version, self.w13.data_ptr(), self.w2.data_ptr())

    def fp8_weights(self):
        if self._fp8 is None or self._fp8[0] != self._versions():
            q13, s13 = G.quantize_weight_blocks(self.w13.detach().float())
            q2, s2 = G.quantize_weight_blocks(self.w2.detach().float())
            self._fp8 = (self._versions(), (q13, s13, q2, s2))
        return self._fp8[1]

    def fp8_transposed_weights(self):
        """``(w2^T e4m3 [El, I, H], its scales, w13^T e4m3 [El, H, 2I], its scales)``: the forward e4m3 weights transposed (a
        128 x 128 scale block of W is a 128 x 128 scale block of W^T, so nothing is quantised again)."""
        if self._fp8_t is None or self._fp8_t[0] != self._versions():
            q13, s13, q2, s2 = self.fp8_weights()
            t = lambda w: w.transpose(1, 2).contiguous()    # noqa: E731
            self._fp8_t = (self._versions(), (t(q2.view(torch.uint8)).view(torch.float8_e4m3fn), t(s2),
                                              t(q13.view(torch.uint8)).view(torch.float8_e4m3fn), t(s13)))
        return self._fp8_t[1]

    def transposed_weights(self):
        if self._t is None or self._t[0] != self._versions():
            self._t = (self._versions(), (self.w2.detach().transpose(1, 2).contiguous(), self.w13.detach().transpose(1, 2).contiguous()))
        return self._t[1]

    def forward(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        return _MoEFunction.apply(x, topk_weights, self.w13, self.w2, self, topk_idx)


def moe_reference(x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, w13_all: torch.Tensor,
                  w2_all: torch.Tensor) -> torch.Tensor:
    """Plain PyTorch fp32 statement of the layer with ALL experts' weights on one device (for tests)."""
    T, H = x.shape
    I = w2_all.shape[2]
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    for k in range(topk_idx.shape[1]):
        for e in topk_idx[:, k].unique().tolist():
            if e < 0:
                continue
            m = topk_idx[:, k] == e
            h = x[m].float() @ w13_all[e].float().t()
            act = torch.nn.functional.silu(h[:, :I]) * h[:, I:]
            out[m] += topk_weights[m, k].unsqueeze(1) * (act @ w2_all[e].float().t())
    return out
