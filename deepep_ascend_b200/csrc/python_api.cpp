// Python bindings of the native runtime (module `_C`).
// Parity: csrc/python_api.cpp:1-54, csrc/elastic/binding.hpp:9-44 of the reference.
#include <torch/extension.h>

#include "kernels/api.h"
#include "runtime/coordinator.hpp"
#include "runtime/elastic_buffer.hpp"
#include "runtime/layout.hpp"
#include "runtime/low_latency.hpp"

namespace py = pybind11;
using namespace ep_host;

namespace {

std::vector<at::Tensor> get_dispatch_layout(const at::Tensor& topk_idx, int64_t num_experts, int64_t num_ranks) {
    TORCH_CHECK(topk_idx.is_cuda() && topk_idx.is_contiguous() && topk_idx.dim() == 2, "topk_idx must be contiguous [T, K]");
    TORCH_CHECK(topk_idx.scalar_type() == at::kLong || topk_idx.scalar_type() == at::kInt, "topk_idx must be int64 or int32");
    TORCH_CHECK(num_experts % num_ranks == 0 && num_ranks <= 32, "bad expert / rank counts");
    auto iopts = topk_idx.options().dtype(at::kInt);
    at::Tensor per_rank = at::zeros({num_ranks}, iopts);
    at::Tensor per_expert = at::zeros({num_experts}, iopts);
    at::Tensor in_rank = at::empty({topk_idx.size(0), num_ranks}, topk_idx.options().dtype(at::kBool));
    LayoutArgs a{};
    a.topk_idx = topk_idx.data_ptr();
    a.idx_is_64 = topk_idx.scalar_type() == at::kLong;
    a.num_tokens = static_cast<int>(topk_idx.size(0));
    a.num_topk = static_cast<int>(topk_idx.size(1));
    a.num_experts = static_cast<int>(num_experts);
    a.num_ranks = static_cast<int>(num_ranks);
    a.num_tokens_per_rank = per_rank.data_ptr<int32_t>();
    a.num_tokens_per_expert = per_expert.data_ptr<int32_t>();
    a.is_token_in_rank = reinterpret_cast<uint8_t*>(in_rank.data_ptr());
    cuda_check(ep::launch_layout(a, at::cuda::getCurrentCUDAStream()), "layout launch");
    return {per_rank, per_expert, in_rank};
}

// bf16 [T, H] -> (e4m3 [T, H], scales).  Scales are fp32 [T, ceil(H/128)] or, with use_ue8m0, int32
// [T, ceil(H/512)] holding four power-of-two exponents each.
std::vector<at::Tensor> per_token_cast_to_fp8(const at::Tensor& x, bool round_scale, bool use_ue8m0) {
    TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() == 2 && x.scalar_type() == at::kBFloat16, "x must be contiguous bf16 [T, H]");
    const int64_t T = x.size(0), H = x.size(1);
    TORCH_CHECK(H % 16 == 0, "hidden must be a multiple of 16");
    const int64_t G = (H + 127) / 128;
    at::Tensor q = at::empty({T, H}, x.options().dtype(at::kFloat8_e4m3fn));
    at::Tensor sf = use_ue8m0 ? at::zeros({T, (G + 3) / 4}, x.options().dtype(at::kInt)) : at::empty({T, G}, x.options().dtype(at::kFloat));
    QuantArgs a{};
    a.x = x.data_ptr();
    a.q = q.data_ptr();
    a.sf = reinterpret_cast<float*>(sf.data_ptr());
    a.num_tokens = static_cast<int>(T);
    a.hidden = static_cast<int>(H);
    a.round_scale = round_scale;
    a.use_ue8m0 = use_ue8m0;
    a.sf_stride_row = sf.size(1);
    a.sf_stride_col = 1;
    cuda_check(ep::launch_quant(a, at::cuda::getCurrentCUDAStream()), "quant launch");
    return {q, sf};
}

// Device int that the GEMM kernels raise when one of their bounded pipeline waits runs out (one per device).
at::Tensor& gemm_error_flag(int device) {
    static std::vector<at::Tensor> flags(64);
    if (!flags[device].defined()) flags[device] = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
    return flags[device];
}

// C[M, N] (bf16) = A[M, K] @ B[g][N, K]^T on the tcgen05 tensor cores.  bf16 operands, or float8_e4m3fn operands
// with fp32 block scales (sfa [M, ceil(K/128)] any strides, sfb [G, ceil(N/128), ceil(K/128)] contiguous).
// `tile_group` int32 [ceil(M/128)]: weights group of every 128-row tile (-1 = skip the tile).
at::Tensor gemm_nt(const at::Tensor& a, const at::Tensor& b, const std::optional<at::Tensor>& sfa, const std::optional<at::Tensor>& sfb,
                   const std::optional<at::Tensor>& tile_group, const std::optional<at::Tensor>& out, int64_t num_sms,
                   const std::optional<at::Tensor>& a_ready_flags, int64_t a_ready_value, const std::optional<at::Tensor>& a_flag_of_tile,
                   ElasticBufferCore* report_to) {
    TORCH_CHECK(a.is_cuda() && a.dim() == 2 && a.stride(1) == 1, "A must be [M, K] with contiguous rows");
    TORCH_CHECK(b.is_cuda() && (b.dim() == 2 || b.dim() == 3) && b.is_contiguous(), "B must be contiguous [N, K] or [G, N, K]");
    const bool fp8 = a.scalar_type() == at::kFloat8_e4m3fn;
    TORCH_CHECK(fp8 || a.scalar_type() == at::kBFloat16, "A must be bf16 or float8_e4m3fn");
    TORCH_CHECK(b.scalar_type() == a.scalar_type(), "A and B must have the same dtype");
    const int64_t M = a.size(0), K = a.size(1), G = b.dim() == 3 ? b.size(0) : 1, N = b.size(-2);
    TORCH_CHECK(b.size(-1) == K, "K mismatch");
    at::Tensor c = out.has_value() ? *out : at::empty({M, N}, a.options().dtype(at::kBFloat16));
    TORCH_CHECK(c.scalar_type() == at::kBFloat16 && c.dim() == 2 && c.size(0) == M && c.size(1) == N && c.stride(1) == 1, "bad output");
    GemmArgs g{};
    g.a = a.data_ptr();
    g.b = b.data_ptr();
    g.c = c.data_ptr();
    g.M = static_cast<int>(M);
    g.N = static_cast<int>(N);
    g.K = static_cast<int>(K);
    g.num_groups = static_cast<int>(G);
    g.is_fp8 = fp8;
    g.lda = a.stride(0);
    g.ldb = K;
    g.ldc = c.stride(0);
    if (fp8) {
        TORCH_CHECK(sfa.has_value() && sfb.has_value(), "fp8 operands need scale tensors");
        TORCH_CHECK(sfa->scalar_type() == at::kFloat && sfa->dim() == 2 && sfa->size(0) >= M && sfa->size(1) == (K + 127) / 128, "bad sfa");
        TORCH_CHECK(sfb->scalar_type() == at::kFloat && sfb->is_contiguous() && sfb->numel() == G * ((N + 127) / 128) * ((K + 127) / 128), "bad sfb");
        g.sfa = sfa->data_ptr<float>();
        g.sfa_stride_row = sfa->stride(0);
        g.sfa_stride_kb = sfa->stride(1);
        g.sfb = sfb->data_ptr<float>();
    }
    if (tile_group.has_value()) {
        TORCH_CHECK(tile_group->scalar_type() == at::kInt && tile_group->is_contiguous() && tile_group->numel() >= (M + 127) / 128, "bad tile_group");
        g.tile_group = tile_group->data_ptr<int32_t>();
    } else {
        TORCH_CHECK(G == 1, "several weight groups need tile_group");
    }
    if (a_ready_flags.has_value()) {
        TORCH_CHECK(a_ready_flags->scalar_type() == at::kLong, "flags must be int64");
        g.a_ready_flags = reinterpret_cast<const uint64_t*>(a_ready_flags->data_ptr<int64_t>());
        g.a_ready_value = static_cast<uint64_t>(a_ready_value);
        if (a_flag_of_tile.has_value()) g.a_flag_of_tile = a_flag_of_tile->data_ptr<int32_t>();
    }
    g.error = gemm_error_flag(a.get_device()).data_ptr<int>();
    if (report_to != nullptr) {
        // a pipeline wait that runs out is recorded in this buffer's status block (its limit applies too), so the
        // buffer's check_status() raises and poisons it like any other failed device wait
        report_to->check_status();
        const RankCtx c0 = report_to->ctx();
        g.status = c0.status;
        g.status_rank = c0.rank;
        g.timeout_ns = c0.timeout_ns;
    }
    const int sms = num_sms > 0 ? static_cast<int>(num_sms) : at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    cuda_check(ep::launch_gemm(g, sms, at::cuda::getCurrentCUDAStream()), "tcgen05 GEMM launch");
    return c;
}

// One-kernel all-gather + GEMM: `a_full` is the gathered [M, K] bf16 matrix inside the symmetric buffer (this rank
// has already written its own rows); copier CTAs of the GEMM kernel pull the other ranks' rows over NVLink while
// the tensor-core CTAs start on the local rows.  -> bf16 [M, N]
at::Tensor ag_gemm(ElasticBufferCore& core, int64_t off_full, int64_t M, int64_t K, const at::Tensor& b, int64_t num_sms, int64_t num_copy_ctas) {
    TORCH_CHECK(b.is_cuda() && b.dim() == 2 && b.is_contiguous() && b.scalar_type() == at::kBFloat16 && b.size(1) == K, "B must be contiguous bf16 [N, K]");
    const int64_t N = b.size(0);
    at::Tensor a_full = core.view(off_full, {M, K}, {K, 1}, at::kBFloat16);
    at::Tensor c = at::empty({M, N}, b.options());
    GemmArgs g{};
    g.a = a_full.data_ptr();
    g.b = b.data_ptr();
    g.c = c.data_ptr();
    g.M = static_cast<int>(M);
    g.N = static_cast<int>(N);
    g.K = static_cast<int>(K);
    g.num_groups = 1;
    g.lda = K;
    g.ldb = K;
    g.ldc = N;
    g.error = gemm_error_flag(b.get_device()).data_ptr<int>();
    g.fuse = EP_GEMM_FUSE_ALL_GATHER;
    g.ctx = core.ctx();
    g.status = g.ctx.status;
    g.status_rank = g.ctx.rank;
    g.timeout_ns = g.ctx.timeout_ns;
    g.num_copy_ctas = static_cast<int>(num_copy_ctas);
    g.off_full = off_full;
    g.m_tile_offset = static_cast<int>(core.rank() * (M / 128 / core.num_ranks()));
    core.check_status();
    cuda_check(ep::launch_gemm(g, static_cast<int>(num_sms), at::cuda::getCurrentCUDAStream()), "all-gather GEMM launch");
    return c;
}

// One-kernel GEMM + reduce-scatter: partial = a [M, K_local] @ b [N, K_local]^T; the epilogue bulk-stores every row
// of the partial result into the slot of the rank that owns it; after a cross-GPU barrier the same kernel sums the
// R slots.  -> bf16 [M / R, N]
at::Tensor gemm_rs(ElasticBufferCore& core, const at::Tensor& a, const at::Tensor& b, int64_t off_slots, int64_t slot_set_bytes, int64_t num_sms) {
    TORCH_CHECK(a.is_cuda() && a.dim() == 2 && a.is_contiguous() && a.scalar_type() == at::kBFloat16, "A must be contiguous bf16 [M, K]");
    TORCH_CHECK(b.is_cuda() && b.dim() == 2 && b.is_contiguous() && b.scalar_type() == at::kBFloat16 && b.size(1) == a.size(1), "B must be contiguous bf16 [N, K]");
    const int64_t M = a.size(0), K = a.size(1), N = b.size(0), R = core.num_ranks();
    TORCH_CHECK(off_slots % 16 == 0 && slot_set_bytes >= M * N * 2 && off_slots + 2 * slot_set_bytes <= core.num_bytes(), "slot region too small");
    at::Tensor out = at::empty({M / R, N}, a.options());
    GemmArgs g{};
    g.a = a.data_ptr();
    g.b = b.data_ptr();
    g.c = out.data_ptr();
    g.M = static_cast<int>(M);
    g.N = static_cast<int>(N);
    g.K = static_cast<int>(K);
    g.num_groups = 1;
    g.lda = K;
    g.ldb = K;
    g.ldc = N;
    g.error = gemm_error_flag(a.get_device()).data_ptr<int>();
    g.fuse = EP_GEMM_FUSE_REDUCE_SCATTER;
    g.ctx = core.ctx();
    g.status = g.ctx.status;
    g.status_rank = g.ctx.rank;
    g.timeout_ns = g.ctx.timeout_ns;
    g.off_slots = off_slots;
    g.slot_set_bytes = slot_set_bytes;
    g.rs_out = out.data_ptr();
    // start with the tiles that belong to the next rank so that the ranks do not all write to the same owner at once
    g.m_tile_offset = static_cast<int>(((core.rank() + 1) % R) * (M / 128 / R));
    core.check_status();
    cuda_check(ep::launch_gemm(g, static_cast<int>(num_sms), at::cuda::getCurrentCUDAStream()), "GEMM reduce-scatter launch");
    return out;
}

// h [rows, 2I] bf16 (gate | up) -> (e4m3 [rows, I], fp32 scales [rows, I/128], optional bf16 activation)
std::vector<at::Tensor> swiglu_quant(const at::Tensor& h, bool keep_bf16) {
    TORCH_CHECK(h.is_cuda() && h.dim() == 2 && h.stride(1) == 1 && h.scalar_type() == at::kBFloat16 && h.size(1) % 32 == 0,
                "h must be bf16 [rows, 2 * I] with contiguous rows and I a multiple of 16");
    const int64_t rows = h.size(0), I = h.size(1) / 2;
    at::Tensor q = at::empty({rows, I}, h.options().dtype(at::kFloat8_e4m3fn));
    at::Tensor sf = at::empty({rows, (I + 127) / 128}, h.options().dtype(at::kFloat));
    at::Tensor act = keep_bf16 ? at::empty({rows, I}, h.options()) : at::Tensor();
    SwigluQuantArgs a{};
    a.h = h.data_ptr();
    a.ldh = h.stride(0);
    a.q = q.data_ptr();
    a.sf = sf.data_ptr<float>();
    a.sf_stride_row = sf.stride(0);
    a.sf_stride_col = 1;
    a.act_bf16 = keep_bf16 ? act.data_ptr() : nullptr;
    a.rows = static_cast<int>(rows);
    a.inter = static_cast<int>(I);
    cuda_check(ep::launch_swiglu_quant(a, at::cuda::getCurrentCUDAStream()), "swiglu launch");
    if (keep_bf16) return {q, sf, act};
    return {q, sf};
}

// Expand-layout bookkeeping in one launch -> (tile_group int32 [ceil(rows / 128)], valid_row bool [rows], seg_off int32 [G + 1]).
std::vector<at::Tensor> expert_segments(const at::Tensor& psum_ends, int64_t num_rows, int64_t alignment) {
    TORCH_CHECK(psum_ends.is_cuda() && psum_ends.is_contiguous() && psum_ends.scalar_type() == at::kInt && psum_ends.dim() == 1,
                "psum_ends must be a contiguous int32 vector on the device");
    TORCH_CHECK(num_rows >= 0 && num_rows < (int64_t(1) << 31) && alignment >= 128 && alignment % 128 == 0, "bad num_rows / alignment");
    const auto i32 = psum_ends.options();
    at::Tensor tile_group = at::empty({(num_rows + 127) / 128}, i32);
    at::Tensor valid = at::empty({num_rows}, i32.dtype(at::kBool));
    at::Tensor seg_off = at::empty({psum_ends.numel() + 1}, i32);
    ExpertSegmentsArgs a{};
    a.psum_ends = psum_ends.data_ptr<int32_t>();
    a.num_groups = static_cast<int>(psum_ends.numel());
    a.num_rows = static_cast<int>(num_rows);
    a.alignment = static_cast<int>(alignment);
    a.tile_group = tile_group.data_ptr<int32_t>();
    a.valid_row = reinterpret_cast<uint8_t*>(valid.data_ptr());
    a.seg_off = seg_off.data_ptr<int32_t>();
    cuda_check(ep::launch_expert_segments(a, at::cuda::getCurrentCUDAStream()), "expert_segments launch");
    return {tile_group, valid, seg_off};
}

// Numbers the (row, k) pairs of a non-expand dispatch inside their experts' 128-aligned segments
// -> (pos int32 [rows, K] (-1: no local expert), seg_end int32 [El]: end of the token rows of every segment).
std::vector<at::Tensor> local_expand_plan(const at::Tensor& recv_idx, const at::Tensor& seg_end_aligned) {
    TORCH_CHECK(recv_idx.is_cuda() && recv_idx.dim() == 2 && recv_idx.stride(1) == 1 &&
                    (recv_idx.scalar_type() == at::kLong || recv_idx.scalar_type() == at::kInt),
                "recv_idx must be int64 / int32 [rows, K] with contiguous rows");
    TORCH_CHECK(seg_end_aligned.is_cuda() && seg_end_aligned.is_contiguous() && seg_end_aligned.scalar_type() == at::kInt && seg_end_aligned.dim() == 1,
                "seg_end_aligned must be a contiguous int32 vector");
    const int64_t rows = recv_idx.size(0), K = recv_idx.size(1), El = seg_end_aligned.numel();
    TORCH_CHECK(rows * K < (int64_t(1) << 31), "too many (row, k) pairs");
    const auto i32 = seg_end_aligned.options();
    at::Tensor pos = at::full({rows, K}, -1, i32);
    at::Tensor seg_end = at::empty({El}, i32);
    LocalExpandPlanArgs a{};
    a.recv_idx = recv_idx.data_ptr();
    a.idx_is_64 = recv_idx.scalar_type() == at::kLong;
    a.idx_pitch = recv_idx.stride(0);
    a.num_rows = static_cast<int>(rows);
    a.num_topk = static_cast<int>(K);
    a.num_local_experts = static_cast<int>(El);
    a.seg_end_aligned = seg_end_aligned.data_ptr<int32_t>();
    a.pos = pos.data_ptr<int32_t>();
    a.seg_end = seg_end.data_ptr<int32_t>();
    // one CTA per ~4096 pairs, at most one per SM: every warp sums the counts of all warps before it
    a.num_ctas = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(148, (rows * K + 4095) / 4096)));
    at::Tensor scratch = at::empty({a.num_ctas * 9, El}, i32);
    a.warp_counts = scratch.data_ptr<int32_t>();
    a.cta_counts = a.warp_counts + static_cast<int64_t>(a.num_ctas) * 8 * El;
    cuda_check(ep::launch_local_expand_plan(a, at::cuda::getCurrentCUDAStream()), "local_expand_plan launch");
    return {pos, seg_end};
}

// Copies every received row (and its scales / weights) to its expert rows -> (rows_out [num_out, width], sf_out or none, w_out or none).
std::vector<at::Tensor> local_expand_copy(const at::Tensor& pos, const at::Tensor& x, int64_t num_out, const std::optional<at::Tensor>& sf,
                                          const std::optional<at::Tensor>& w) {
    TORCH_CHECK(pos.is_cuda() && pos.is_contiguous() && pos.scalar_type() == at::kInt && pos.dim() == 2, "pos must be contiguous int32 [rows, K]");
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1 && x.size(0) == pos.size(0), "x must be [rows, width] with contiguous rows");
    const int64_t row_bytes = x.size(1) * x.element_size();
    at::Tensor out = at::empty({num_out, x.size(1)}, x.options());
    LocalExpandCopyArgs a{};
    a.pos = pos.data_ptr<int32_t>();
    a.num_rows = static_cast<int>(pos.size(0));
    a.num_topk = static_cast<int>(pos.size(1));
    a.src = x.data_ptr();
    a.src_pitch = x.stride(0) * x.element_size();
    a.row_bytes = static_cast<int>(row_bytes);
    a.dst = out.data_ptr();
    at::Tensor sf_out, w_out;
    if (sf.has_value()) {
        TORCH_CHECK(sf->is_cuda() && sf->dim() == 2 && sf->scalar_type() == at::kFloat && sf->size(0) == x.size(0), "sf must be fp32 [rows, groups]");
        sf_out = at::empty({num_out, sf->size(1)}, sf->options());
        a.sf_src = sf->data_ptr<float>();
        a.sf_stride_row = sf->stride(0);
        a.sf_stride_col = sf->stride(1);
        a.sf_cols = static_cast<int>(sf->size(1));
        a.sf_dst = sf_out.data_ptr<float>();
    }
    if (w.has_value()) {
        TORCH_CHECK(w->is_cuda() && w->dim() == 2 && w->scalar_type() == at::kFloat && w->stride(1) == 1 && w->size(0) == x.size(0) &&
                        w->size(1) == pos.size(1), "w must be fp32 [rows, K] with contiguous rows");
        w_out = at::zeros({num_out}, w->options());
        a.w_src = w->data_ptr<float>();
        a.w_pitch = w->stride(0);
        a.w_dst = w_out.data_ptr<float>();
    }
    cuda_check(ep::launch_local_expand_copy(a, at::cuda::getCurrentCUDAStream()), "local_expand_copy launch");
    std::vector<at::Tensor> res{out};
    if (sf.has_value()) res.push_back(sf_out);
    if (w.has_value()) res.push_back(w_out);
    return res;
}

// out[row] = sum_k (w[pos[row, k]] *) y[pos[row, k]] in fp32, rounded once to bf16; `out` may be given (e.g. a combine input region).
at::Tensor local_reduce(const at::Tensor& pos, const at::Tensor& y, const std::optional<at::Tensor>& w, const std::optional<at::Tensor>& out) {
    TORCH_CHECK(pos.is_cuda() && pos.is_contiguous() && pos.scalar_type() == at::kInt && pos.dim() == 2, "pos must be contiguous int32 [rows, K]");
    TORCH_CHECK(y.is_cuda() && y.is_contiguous() && y.dim() == 2 && y.scalar_type() == at::kBFloat16 && y.size(1) % 8 == 0,
                "y must be contiguous bf16 [expert rows, cols] with cols a multiple of 8");
    at::Tensor res = out.has_value() ? *out : at::empty({pos.size(0), y.size(1)}, y.options());
    TORCH_CHECK(res.is_cuda() && res.is_contiguous() && res.scalar_type() == at::kBFloat16 && res.size(0) == pos.size(0) && res.size(1) == y.size(1),
                "out must be contiguous bf16 [rows, cols]");
    LocalReduceArgs a{};
    a.pos = pos.data_ptr<int32_t>();
    a.num_rows = static_cast<int>(pos.size(0));
    a.num_topk = static_cast<int>(pos.size(1));
    a.src = y.data_ptr();
    a.cols = static_cast<int>(y.size(1));
    if (w.has_value()) {
        TORCH_CHECK(w->is_cuda() && w->is_contiguous() && w->dim() == 1 && w->scalar_type() == at::kFloat && w->size(0) == y.size(0),
                    "w must be contiguous fp32 [expert rows]");
        a.w = w->data_ptr<float>();
    }
    a.dst = res.data_ptr();
    cuda_check(ep::launch_local_reduce(a, at::cuda::getCurrentCUDAStream()), "local_reduce launch");
    return res;
}

// Weight gradients of a grouped layer: out[e] = a_t[:, k0:k1] @ b_t[:, k0:k1]^T with (k0, k1) = k_off[e], k_off[e + 1]
// (a_t [M, K_total], b_t [N, K_total] bf16, K = rows of the expert segment; k_off int32 [G + 1], multiples of 64).
at::Tensor gemm_kgrouped(const at::Tensor& a_t, const at::Tensor& b_t, const at::Tensor& k_off, int64_t num_sms) {
    TORCH_CHECK(a_t.is_cuda() && a_t.dim() == 2 && a_t.is_contiguous() && a_t.scalar_type() == at::kBFloat16, "a_t must be contiguous bf16 [M, K]");
    TORCH_CHECK(b_t.is_cuda() && b_t.dim() == 2 && b_t.is_contiguous() && b_t.scalar_type() == at::kBFloat16 && b_t.size(1) == a_t.size(1),
                "b_t must be contiguous bf16 [N, K]");
    TORCH_CHECK(k_off.is_cuda() && k_off.scalar_type() == at::kInt && k_off.is_contiguous() && k_off.numel() >= 2, "k_off must be int32 [G + 1]");
    const int64_t M = a_t.size(0), N = b_t.size(0), K = a_t.size(1), G = k_off.numel() - 1;
    at::Tensor c = at::empty({G, M, N}, a_t.options());
    GemmArgs g{};
    g.a = a_t.data_ptr();
    g.b = b_t.data_ptr();
    g.c = c.data_ptr();
    g.M = static_cast<int>(M);
    g.N = static_cast<int>(N);
    g.K = static_cast<int>(K);
    g.num_groups = static_cast<int>(G);
    g.lda = K;
    g.ldb = K;
    g.ldc = N;
    g.k_group_off = k_off.data_ptr<int32_t>();
    g.error = gemm_error_flag(a_t.get_device()).data_ptr<int>();
    const int sms = num_sms > 0 ? static_cast<int>(num_sms) : at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    cuda_check(ep::launch_gemm(g, sms, at::cuda::getCurrentCUDAStream()), "K-grouped tcgen05 GEMM launch");
    return c;
}

const uint8_t* valid_ptr(const at::Tensor& valid, int64_t rows) {
    TORCH_CHECK(valid.is_cuda() && valid.is_contiguous() && valid.numel() == rows && (valid.scalar_type() == at::kBool || valid.scalar_type() == at::kByte),
                "valid must be a bool / uint8 tensor with one entry per row");
    return reinterpret_cast<const uint8_t*>(valid.data_ptr());
}

// Backward of the weighted combine at the expert rows: (g * w [rows, H], its transpose [H, rows], sum(g * y) per row)
std::vector<at::Tensor> moe_bwd_prep(const at::Tensor& g_rows, const at::Tensor& y, const at::Tensor& w, const at::Tensor& valid) {
    TORCH_CHECK(g_rows.is_cuda() && g_rows.dim() == 2 && g_rows.is_contiguous() && g_rows.scalar_type() == at::kBFloat16, "g must be contiguous bf16 [rows, H]");
    TORCH_CHECK(y.is_contiguous() && y.scalar_type() == at::kBFloat16 && y.sizes() == g_rows.sizes(), "y must match g");
    const int64_t rows = g_rows.size(0), H = g_rows.size(1);
    TORCH_CHECK(w.is_contiguous() && w.scalar_type() == at::kFloat && w.numel() == rows, "w must be fp32 [rows]");
    at::Tensor out = at::empty({rows, H}, g_rows.options()), out_t = at::empty({H, rows}, g_rows.options());
    at::Tensor dot = at::empty({static_cast<int64_t>(ep::moe_bwd_prep_col_blocks(static_cast<int>(H))), rows}, g_rows.options().dtype(at::kFloat));
    MoeBwdArgs a{};
    a.op = EP_MOE_BWD_PREP;
    a.rows = static_cast<int>(rows);
    a.cols = static_cast<int>(H);
    a.valid = valid_ptr(valid, rows);
    a.g = g_rows.data_ptr();
    a.y = y.data_ptr();
    a.w = w.data_ptr<float>();
    a.out = out.data_ptr();
    a.out_t = out_t.data_ptr();
    a.row_dot = dot.data_ptr<float>();
    cuda_check(ep::launch_moe_bwd(a, at::cuda::getCurrentCUDAStream()), "MoE backward prep launch");
    return {out, out_t, dot.sum(0)};
}

// Backward of SwiGLU: (d_h [rows, 2I], d_h^T [2I, rows], activation^T [I, rows]).  With `row_weight` [rows] the incoming
// gradient is multiplied by it first and a fourth result, sum_i d_act[row, i] * activation[row, i] (the gradient of the
// row weight), is returned.
std::vector<at::Tensor> swiglu_bwd(const at::Tensor& d_act, const at::Tensor& h, const at::Tensor& valid, const std::optional<at::Tensor>& row_weight) {
    TORCH_CHECK(d_act.is_cuda() && d_act.dim() == 2 && d_act.is_contiguous() && d_act.scalar_type() == at::kBFloat16, "d_act must be contiguous bf16 [rows, I]");
    const int64_t rows = d_act.size(0), I = d_act.size(1);
    TORCH_CHECK(h.is_contiguous() && h.scalar_type() == at::kBFloat16 && h.dim() == 2 && h.size(0) == rows && h.size(1) == 2 * I, "h must be bf16 [rows, 2I]");
    at::Tensor out = at::empty({rows, 2 * I}, h.options()), out_t = at::empty({2 * I, rows}, h.options()), act_t = at::empty({I, rows}, h.options());
    at::Tensor dot;
    MoeBwdArgs a{};
    a.op = EP_MOE_BWD_SWIGLU;
    a.rows = static_cast<int>(rows);
    a.cols = static_cast<int>(I);
    a.valid = valid_ptr(valid, rows);
    a.g = d_act.data_ptr();
    a.y = h.data_ptr();
    a.out = out.data_ptr();
    a.out_t = out_t.data_ptr();
    a.out2_t = act_t.data_ptr();
    if (row_weight.has_value()) {
        TORCH_CHECK(row_weight->is_cuda() && row_weight->is_contiguous() && row_weight->scalar_type() == at::kFloat && row_weight->numel() == rows,
                    "row_weight must be fp32 [rows]");
        dot = at::empty({I / 64, rows}, h.options().dtype(at::kFloat));
        a.w = row_weight->data_ptr<float>();
        a.row_dot = dot.data_ptr<float>();
    }
    cuda_check(ep::launch_moe_bwd(a, at::cuda::getCurrentCUDAStream()), "SwiGLU backward launch");
    if (row_weight.has_value()) return {out, out_t, act_t, dot.sum(0)};
    return {out, out_t, act_t};
}

// (g * w)^T [H, rows] in bf16 (padding rows zero): the transposed operand of the down-projection weight gradient
at::Tensor weighted_transpose(const at::Tensor& g_rows, const at::Tensor& w, const at::Tensor& valid) {
    TORCH_CHECK(g_rows.is_cuda() && g_rows.dim() == 2 && g_rows.is_contiguous() && g_rows.scalar_type() == at::kBFloat16, "g must be contiguous bf16 [rows, H]");
    const int64_t rows = g_rows.size(0), H = g_rows.size(1);
    TORCH_CHECK(w.is_contiguous() && w.scalar_type() == at::kFloat && w.numel() == rows, "w must be fp32 [rows]");
    at::Tensor out_t = at::empty({H, rows}, g_rows.options());
    MoeBwdArgs a{};
    a.op = EP_MOE_BWD_PREP;
    a.rows = static_cast<int>(rows);
    a.cols = static_cast<int>(H);
    a.valid = valid_ptr(valid, rows);
    a.g = g_rows.data_ptr();
    a.w = w.data_ptr<float>();
    a.out_t = out_t.data_ptr();
    cuda_check(ep::launch_moe_bwd(a, at::cuda::getCurrentCUDAStream()), "weighted transpose launch");
    return out_t;
}

// (q e4m3 [rows, H], scales per (row, 128 channels), any strides) -> bf16 (q * scale)^T [H, rows]
at::Tensor dequant_transpose(const at::Tensor& q, const at::Tensor& sf, const at::Tensor& valid) {
    TORCH_CHECK(q.is_cuda() && q.dim() == 2 && q.is_contiguous() && q.scalar_type() == at::kFloat8_e4m3fn, "q must be contiguous e4m3 [rows, H]");
    const int64_t rows = q.size(0), H = q.size(1);
    TORCH_CHECK(sf.scalar_type() == at::kFloat && sf.dim() == 2 && sf.size(0) >= rows && sf.size(1) == (H + 127) / 128, "bad scales");
    at::Tensor out_t = at::empty({H, rows}, q.options().dtype(at::kBFloat16));
    MoeBwdArgs a{};
    a.op = EP_MOE_BWD_DEQUANT_T;
    a.rows = static_cast<int>(rows);
    a.cols = static_cast<int>(H);
    a.valid = valid_ptr(valid, rows);
    a.y = q.data_ptr();
    a.w = sf.data_ptr<float>();
    a.sf_stride_row = sf.stride(0);
    a.sf_stride_col = sf.stride(1);
    a.out_t = out_t.data_ptr();
    cuda_check(ep::launch_moe_bwd(a, at::cuda::getCurrentCUDAStream()), "dequant-transpose launch");
    return out_t;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "Blackwell-native expert-parallel communication runtime";
    m.def("get_platform", [] { return std::string("cuda-sm100a"); });
    m.def("get_elastic_buffer_alignment", [] { return static_cast<int64_t>(EP_BUFFER_ALIGNMENT); });
    m.def("get_workspace_bytes", [] { return static_cast<int64_t>(EP_WORKSPACE_BYTES); });
    m.attr("MAX_RANKS") = EP_MAX_RANKS;
    m.attr("MAX_EXPERTS") = EP_MAX_EXPERTS;
    m.attr("MAX_TOPK") = EP_MAX_TOPK;

    py::register_exception<BufferError>(m, "BufferError", PyExc_RuntimeError);

    py::class_<MoeShape>(m, "MoeShape")
        .def(py::init<>())
        .def_readwrite("num_ranks", &MoeShape::num_ranks)
        .def_readwrite("num_max_tokens_per_rank", &MoeShape::num_max_tokens_per_rank)
        .def_readwrite("hidden", &MoeShape::hidden)
        .def_readwrite("num_topk", &MoeShape::num_topk)
        .def_readwrite("num_experts_hint", &MoeShape::num_experts_hint)
        .def_readwrite("expert_alignment", &MoeShape::expert_alignment)
        .def_readwrite("use_fp8_dispatch", &MoeShape::use_fp8_dispatch)
        .def_readwrite("enable_expand", &MoeShape::enable_expand)
        .def_readwrite("num_recv_slots", &MoeShape::num_recv_slots);
    py::class_<RecvSlot>(m, "RecvSlot")
        .def_readonly("x", &RecvSlot::x)
        .def_readonly("sf", &RecvSlot::sf)
        .def_readonly("idx", &RecvSlot::idx)
        .def_readonly("w", &RecvSlot::w)
        .def_readonly("meta", &RecvSlot::meta)
        .def_readonly("tail", &RecvSlot::tail);
    py::class_<RegionLayout>(m, "RegionLayout")
        .def_readonly("capacity_rows", &RegionLayout::capacity_rows)
        .def_readonly("x_row_bytes", &RegionLayout::x_row_bytes)
        .def_readonly("sf_cols", &RegionLayout::sf_cols)
        .def_readonly("tail_bytes", &RegionLayout::tail_bytes)
        .def_readonly("sf_row_bytes", &RegionLayout::sf_row_bytes)
        .def_readonly("num_recv_slots", &RegionLayout::num_recv_slots)
        .def("slot", [](const RegionLayout& r, int i) {
            TORCH_CHECK(i >= 0 && i < r.num_recv_slots, "slot index out of range");
            return r.slots[i];
        })
        .def("combine_x", [](const RegionLayout& r, int i) { return r.combine_x[i & 1]; })
        .def("combine_w", [](const RegionLayout& r, int i) { return r.combine_w[i & 1]; })
        .def_readonly("extra", &RegionLayout::extra)
        .def_readonly("moe_bytes", &RegionLayout::moe_bytes);
    m.def("plan_regions", &plan_regions);
    m.def("calculate_elastic_buffer_size", [](const MoeShape& s) { return plan_regions(s).moe_bytes; });

    py::class_<DispatchCall>(m, "DispatchCall")
        .def(py::init<>())
        .def_readwrite("x", &DispatchCall::x)
        .def_readwrite("sf", &DispatchCall::sf)
        .def_readwrite("topk_idx", &DispatchCall::topk_idx)
        .def_readwrite("topk_weights", &DispatchCall::topk_weights)
        .def_readwrite("stats", &DispatchCall::stats)
        .def_readwrite("lane_src", &DispatchCall::lane_src)
        .def_readwrite("plan", &DispatchCall::plan)
        .def_readwrite("psum_rank", &DispatchCall::psum_rank)
        .def_readwrite("psum_expert", &DispatchCall::psum_expert)
        .def_readwrite("recv_per_expert", &DispatchCall::recv_per_expert)
        .def_readwrite("num_experts", &DispatchCall::num_experts)
        .def_readwrite("expert_alignment", &DispatchCall::expert_alignment)
        .def_readwrite("num_max_tokens", &DispatchCall::num_max_tokens)
        .def_readwrite("quantize", &DispatchCall::quantize)
        .def_readwrite("do_expand", &DispatchCall::do_expand)
        .def_readwrite("cached", &DispatchCall::cached)
        .def_readwrite("off_recv_x", &DispatchCall::off_recv_x)
        .def_readwrite("off_recv_sf", &DispatchCall::off_recv_sf)
        .def_readwrite("off_recv_idx", &DispatchCall::off_recv_idx)
        .def_readwrite("off_recv_w", &DispatchCall::off_recv_w)
        .def_readwrite("off_recv_meta", &DispatchCall::off_recv_meta)
        .def_readwrite("sf_stride_row", &DispatchCall::sf_stride_row)
        .def_readwrite("sf_stride_col", &DispatchCall::sf_stride_col)
        .def_readwrite("recv_capacity_rows", &DispatchCall::recv_capacity_rows)
        .def_readwrite("prof", &DispatchCall::prof)
        .def_readwrite("side_packed", &DispatchCall::side_packed)
        .def_readwrite("tail_bytes", &DispatchCall::tail_bytes)
        .def_readwrite("tail_off_w", &DispatchCall::tail_off_w)
        .def_readwrite("tail_off_meta", &DispatchCall::tail_off_meta)
        .def_readwrite("off_recv_tail", &DispatchCall::off_recv_tail)
        .def_readwrite("tail_pitch", &DispatchCall::tail_pitch)
        .def_readwrite("do_zero_padding", &DispatchCall::do_zero_padding)
        .def_readwrite("tune_warps", &DispatchCall::tune_warps)
        .def_readwrite("tune_stages", &DispatchCall::tune_stages);
    py::class_<CombineCall>(m, "CombineCall")
        .def(py::init<>())
        .def_readwrite("off_x", &CombineCall::off_x)
        .def_readwrite("off_w", &CombineCall::off_w)
        .def_readwrite("w_cols", &CombineCall::w_cols)
        .def_readwrite("plan", &CombineCall::plan)
        .def_readwrite("lane_src", &CombineCall::lane_src)
        .def_readwrite("mul_weights", &CombineCall::mul_weights)
        .def_readwrite("bias0", &CombineCall::bias0)
        .def_readwrite("bias1", &CombineCall::bias1)
        .def_readwrite("out", &CombineCall::out)
        .def_readwrite("out_w", &CombineCall::out_w)
        .def_readwrite("hidden", &CombineCall::hidden)
        .def_readwrite("prof", &CombineCall::prof);

    py::class_<ElasticBufferCore>(m, "ElasticBuffer")
        .def(py::init<int, int, int64_t, double, double, int64_t, bool>(), py::arg("rank"), py::arg("num_ranks"), py::arg("num_bytes"),
             py::arg("gpu_timeout_secs") = 100.0, py::arg("cpu_timeout_secs") = 300.0, py::arg("num_cpu_bytes") = 0,
             py::arg("use_vmm") = false)
        .def("finish_export", &ElasticBufferCore::finish_export)
        .def("uses_vmm", &ElasticBufferCore::uses_vmm)
        .def("num_cpu_bytes", &ElasticBufferCore::num_cpu_bytes)
        .def("get_local_cpu_segment_name", &ElasticBufferCore::get_local_cpu_segment_name)
        .def("open_cpu_peers", &ElasticBufferCore::open_cpu_peers)
        .def("unlink_cpu_segment_name", &ElasticBufferCore::unlink_cpu_segment_name)
        .def("cpu_segment_write", &ElasticBufferCore::cpu_segment_write)
        .def("get_local_ipc_handle", &ElasticBufferCore::get_local_ipc_handle)
        .def("open_peers", [](ElasticBufferCore& b, const std::vector<py::bytes>& handles) {
            std::vector<std::string> hs;
            for (const auto& h : handles) hs.push_back(static_cast<std::string>(h));
            b.open_peers(hs);
        })
        .def_static("link_local", &ElasticBufferCore::link_local)
        .def("destroy", &ElasticBufferCore::destroy)
        .def("rank", &ElasticBufferCore::rank)
        .def("num_ranks", &ElasticBufferCore::num_ranks)
        .def("num_bytes", &ElasticBufferCore::num_bytes)
        .def("state", &ElasticBufferCore::state)
        .def("generation", &ElasticBufferCore::generation)
        .def("set_gpu_timeout", &ElasticBufferCore::set_gpu_timeout)
        .def("view", &ElasticBufferCore::view)
        .def("read_status", &ElasticBufferCore::read_status)
        .def("check_status", &ElasticBufferCore::check_status)
        .def("wait_recv_counts", &ElasticBufferCore::wait_recv_counts)
        .def("dispatch", &ElasticBufferCore::dispatch)
        .def("combine", &ElasticBufferCore::combine)
        .def("barrier", &ElasticBufferCore::barrier, py::arg("channel") = static_cast<int>(EP_CH_BARRIER))
        .def("peer_copy", &ElasticBufferCore::peer_copy)
        .def("signal_and_wait_memops", &ElasticBufferCore::signal_and_wait_memops)
        .def_static("engram_fetch_group", &ElasticBufferCore::engram_fetch_group)
        .def("wait_flag_test", &ElasticBufferCore::wait_flag_test)
        .def_static("dispatch_group", &ElasticBufferCore::dispatch_group)
        .def_static("combine_group", &ElasticBufferCore::combine_group)
        .def_static("barrier_group", &ElasticBufferCore::barrier_group, py::arg("group"), py::arg("channel") = static_cast<int>(EP_CH_BARRIER))
        .def_static("wait_flag_test_group", &ElasticBufferCore::wait_flag_test_group);

    py::class_<LLDispatchCall>(m, "LLDispatchCall")
        .def(py::init<>())
        .def_readwrite("x", &LLDispatchCall::x)
        .def_readwrite("topk_idx", &LLDispatchCall::topk_idx)
        .def_readwrite("num_experts", &LLDispatchCall::num_experts)
        .def_readwrite("num_max_tokens", &LLDispatchCall::num_max_tokens)
        .def_readwrite("use_fp8", &LLDispatchCall::use_fp8)
        .def_readwrite("round_scale", &LLDispatchCall::round_scale)
        .def_readwrite("use_ue8m0", &LLDispatchCall::use_ue8m0)
        .def_readwrite("phases", &LLDispatchCall::phases)
        .def_readwrite("off_slab0", &LLDispatchCall::off_slab0)
        .def_readwrite("off_slab1", &LLDispatchCall::off_slab1)
        .def_readwrite("msg_bytes", &LLDispatchCall::msg_bytes)
        .def_readwrite("packed_x", &LLDispatchCall::packed_x)
        .def_readwrite("packed_sf", &LLDispatchCall::packed_sf)
        .def_readwrite("packed_src_info", &LLDispatchCall::packed_src_info)
        .def_readwrite("layout_range", &LLDispatchCall::layout_range)
        .def_readwrite("packed_count", &LLDispatchCall::packed_count)
        .def_readwrite("stats", &LLDispatchCall::stats)
        .def_readwrite("wait_stats", &LLDispatchCall::wait_stats)
        .def_readwrite("prof", &LLDispatchCall::prof)
        .def_readwrite("mask", &LLDispatchCall::mask)
        .def_readwrite("shrink", &LLDispatchCall::shrink);
    py::class_<LLCombineCall>(m, "LLCombineCall")
        .def(py::init<>())
        .def_readwrite("x", &LLCombineCall::x)
        .def_readwrite("topk_idx", &LLCombineCall::topk_idx)
        .def_readwrite("topk_weights", &LLCombineCall::topk_weights)
        .def_readwrite("src_info", &LLCombineCall::src_info)
        .def_readwrite("layout_range", &LLCombineCall::layout_range)
        .def_readwrite("out", &LLCombineCall::out)
        .def_readwrite("num_experts", &LLCombineCall::num_experts)
        .def_readwrite("num_max_tokens", &LLCombineCall::num_max_tokens)
        .def_readwrite("phases", &LLCombineCall::phases)
        .def_readwrite("off_slab0", &LLCombineCall::off_slab0)
        .def_readwrite("off_slab1", &LLCombineCall::off_slab1)
        .def_readwrite("wait_stats", &LLCombineCall::wait_stats)
        .def_readwrite("prof", &LLCombineCall::prof)
        .def_readwrite("mask", &LLCombineCall::mask)
        .def_readwrite("shrink", &LLCombineCall::shrink)
        .def_readwrite("use_logfmt", &LLCombineCall::use_logfmt);
    m.def("ll_dispatch_group", &ll_dispatch_group);
    m.def("ll_combine_group", &ll_combine_group);
    m.def("ll_message_bytes", &ll_message_bytes);
    m.def("get_low_latency_rdma_size_hint", &ll_size_hint, py::arg("num_max_dispatch_tokens_per_rank"), py::arg("hidden"),
          py::arg("num_ranks"), py::arg("num_experts"), py::arg("num_topk") = 8);
    m.def("reduce_slots", [](const at::Tensor& slots, at::Tensor out) {
        TORCH_CHECK(slots.is_cuda() && slots.is_contiguous() && out.is_contiguous() && slots.dim() >= 1 &&
                        slots.scalar_type() == out.scalar_type() && slots.numel() == slots.size(0) * out.numel(),
                    "slots must be [num_slots, ...] matching out");
        TORCH_CHECK(slots.scalar_type() == at::kBFloat16 || slots.scalar_type() == at::kFloat, "bf16 or fp32 only");
        ReduceSlotsArgs a{};
        a.slots = slots.data_ptr();
        a.out = out.data_ptr();
        a.n = out.numel();
        a.num_slots = static_cast<int>(slots.size(0));
        a.is_bf16 = slots.scalar_type() == at::kBFloat16;
        cuda_check(ep::launch_reduce_slots(a, at::cuda::getCurrentCUDAStream()), "reduce launch");
    });
    m.attr("CH_BARRIER") = static_cast<int>(EP_CH_BARRIER);
    m.attr("CH_AGRS") = static_cast<int>(EP_CH_AGRS);
    m.attr("CH_PP") = static_cast<int>(EP_CH_PP);
    m.attr("CH_ENGRAM") = static_cast<int>(EP_CH_ENGRAM);
    m.def("gemm_nt", &gemm_nt, py::arg("a"), py::arg("b"), py::arg("sfa") = py::none(), py::arg("sfb") = py::none(),
          py::arg("tile_group") = py::none(), py::arg("out") = py::none(), py::arg("num_sms") = 0, py::arg("a_ready_flags") = py::none(),
          py::arg("a_ready_value") = 0, py::arg("a_flag_of_tile") = py::none(), py::arg("report_to") = nullptr);
    m.def("ag_gemm", &ag_gemm);
    m.def("gemm_rs", &gemm_rs);
    m.def("local_expand_plan", &local_expand_plan, py::arg("recv_idx"), py::arg("seg_end_aligned"));
    m.def("local_expand_copy", &local_expand_copy, py::arg("pos"), py::arg("x"), py::arg("num_out"), py::arg("sf") = py::none(),
          py::arg("w") = py::none());
    m.def("local_reduce", &local_reduce, py::arg("pos"), py::arg("y"), py::arg("w") = py::none(), py::arg("out") = py::none());
    m.def("expert_segments", &expert_segments, py::arg("psum_ends"), py::arg("num_rows"), py::arg("alignment") = 128);
    m.def("swiglu_quant", &swiglu_quant, py::arg("h"), py::arg("keep_bf16") = false);
    m.def("gemm_kgrouped", &gemm_kgrouped, py::arg("a_t"), py::arg("b_t"), py::arg("k_off"), py::arg("num_sms") = 0);
    m.def("moe_bwd_prep", &moe_bwd_prep);
    m.def("swiglu_bwd", &swiglu_bwd, py::arg("d_act"), py::arg("h"), py::arg("valid"), py::arg("row_weight") = py::none());
    m.def("weighted_transpose", &weighted_transpose);
    m.def("dequant_transpose", &dequant_transpose);
    m.def("gemm_error", [](int device) { return gemm_error_flag(device).item<int>(); });
    m.def("get_dispatch_layout", &get_dispatch_layout);
    m.def("per_token_cast_to_fp8", &per_token_cast_to_fp8, py::arg("x"), py::arg("round_scale") = false,
          py::arg("use_ue8m0") = false);
}
