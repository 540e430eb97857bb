// Host side of the low-latency dispatch / combine kernels: argument validation and launch.
// Parity: the low-latency methods of csrc/legacy/buffer.hpp:1431-1748 and the buffer layout of
// csrc/legacy/config.hpp:122-188.
#pragma once
#include "elastic_buffer.hpp"

namespace ep_host {

struct LLDispatchCall {
    at::Tensor x;                 // [T, H] bf16
    at::Tensor topk_idx;          // [T, K]
    int64_t num_experts = 0, num_max_tokens = 0;
    bool use_fp8 = true, round_scale = false, use_ue8m0 = false;
    int64_t phases = EP_LL_SEND | EP_LL_RECV;
    int64_t off_slab0 = 0, off_slab1 = 0, msg_bytes = 0;
    at::Tensor packed_x, packed_src_info, layout_range, packed_count;
    OptTensor packed_sf, stats, wait_stats, mask, prof;
    bool shrink = false;
};

struct LLCombineCall {
    at::Tensor x;                 // [E_local, R*M, H] bf16
    at::Tensor topk_idx, topk_weights, src_info, layout_range, out;
    int64_t num_experts = 0, num_max_tokens = 0;
    int64_t phases = EP_LL_SEND | EP_LL_RECV;
    int64_t off_slab0 = 0, off_slab1 = 0;
    OptTensor wait_stats, mask, prof;
    bool shrink = false;
    bool use_logfmt = false;      // rows travel as 10-bit logarithmic codes (hidden must be a multiple of 128)
};

inline int64_t ll_message_bytes(int64_t hidden) {
    // header + the larger of {e4m3 payload + fp32 scales, bf16 payload}
    const int64_t fp8 = hidden + (hidden + 127) / 128 * 4, bf16 = hidden * 2;
    return align_up(16 + (fp8 > bf16 ? fp8 : bf16), 16);
}

// bytes of the low-latency regions: two buffer sets of {dispatch slab, combine slab}
inline int64_t ll_size_hint(int64_t num_max_tokens, int64_t hidden, int64_t num_ranks, int64_t num_experts, int64_t num_topk) {
    const int64_t dispatch = checked_mul(checked_mul(num_experts, num_max_tokens), ll_message_bytes(hidden));
    const int64_t combine = checked_mul(checked_mul(num_max_tokens, num_topk), hidden * 2);
    (void)num_ranks;
    return align_up(2 * (align_up(dispatch, 1024) + align_up(combine, 1024)), EP_BUFFER_ALIGNMENT);
}

inline LLDispatchArgs make_ll_dispatch_args(ElasticBufferCore& core, const LLDispatchCall& c) {
    LLDispatchArgs a{};
    a.ctx = core.ctx();
    const int R = a.ctx.num_ranks;
    TORCH_CHECK(c.x.is_cuda() && c.x.is_contiguous() && c.x.dim() == 2 && c.x.scalar_type() == at::kBFloat16,
                "x must be contiguous bf16 [T, H]");
    const int64_t T = c.x.size(0), H = c.x.size(1), K = c.topk_idx.size(1);
    TORCH_CHECK(H % 16 == 0 && T <= c.num_max_tokens && c.num_max_tokens < (1 << 20), "bad low-latency shape");
    TORCH_CHECK(c.topk_idx.is_contiguous() && c.topk_idx.size(0) == T && K <= EP_MAX_TOPK && K <= 16 &&
                    (c.topk_idx.scalar_type() == at::kLong || c.topk_idx.scalar_type() == at::kInt),
                "topk_idx must be contiguous int64/int32 [T, K] with K <= 16");
    TORCH_CHECK(c.num_experts % R == 0 && c.num_experts <= EP_MAX_EXPERTS, "bad expert count");
    const int64_t El = c.num_experts / R, rows = static_cast<int64_t>(R) * c.num_max_tokens;
    const int64_t payload = c.use_fp8 ? H : 2 * H, G = (H + 127) / 128;
    TORCH_CHECK(c.msg_bytes % 16 == 0 && c.msg_bytes >= 16 + payload + (c.use_fp8 ? G * 4 : 0), "message size too small");
    const int64_t slab = El * rows * c.msg_bytes;
    for (int64_t off : {c.off_slab0, c.off_slab1})
        TORCH_CHECK(off >= static_cast<int64_t>(EP_WORKSPACE_BYTES) && off % 16 == 0 && off + slab <= core.num_bytes(),
                    "low-latency dispatch slab does not fit the symmetric buffer");
    TORCH_CHECK(c.packed_x.is_contiguous() && c.packed_x.numel() * c.packed_x.element_size() == El * rows * payload,
                "packed_x has the wrong size");
    TORCH_CHECK(c.packed_src_info.scalar_type() == at::kInt && c.packed_src_info.numel() == El * rows &&
                    c.layout_range.scalar_type() == at::kLong && c.layout_range.numel() == El * R &&
                    c.packed_count.scalar_type() == at::kInt && c.packed_count.numel() == El,
                "low-latency metadata tensors have the wrong size");
    if (c.use_fp8) TORCH_CHECK(c.packed_sf.has_value(), "fp8 dispatch needs a scale tensor");
    if (c.mask.has_value()) TORCH_CHECK(c.mask->scalar_type() == at::kInt && c.mask->numel() == R, "mask must be int32 [R]");
    if (c.wait_stats.has_value()) TORCH_CHECK(c.wait_stats->scalar_type() == at::kLong && c.wait_stats->numel() == R, "wait stats must be int64 [R]");
    a.x = c.x.data_ptr();
    a.topk_idx = c.topk_idx.data_ptr();
    a.idx_is_64 = c.topk_idx.scalar_type() == at::kLong;
    a.num_tokens = static_cast<int>(T);
    a.hidden = static_cast<int>(H);
    a.num_topk = static_cast<int>(K);
    a.num_experts = static_cast<int>(c.num_experts);
    a.num_max_tokens = static_cast<int>(c.num_max_tokens);
    a.use_fp8 = c.use_fp8;
    a.round_scale = c.round_scale;
    a.use_ue8m0 = c.use_ue8m0;
    a.phases = static_cast<int>(c.phases);
    a.off_slab[0] = c.off_slab0;
    a.off_slab[1] = c.off_slab1;
    a.msg_bytes = static_cast<int>(c.msg_bytes);
    a.packed_x = c.packed_x.data_ptr();
    a.packed_sf = c.packed_sf.has_value() ? c.packed_sf->data_ptr() : nullptr;
    a.packed_src_info = c.packed_src_info.data_ptr<int32_t>();
    a.layout_range = c.layout_range.data_ptr<int64_t>();
    a.packed_count = c.packed_count.data_ptr<int32_t>();
    a.stats = c.stats.has_value() ? c.stats->data_ptr<int32_t>() : nullptr;
    a.wait_stats = c.wait_stats.has_value() ? c.wait_stats->data_ptr<int64_t>() : nullptr;
    a.mask = c.mask.has_value() ? c.mask->data_ptr<int32_t>() : nullptr;
    a.shrink = c.shrink;
    if (c.prof.has_value()) {
        TORCH_CHECK(c.prof->scalar_type() == at::kLong && c.prof->numel() >= 8 && c.prof->is_cuda(), "prof must be int64 [8] on the GPU");
        a.prof = reinterpret_cast<uint64_t*>(c.prof->data_ptr<int64_t>());
    }
    return a;
}

inline LLCombineArgs make_ll_combine_args(ElasticBufferCore& core, const LLCombineCall& c) {
    LLCombineArgs a{};
    a.ctx = core.ctx();
    const int R = a.ctx.num_ranks;
    TORCH_CHECK(c.x.is_cuda() && c.x.is_contiguous() && c.x.dim() == 3 && c.x.scalar_type() == at::kBFloat16,
                "x must be contiguous bf16 [E_local, R * max_tokens, H]");
    const int64_t El = c.num_experts / R, H = c.x.size(2), T = c.topk_idx.size(0), K = c.topk_idx.size(1);
    TORCH_CHECK(c.x.size(0) == El && c.x.size(1) == R * c.num_max_tokens && H % 16 == 0, "x has the wrong shape");
    TORCH_CHECK(c.topk_idx.is_contiguous() && c.topk_weights.is_contiguous() && c.topk_weights.scalar_type() == at::kFloat &&
                    c.topk_weights.size(0) == T && c.topk_weights.size(1) == K && T <= c.num_max_tokens && K <= 16,
                "bad top-k tensors");
    TORCH_CHECK(c.src_info.scalar_type() == at::kInt && c.src_info.numel() == El * R * c.num_max_tokens &&
                    c.layout_range.scalar_type() == at::kLong && c.layout_range.numel() == El * R,
                "handle tensors have the wrong size");
    TORCH_CHECK(c.out.is_contiguous() && c.out.scalar_type() == at::kBFloat16 && c.out.size(0) == T && c.out.size(1) == H,
                "out must be contiguous bf16 [T, H]");
    const int64_t slab = c.num_max_tokens * K * H * 2;
    for (int64_t off : {c.off_slab0, c.off_slab1})
        TORCH_CHECK(off >= static_cast<int64_t>(EP_WORKSPACE_BYTES) && off % 16 == 0 && off + slab <= core.num_bytes(),
                    "low-latency combine slab does not fit the symmetric buffer");
    a.x = c.x.data_ptr();
    a.topk_idx = c.topk_idx.data_ptr();
    a.idx_is_64 = c.topk_idx.scalar_type() == at::kLong;
    a.topk_weights = c.topk_weights.data_ptr<float>();
    a.src_info = c.src_info.data_ptr<int32_t>();
    a.layout_range = c.layout_range.data_ptr<int64_t>();
    a.num_tokens = static_cast<int>(T);
    a.hidden = static_cast<int>(H);
    a.num_topk = static_cast<int>(K);
    a.num_experts = static_cast<int>(c.num_experts);
    a.num_max_tokens = static_cast<int>(c.num_max_tokens);
    a.phases = static_cast<int>(c.phases);
    a.off_slab[0] = c.off_slab0;
    a.off_slab[1] = c.off_slab1;
    a.out = c.out.data_ptr();
    a.wait_stats = c.wait_stats.has_value() ? c.wait_stats->data_ptr<int64_t>() : nullptr;
    a.mask = c.mask.has_value() ? c.mask->data_ptr<int32_t>() : nullptr;
    a.shrink = c.shrink;
    TORCH_CHECK(!c.use_logfmt || H % 128 == 0, "LogFMT coding needs a hidden size that is a multiple of 128");
    a.use_logfmt = c.use_logfmt;
    if (c.prof.has_value()) {
        TORCH_CHECK(c.prof->scalar_type() == at::kLong && c.prof->numel() >= 8 && c.prof->is_cuda(), "prof must be int64 [8] on the GPU");
        a.prof = reinterpret_cast<uint64_t*>(c.prof->data_ptr<int64_t>());
    }
    return a;
}

inline void ll_dispatch_group(const std::vector<ElasticBufferCore*>& group, const std::vector<LLDispatchCall>& calls, int num_sms) {
    TORCH_CHECK(group.size() == calls.size() && !group.empty(), "one call per buffer is required");
    std::vector<std::unique_ptr<OperationScope>> scopes;
    std::vector<LLDispatchArgs> args(group.size());
    for (size_t i = 0; i < group.size(); ++i) {
        scopes.push_back(std::make_unique<OperationScope>(group[i]->coordinator(), "low_latency_dispatch"));
        group[i]->check_status();
        args[i] = make_ll_dispatch_args(*group[i], calls[i]);
    }
    cuda_check(ep::launch_ll_dispatch(args.data(), static_cast<int>(args.size()), num_sms, at::cuda::getCurrentCUDAStream()),
               "low-latency dispatch launch");
    for (auto& s : scopes) s->commit();
}

inline void ll_combine_group(const std::vector<ElasticBufferCore*>& group, const std::vector<LLCombineCall>& calls, int num_sms) {
    TORCH_CHECK(group.size() == calls.size() && !group.empty(), "one call per buffer is required");
    std::vector<std::unique_ptr<OperationScope>> scopes;
    std::vector<LLCombineArgs> args(group.size());
    for (size_t i = 0; i < group.size(); ++i) {
        scopes.push_back(std::make_unique<OperationScope>(group[i]->coordinator(), "low_latency_combine"));
        group[i]->check_status();
        args[i] = make_ll_combine_args(*group[i], calls[i]);
    }
    cuda_check(ep::launch_ll_combine(args.data(), static_cast<int>(args.size()), num_sms, at::cuda::getCurrentCUDAStream()),
               "low-latency combine launch");
    for (auto& s : scopes) s->commit();
}

}  // namespace ep_host
