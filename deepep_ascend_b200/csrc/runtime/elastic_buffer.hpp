// Native core of ElasticBuffer: owns the symmetric memory, the status block and the operation coordinator,
// validates every call, fills the kernel argument structs and launches on the current CUDA stream.  The
// Python class of the same name adds process-group plumbing, stream/event control and handle objects.
//
// Every operation exists in two forms: a method (this process drives one GPU) and a static `*_group` function
// that takes the cores of several virtual ranks living on ONE device and runs them as a single cooperative
// launch, which is how the multi-rank protocols are tested on a single GPU.
// Parity: csrc/elastic/buffer.hpp:19-1346 (deep_ep::elastic::ElasticBuffer).
#pragma once
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <chrono>
#include <memory>
#include <optional>
#include <thread>
#include <vector>

#include "../kernels/api.h"
#include "coordinator.hpp"
#include "layout.hpp"
#include "symmetric.hpp"

namespace ep_host {

using OptTensor = std::optional<at::Tensor>;

struct DispatchCall {
    at::Tensor x;                  // [T, H] bf16 or float8_e4m3fn
    OptTensor sf;                  // [T, H/128] fp32 when x is fp8
    OptTensor topk_idx;            // [T, K] int64 / int32 (absent with a cached layout)
    OptTensor topk_weights;        // [T, K] fp32
    OptTensor stats;               // [E_local] int32 cumulative counters
    at::Tensor lane_src, plan;     // [T, K] int32 handle tensors (outputs, or inputs when cached)
    at::Tensor psum_rank, psum_expert, recv_per_expert;   // int32 handle tensors
    int64_t num_experts = 0;
    int64_t expert_alignment = 1;
    int64_t num_max_tokens = 0;
    bool quantize = false;
    bool do_expand = false;
    bool cached = false;
    int64_t off_recv_x = 0, off_recv_sf = 0, off_recv_idx = 0, off_recv_w = 0, off_recv_meta = 0;
    int64_t sf_stride_row = 0, sf_stride_col = 1;
    int64_t recv_capacity_rows = 0;
    OptTensor prof;               // int64 [8]: phase timestamps (profiling)
    bool side_packed = false;     // scales and a tail record {ids | weights | metadata} travel as bulk stores
    int64_t tail_bytes = 0, tail_off_w = 0, tail_off_meta = 0, off_recv_tail = 0;
    int64_t tail_pitch = 0;       // 0 = tail_bytes
    bool do_zero_padding = false;
    int64_t tune_warps = 0, tune_stages = 0;
};

struct CombineCall {
    int64_t off_x = 0, off_w = 0;
    int64_t w_cols = 0;
    at::Tensor plan, lane_src;     // [T, K] int32
    OptTensor mul_weights;         // [T, K] fp32
    OptTensor bias0, bias1;        // [T, H] bf16
    at::Tensor out;                // [T, H] bf16
    OptTensor out_w;               // [T, K] fp32
    int64_t hidden = 0;
    OptTensor prof;                // int64 [8]: phase timestamps of CTA 0 (profiling)
};

class ElasticBufferCore {
public:
    ElasticBufferCore(int rank, int num_ranks, int64_t num_bytes, double gpu_timeout_secs, double cpu_timeout_secs,
                      int64_t num_cpu_bytes = 0, bool use_vmm = false)
        : mem_(std::make_unique<SymmetricMemory>(rank, num_ranks, num_bytes, num_cpu_bytes, use_vmm)),
          gpu_timeout_ns_(static_cast<uint64_t>(gpu_timeout_secs * 1e9)),
          cpu_timeout_secs_(cpu_timeout_secs) {}

    ~ElasticBufferCore() {
        if (!mem_->released()) destroy();
    }

    // ------------------------------------------------------------------ set-up / tear-down
    py::bytes get_local_ipc_handle() { return py::bytes(mem_->export_handle()); }
    void open_peers(const std::vector<std::string>& handles) { mem_->open_peers(handles); }
    void finish_export() { mem_->finish_export(); }
    bool uses_vmm() const { return mem_->uses_vmm(); }
    static void link_local(const std::vector<ElasticBufferCore*>& group) {
        std::vector<SymmetricMemory*> mems;
        for (auto* g : group) mems.push_back(g->mem_.get());
        SymmetricMemory::link_local(mems);
    }
    void destroy() {
        if (!coord_.begin_destroy()) return;
        cudaDeviceSynchronize();
        coord_.end_destroy(mem_->release());
    }

    int rank() const { return mem_->rank(); }
    int num_ranks() const { return mem_->num_ranks(); }
    int64_t num_bytes() const { return mem_->bytes(); }
    std::string state() const { return to_string(coord_.state()); }
    uint64_t generation() const { return coord_.generation(); }
    void set_gpu_timeout(double secs) { gpu_timeout_ns_ = static_cast<uint64_t>(secs * 1e9); }

    // a tensor that aliases [offset, offset + bytes) of the local symmetric buffer
    at::Tensor view(int64_t offset, std::vector<int64_t> sizes, std::vector<int64_t> strides, at::ScalarType dtype) const {
        int64_t max_index = 0;
        for (size_t i = 0; i < sizes.size(); ++i) {
            if (sizes[i] == 0) { max_index = -1; break; }
            max_index += (sizes[i] - 1) * strides[i];
        }
        const int64_t end = offset + (max_index + 1) * static_cast<int64_t>(c10::elementSize(dtype));
        TORCH_CHECK(offset >= static_cast<int64_t>(EP_WORKSPACE_BYTES) && end <= mem_->bytes(),
                    "view [", offset, ", ", end, ") is outside the data area of the symmetric buffer");
        auto opts = at::TensorOptions().dtype(dtype).device(at::kCUDA, mem_->device());
        return at::from_blob(mem_->local() + offset, sizes, strides, [](void*) {}, opts);
    }

    // ------------------------------------------------------------------ status
    // (code, phase, peer, expected, observed, rank)
    std::vector<int64_t> read_status() const {
        const volatile uint64_t* st = mem_->status();
        return {static_cast<int64_t>(st[EP_STATUS_CODE]), static_cast<int64_t>(st[EP_STATUS_PHASE]),
                static_cast<int64_t>(st[EP_STATUS_PEER]), static_cast<int64_t>(st[EP_STATUS_EXPECTED]),
                static_cast<int64_t>(st[EP_STATUS_OBSERVED]), static_cast<int64_t>(st[EP_STATUS_RANK])};
    }
    // throws (and poisons the buffer) if any kernel reported a failed wait
    void check_status() {
        const volatile uint64_t* st = mem_->status();
        if (st[EP_STATUS_CODE] != EP_OK) {
            const std::string msg = describe_status(st);
            coord_.poison(msg);
            throw BufferError(msg);
        }
    }

    // Host side of do_cpu_sync: spin on the mapped counters of dispatch number `epoch` (1-based).
    // -> [num_recv, num_expanded, count of local expert 0, 1, ...]
    std::vector<int64_t> wait_recv_counts(int64_t num_local_experts) {
        const volatile uint64_t* st = mem_->status();
        const uint64_t epoch = dispatch_epoch_ & 0xffffffffull;
        const auto t0 = std::chrono::steady_clock::now();
        std::vector<int64_t> out(2 + num_local_experts);
        py::gil_scoped_release release;
        auto ready = [&](uint64_t w) { return (w >> 32) == epoch; };
        while (true) {
            bool all = ready(st[EP_STATUS_NUM_RECV]) && ready(st[EP_STATUS_NUM_EXPANDED]);
            for (int64_t j = 0; all && j < num_local_experts; ++j) all = ready(st[EP_STATUS_EXPERT_BASE + j]);
            if (all) break;
            if (st[EP_STATUS_CODE] != EP_OK) {
                const std::string msg = describe_status(st);
                coord_.poison(msg);
                throw BufferError(msg);
            }
            const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            if (waited > cpu_timeout_secs_) {
                coord_.poison("host timed out waiting for receive counts");
                throw BufferError("host timed out waiting for the receive counts of dispatch " + std::to_string(dispatch_epoch_));
            }
            std::this_thread::yield();
        }
        out[0] = static_cast<int64_t>(st[EP_STATUS_NUM_RECV] & 0xffffffffull);
        out[1] = static_cast<int64_t>(st[EP_STATUS_NUM_EXPANDED] & 0xffffffffull);
        for (int64_t j = 0; j < num_local_experts; ++j)
            out[2 + j] = static_cast<int64_t>(st[EP_STATUS_EXPERT_BASE + j] & 0xffffffffull);
        return out;
    }

    // ------------------------------------------------------------------ operations
    void dispatch(const DispatchCall& call, int num_sms) { dispatch_group({this}, {call}, num_sms); }
    void combine(const CombineCall& call, int num_sms) { combine_group({this}, {call}, num_sms); }
    void barrier(int channel) { barrier_group({this}, channel); }
    void wait_flag_test(int64_t expected) { wait_flag_test_group({this}, expected); }

    static void dispatch_group(const std::vector<ElasticBufferCore*>& group, const std::vector<DispatchCall>& calls,
                               int num_sms) {
        TORCH_CHECK(group.size() == calls.size() && !group.empty(), "one call per buffer is required");
        std::vector<std::unique_ptr<OperationScope>> scopes;
        std::vector<DispatchArgs> args(group.size());
        for (size_t i = 0; i < group.size(); ++i) {
            scopes.push_back(std::make_unique<OperationScope>(group[i]->coord_, "dispatch"));
            group[i]->check_status();
            args[i] = group[i]->make_dispatch_args(calls[i]);
            TORCH_CHECK(args[i].quantize == args[0].quantize && args[i].hidden == args[0].hidden &&
                            args[i].num_experts == args[0].num_experts && args[i].num_topk == args[0].num_topk &&
                            args[i].x_is_fp8 == args[0].x_is_fp8,
                        "all virtual ranks must use the same dispatch configuration");
        }
        auto stream = at::cuda::getCurrentCUDAStream();
        cuda_check(ep::launch_dispatch(args.data(), static_cast<int>(args.size()), num_sms, stream), "dispatch launch");
        for (size_t i = 0; i < group.size(); ++i) {
            group[i]->dispatch_epoch_ += 1;
            scopes[i]->commit();
        }
    }

    static void combine_group(const std::vector<ElasticBufferCore*>& group, const std::vector<CombineCall>& calls,
                              int num_sms) {
        TORCH_CHECK(group.size() == calls.size() && !group.empty(), "one call per buffer is required");
        std::vector<std::unique_ptr<OperationScope>> scopes;
        std::vector<CombineArgs> args(group.size());
        for (size_t i = 0; i < group.size(); ++i) {
            scopes.push_back(std::make_unique<OperationScope>(group[i]->coord_, "combine"));
            group[i]->check_status();
            args[i] = group[i]->make_combine_args(calls[i]);
            TORCH_CHECK(args[i].hidden == args[0].hidden && args[i].num_topk == args[0].num_topk,
                        "all virtual ranks must use the same combine configuration");
        }
        auto stream = at::cuda::getCurrentCUDAStream();
        cuda_check(ep::launch_combine(args.data(), static_cast<int>(args.size()), num_sms, stream), "combine launch");
        for (auto& s : scopes) s->commit();
    }

    static void barrier_group(const std::vector<ElasticBufferCore*>& group, int channel) {
        std::vector<std::unique_ptr<OperationScope>> scopes;
        std::vector<RankCtx> ctxs;
        for (auto* g : group) {
            scopes.push_back(std::make_unique<OperationScope>(g->coord_, "barrier"));
            g->check_status();
            ctxs.push_back(g->ctx());
        }
        cuda_check(ep::launch_barrier(ctxs.data(), static_cast<int>(ctxs.size()), channel, at::cuda::getCurrentCUDAStream()),
                   "barrier launch");
        for (auto& s : scopes) s->commit();
    }

    // Cross-GPU completion signal without any SM: after everything queued so far on the current stream (e.g. the peer copies
    // of an all-gather), write this rank's next sequence number into every peer's host-flag word for `channel` and make the
    // stream wait until every peer's word in the LOCAL buffer has reached the same number (stream memory operations, what
    // the reference does with cuStreamBatchMemOp, csrc/kernels/backend/cuda_driver.cu:12-52).  Returns false when the driver
    // refuses the operations, in which case nothing was queued and the caller uses the signal kernel instead.
    bool signal_and_wait_memops(int channel) {
        TORCH_CHECK(channel >= 0 && channel < EP_NUM_CHANNELS, "bad channel");
        check_status();
        const RankCtx c = ctx();
        const DriverApi& api = DriverApi::get();
        CUstream stream = at::cuda::getCurrentCUDAStream().stream();
        const uint64_t seq = memop_seq_[channel] + 1;
        const size_t word = EP_WS_HOST_FLAGS_OFFSET + (static_cast<size_t>(channel) * EP_MAX_RANKS) * sizeof(uint64_t);
        for (int step = 0; step < c.num_ranks; ++step) {
            const int p = (c.rank + step) % c.num_ranks;
            const CUdeviceptr dst = reinterpret_cast<CUdeviceptr>(c.peer_base[p]) + word + c.rank * sizeof(uint64_t);
            const CUresult r = api.StreamWriteValue64(stream, dst, seq, CU_STREAM_WRITE_VALUE_DEFAULT);
            if (r != CUDA_SUCCESS) {
                TORCH_CHECK(step == 0, "stream memory operation failed half way (driver error ", static_cast<int>(r), ")");
                return false;
            }
        }
        for (int p = 0; p < c.num_ranks; ++p) {
            const CUdeviceptr src = reinterpret_cast<CUdeviceptr>(c.peer_base[c.rank]) + word + p * sizeof(uint64_t);
            driver_check(api.StreamWaitValue64(stream, src, seq, CU_STREAM_WAIT_VALUE_GEQ), "cuStreamWaitValue64");
        }
        memop_seq_[channel] = seq;
        return true;
    }

    // Launches a kernel that waits (bounded by the GPU timeout) for a flag nothing sets; used to test that a
    // failed wait ends in a status record and a poisoned buffer instead of a trap or a hang.
    static void wait_flag_test_group(const std::vector<ElasticBufferCore*>& group, int64_t expected) {
        std::vector<RankCtx> ctxs;
        for (auto* g : group) ctxs.push_back(g->ctx());
        cuda_check(ep::launch_wait_flag_test(ctxs.data(), static_cast<int>(ctxs.size()), static_cast<uint64_t>(expected),
                                             at::cuda::getCurrentCUDAStream()),
                   "wait-flag launch");
    }

    // Copy-engine push of a contiguous tensor into `dst_rank`'s symmetric buffer at `dst_offset` (stream ordered).
    void peer_copy(int dst_rank, int64_t dst_offset, const at::Tensor& src) {
        TORCH_CHECK(src.is_cuda() && src.is_contiguous(), "src must be a contiguous CUDA tensor");
        const int64_t bytes = src.numel() * src.element_size();
        TORCH_CHECK(dst_rank >= 0 && dst_rank < num_ranks(), "bad destination rank");
        TORCH_CHECK(dst_offset >= static_cast<int64_t>(EP_WORKSPACE_BYTES) && dst_offset + bytes <= mem_->bytes(),
                    "peer copy [", dst_offset, ", ", dst_offset + bytes, ") is outside the symmetric buffer");
        const RankCtx c = ctx();
        if (bytes == 0) return;
        cuda_check(cudaMemcpyAsync(c.peer_base[dst_rank] + dst_offset, src.data_ptr(), static_cast<size_t>(bytes),
                                   cudaMemcpyDeviceToDevice, at::cuda::getCurrentCUDAStream()),
                   "peer cudaMemcpyAsync");
    }

    // ------------------------------------------------------------------ CPU segment
    int64_t num_cpu_bytes() const { return mem_->cpu_bytes(); }
    std::string get_local_cpu_segment_name() const { return mem_->export_cpu_name(); }
    void open_cpu_peers(const std::vector<std::string>& names) { mem_->open_cpu_peers(names); }
    void unlink_cpu_segment_name() { mem_->unlink_cpu_name(); }
    // stream-ordered copy of a contiguous device tensor into this rank's CPU segment at `offset`
    void cpu_segment_write(int64_t offset, const at::Tensor& src) {
        TORCH_CHECK(mem_->cpu_segment_host() != nullptr, "the buffer was built without a CPU segment (num_cpu_bytes = 0)");
        TORCH_CHECK(src.is_cuda() && src.is_contiguous(), "src must be a contiguous CUDA tensor");
        const int64_t bytes = src.numel() * src.element_size();
        TORCH_CHECK(offset >= 0 && offset + bytes <= mem_->cpu_bytes(), "write outside the CPU segment");
        if (bytes == 0) return;
        cuda_check(cudaMemcpyAsync(mem_->cpu_segment_host() + offset, src.data_ptr(), static_cast<size_t>(bytes), cudaMemcpyDefault,
                                   at::cuda::getCurrentCUDAStream()),
                   "cudaMemcpyAsync(device -> CPU segment)");
    }

    // Engram: pull `indices.numel()` entries of `entry_bytes` from their owners' tables into `out`.  The tables live at
    // `off_storage` of every rank's symmetric buffer, or, with `in_cpu_segment`, at that offset of every rank's CPU
    // segment.  `sf_table` (replicated scale packs of all entries) is gathered locally into `fetched_sf`.
    static void engram_fetch_group(const std::vector<ElasticBufferCore*>& group, const std::vector<at::Tensor>& indices,
                                   const std::vector<at::Tensor>& outs, int64_t entries_per_rank, int64_t entry_bytes,
                                   int64_t off_storage, bool in_cpu_segment, const std::vector<at::Tensor>& sf_tables,
                                   const std::vector<at::Tensor>& fetched_sfs, int64_t entries_per_token, int num_sms) {
        std::vector<EngramFetchArgs> args(group.size());
        TORCH_CHECK(sf_tables.empty() || (sf_tables.size() == group.size() && fetched_sfs.size() == group.size()),
                    "one scale table and one output per buffer");
        for (size_t i = 0; i < group.size(); ++i) {
            group[i]->check_status();
            const at::Tensor& idx = indices[i];
            TORCH_CHECK(idx.is_cuda() && idx.is_contiguous() && idx.scalar_type() == at::kInt, "indices must be contiguous int32");
            TORCH_CHECK(outs[i].is_contiguous() && outs[i].numel() * outs[i].element_size() == idx.numel() * entry_bytes,
                        "output has the wrong size");
            EngramFetchArgs a{};
            a.ctx = group[i]->ctx();
            const int R = a.ctx.num_ranks;
            if (in_cpu_segment) {
                TORCH_CHECK(off_storage >= 0 && off_storage % 16 == 0 && off_storage + entries_per_rank * entry_bytes <= group[i]->num_cpu_bytes(),
                            "engram storage does not fit the CPU segment");
                for (int r = 0; r < R; ++r) {
                    TORCH_CHECK(group[i]->mem_->cpu_segment(r) != nullptr, "the CPU segment of rank ", r, " is not mapped");
                    a.storage[r] = group[i]->mem_->cpu_segment(r) + off_storage;
                }
            } else {
                group[i]->check_region(off_storage, entries_per_rank * entry_bytes, "engram storage");
                for (int r = 0; r < R; ++r) a.storage[r] = a.ctx.peer_base[r] + off_storage;
            }
            a.indices = idx.data_ptr<int32_t>();
            a.num_fetches = static_cast<int>(idx.numel());
            a.entries_per_rank = static_cast<int>(entries_per_rank);
            a.entry_bytes = static_cast<int>(entry_bytes);
            a.out = outs[i].data_ptr();
            a.entries_per_token = static_cast<int>(entries_per_token > 0 ? entries_per_token : 1);
            if (!sf_tables.empty()) {
                const at::Tensor& tab = sf_tables[i];
                const at::Tensor& fsf = fetched_sfs[i];
                TORCH_CHECK(tab.is_cuda() && tab.is_contiguous() && tab.dim() == 2 && tab.element_size() == 4 &&
                                tab.size(0) == entries_per_rank * R, "the scale table must be contiguous [all entries, packs] of 4-byte packs");
                TORCH_CHECK(fsf.is_cuda() && fsf.dim() == 2 && fsf.element_size() == 4 && fsf.size(0) * a.entries_per_token == idx.numel() &&
                                fsf.size(1) == a.entries_per_token * tab.size(1), "fetched scales must be [tokens, entries per token * packs]");
                a.sf_table = reinterpret_cast<const int32_t*>(tab.data_ptr());
                a.fetched_sf = reinterpret_cast<int32_t*>(fsf.data_ptr());
                a.sf_packs = static_cast<int>(tab.size(1));
                a.sf_token_stride = fsf.stride(0);
                a.sf_pack_stride = fsf.stride(1);
            }
            args[i] = a;
        }
        cuda_check(ep::launch_engram_fetch(args.data(), static_cast<int>(args.size()), num_sms, at::cuda::getCurrentCUDAStream()),
                   "engram fetch launch");
    }

    RankCtx ctx() const { return mem_->ctx(gpu_timeout_ns_); }
    OperationCoordinator& coordinator() { return coord_; }
    SymmetricMemory& memory() { return *mem_; }

private:
    static const void* ptr_or_null(const OptTensor& t) { return t.has_value() ? t->data_ptr() : nullptr; }

    void check_region(int64_t off, int64_t bytes, const char* what) const {
        TORCH_CHECK(off >= static_cast<int64_t>(EP_WORKSPACE_BYTES) && off % 16 == 0 && off + bytes <= mem_->bytes(), what,
                    " region [", off, ", ", off + bytes, ") does not fit the symmetric buffer of ", mem_->bytes(), " bytes");
    }

    DispatchArgs make_dispatch_args(const DispatchCall& c) const {
        DispatchArgs a{};
        a.ctx = ctx();
        const int R = a.ctx.num_ranks;
        TORCH_CHECK(c.x.is_cuda() && c.x.dim() == 2 && c.x.is_contiguous(), "x must be a contiguous [T, H] CUDA tensor");
        const bool fp8 = c.x.scalar_type() == at::kFloat8_e4m3fn;
        TORCH_CHECK(fp8 || c.x.scalar_type() == at::kBFloat16, "x must be bf16 or float8_e4m3fn");
        const int64_t T = c.x.size(0), H = c.x.size(1);
        TORCH_CHECK(T <= c.num_max_tokens, "num_tokens exceeds num_max_tokens_per_rank");
        TORCH_CHECK((H * c.x.element_size()) % 16 == 0 && H % 16 == 0, "hidden bytes must be a multiple of 16");
        TORCH_CHECK(reinterpret_cast<uintptr_t>(c.x.data_ptr()) % 16 == 0, "x must be 16-byte aligned");
        TORCH_CHECK(!(c.quantize && fp8), "fused quantization takes bf16 input");
        const int64_t G = (H + 127) / 128;
        if (fp8) {
            TORCH_CHECK(c.sf.has_value() && c.sf->scalar_type() == at::kFloat && c.sf->is_contiguous() &&
                            c.sf->dim() == 2 && c.sf->size(0) == T && c.sf->size(1) == G,
                        "fp8 input needs contiguous fp32 scales [T, ceil(H/128)]");
        }
        TORCH_CHECK(c.num_experts > 0 && c.num_experts % R == 0 && c.num_experts <= EP_MAX_EXPERTS,
                    "num_experts must be a positive multiple of the rank count (at most ", EP_MAX_EXPERTS, ")");
        TORCH_CHECK(!c.do_expand || c.expert_alignment >= 1, "bad expert alignment");
        const at::Tensor& plan = c.plan;
        TORCH_CHECK(plan.scalar_type() == at::kInt && plan.is_contiguous() && plan.dim() == 2 && plan.size(0) == T,
                    "plan must be int32 [T, K]");
        const int64_t K = plan.size(1);
        TORCH_CHECK(K >= 1 && K <= EP_MAX_TOPK, "num_topk out of range");
        TORCH_CHECK(c.lane_src.scalar_type() == at::kInt && c.lane_src.is_contiguous() && c.lane_src.sizes() == plan.sizes(),
                    "lane_src must match plan");
        TORCH_CHECK(c.topk_idx.has_value(), "topk_idx is required (a cached layout passes the handle's copy)");
        {
            const auto& idx = *c.topk_idx;
            TORCH_CHECK(idx.is_contiguous() && idx.dim() == 2 && idx.size(0) == T && idx.size(1) == K &&
                            (idx.scalar_type() == at::kLong || idx.scalar_type() == at::kInt),
                        "topk_idx must be contiguous int64/int32 [T, K]");
            a.topk_idx = idx.data_ptr();
            a.idx_is_64 = idx.scalar_type() == at::kLong;
        }
        if (c.topk_weights.has_value()) {
            TORCH_CHECK(c.topk_weights->scalar_type() == at::kFloat && c.topk_weights->is_contiguous() &&
                            c.topk_weights->size(0) == T && c.topk_weights->size(1) == K,
                        "topk_weights must be contiguous fp32 [T, K]");
        }
        const int64_t El = c.num_experts / R;
        TORCH_CHECK(c.psum_rank.numel() == R && c.psum_expert.numel() == El && c.recv_per_expert.numel() == El,
                    "handle tensors have the wrong size");
        if (c.stats.has_value()) TORCH_CHECK(c.stats->scalar_type() == at::kInt && c.stats->numel() == El, "bad stats tensor");
        const int64_t out_row = (c.quantize || fp8) ? H : H * 2;
        const int64_t cap = c.recv_capacity_rows;
        TORCH_CHECK(cap > 0 && cap < (1 << 24), "bad receive capacity");
        check_region(c.off_recv_x, cap * out_row, "recv_x");
        if (c.quantize || fp8) check_region(c.off_recv_sf, cap * (c.sf_stride_col == 1 ? c.sf_stride_row : G) * 4, "recv_sf");
        if (!c.do_expand) check_region(c.off_recv_idx, cap * K * 8, "recv_topk_idx");
        check_region(c.off_recv_w, cap * (c.do_expand ? 1 : K) * 4, "recv_topk_weights");
        check_region(c.off_recv_meta, cap * 8, "recv_src_metadata");

        a.x = c.x.data_ptr();
        a.sf = fp8 ? c.sf->data_ptr<float>() : nullptr;
        a.topk_weights = c.topk_weights.has_value() ? c.topk_weights->data_ptr<float>() : nullptr;
        a.num_tokens = static_cast<int>(T);
        a.hidden = static_cast<int>(H);
        a.num_topk = static_cast<int>(K);
        a.num_experts = static_cast<int>(c.num_experts);
        a.x_is_fp8 = fp8;
        a.quantize = c.quantize;
        a.do_expand = c.do_expand;
        a.expert_alignment = static_cast<int>(c.expert_alignment);
        a.cached = c.cached;
        a.num_max_tokens = static_cast<int>(c.num_max_tokens);
        a.lane_src = c.lane_src.data_ptr<int32_t>();
        a.plan = c.plan.data_ptr<int32_t>();
        a.psum_rank = c.psum_rank.data_ptr<int32_t>();
        a.psum_expert = c.psum_expert.data_ptr<int32_t>();
        a.recv_per_expert = c.recv_per_expert.data_ptr<int32_t>();
        a.stats = c.stats.has_value() ? c.stats->data_ptr<int32_t>() : nullptr;
        a.off_recv_x = c.off_recv_x;
        a.off_recv_sf = c.off_recv_sf;
        a.off_recv_idx = c.off_recv_idx;
        a.off_recv_w = c.off_recv_w;
        a.off_recv_meta = c.off_recv_meta;
        a.sf_stride_row = c.sf_stride_row;
        a.sf_stride_col = c.sf_stride_col;
        a.recv_capacity_rows = static_cast<int>(cap);
        if (c.prof.has_value()) {
            TORCH_CHECK(c.prof->scalar_type() == at::kLong && c.prof->numel() >= 8 && c.prof->is_cuda(), "prof must be int64 [8] on the GPU");
            a.prof = reinterpret_cast<uint64_t*>(c.prof->data_ptr<int64_t>());
        }
        a.do_zero_padding = c.do_zero_padding;
        TORCH_CHECK(!c.do_zero_padding || c.do_expand, "zero padding needs the expand layout");
        a.tune_warps = static_cast<int>(c.tune_warps);
        a.tune_stages = static_cast<int>(c.tune_stages);
        if (c.side_packed) {
            const int64_t idx_bytes = K * (a.idx_is_64 ? 8 : 4);
            TORCH_CHECK(!c.do_expand && c.sf_stride_col == 1, "bulk side stores need the non-expand layout and row-major scales");
            TORCH_CHECK(!(c.quantize || fp8) || (c.sf_stride_row >= G && c.sf_stride_row % 4 == 0 && (G * 4) % 16 == 0),
                        "bulk side stores need scale rows that start on 16-byte boundaries and are a multiple of 16 bytes long");
            TORCH_CHECK(c.tail_bytes % 16 == 0 && c.tail_off_w % 4 == 0 && c.tail_off_meta % 8 == 0 && c.tail_off_w >= idx_bytes &&
                            c.tail_off_meta >= c.tail_off_w + K * 4 && c.tail_bytes >= c.tail_off_meta + 8,
                        "inconsistent tail record layout");
            const int64_t pitch = c.tail_pitch > 0 ? c.tail_pitch : c.tail_bytes;
            TORCH_CHECK(pitch >= c.tail_bytes && pitch % 16 == 0, "bad tail record pitch");
            check_region(c.off_recv_tail, cap * pitch, "recv tail records");
            a.side_packed = 1;
            a.tail_pitch = static_cast<int>(pitch);
            a.tail_bytes = static_cast<int>(c.tail_bytes);
            a.tail_off_w = static_cast<int>(c.tail_off_w);
            a.tail_off_meta = static_cast<int>(c.tail_off_meta);
            a.off_recv_tail = c.off_recv_tail;
        }
        return a;
    }

    CombineArgs make_combine_args(const CombineCall& c) const {
        CombineArgs a{};
        a.ctx = ctx();
        TORCH_CHECK(c.plan.scalar_type() == at::kInt && c.plan.is_contiguous() && c.plan.dim() == 2, "plan must be int32 [T, K]");
        const int64_t T = c.plan.size(0), K = c.plan.size(1), H = c.hidden;
        TORCH_CHECK(K >= 1 && K <= EP_MAX_TOPK && H > 0 && (H * 2) % 16 == 0, "bad combine shape");
        TORCH_CHECK(c.out.scalar_type() == at::kBFloat16 && c.out.is_contiguous() && c.out.size(0) == T && c.out.size(1) == H,
                    "out must be contiguous bf16 [T, H]");
        for (const OptTensor* b : {&c.bias0, &c.bias1})
            if (b->has_value())
                TORCH_CHECK((*b)->scalar_type() == at::kBFloat16 && (*b)->is_contiguous() && (*b)->sizes() == c.out.sizes(),
                            "bias must be contiguous bf16 [T, H]");
        TORCH_CHECK(c.off_x >= static_cast<int64_t>(EP_WORKSPACE_BYTES) && c.off_x % 16 == 0 && c.off_x < mem_->bytes(),
                    "combine input offset outside the symmetric buffer");
        if (c.out_w.has_value()) {
            TORCH_CHECK(c.out_w->scalar_type() == at::kFloat && c.out_w->is_contiguous() && c.out_w->numel() == T * K &&
                            c.off_w >= static_cast<int64_t>(EP_WORKSPACE_BYTES) && c.w_cols >= 1,
                        "bad weight transport arguments");
            TORCH_CHECK(c.lane_src.scalar_type() == at::kInt && c.lane_src.is_contiguous() && c.lane_src.sizes() == c.plan.sizes(),
                        "lane_src must match plan");
        }
        if (c.mul_weights.has_value())
            TORCH_CHECK(c.mul_weights->scalar_type() == at::kFloat && c.mul_weights->is_contiguous() &&
                            c.mul_weights->numel() == T * K, "mul_weights must be contiguous fp32 [T, K]");
        a.off_x = c.off_x;
        a.off_w = c.off_w;
        a.w_cols = static_cast<int>(c.w_cols);
        a.plan = c.plan.data_ptr<int32_t>();
        a.lane_src = c.out_w.has_value() ? c.lane_src.data_ptr<int32_t>() : nullptr;
        a.mul_weights = c.mul_weights.has_value() ? c.mul_weights->data_ptr<float>() : nullptr;
        a.bias0 = ptr_or_null(c.bias0);
        a.bias1 = ptr_or_null(c.bias1);
        a.out = c.out.data_ptr();
        a.out_w = c.out_w.has_value() ? c.out_w->data_ptr<float>() : nullptr;
        a.num_tokens = static_cast<int>(T);
        a.hidden = static_cast<int>(H);
        a.num_topk = static_cast<int>(K);
        if (c.prof.has_value()) {
            TORCH_CHECK(c.prof->scalar_type() == at::kLong && c.prof->numel() >= 8 && c.prof->is_cuda(), "prof must be int64 [8] on the GPU");
            a.prof = reinterpret_cast<uint64_t*>(c.prof->data_ptr<int64_t>());
        }
        return a;
    }

    std::unique_ptr<SymmetricMemory> mem_;
    OperationCoordinator coord_;
    uint64_t gpu_timeout_ns_;
    double cpu_timeout_secs_;
    uint64_t dispatch_epoch_ = 0;
    uint64_t memop_seq_[EP_NUM_CHANNELS] = {};
};

}  // namespace ep_host
