// Single-rank dispatch whose scratch memory is a fixed array in the library image: see noalloc.h for who needs
// this and for the limits.  The kernel is the regular dispatch kernel; only where its workspace and status words
// live differs.
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "noalloc.h"

namespace {

constexpr size_t kStatusBytes = EP_STATUS_WORDS * sizeof(uint64_t);
constexpr size_t kWorkspaceBytes = (sizeof(ep::Workspace) + 255) / 256 * 256;
constexpr size_t kScratchBytes = kWorkspaceBytes + kStatusBytes;
constexpr int kMaxDevices = 64;

// [ Workspace | status words ].  Zero at load time, which is the state the protocol starts from.  In host code
// this name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

std::mutex g_mu;
unsigned char* g_scratch_addr[kMaxDevices] = {};   // per device, filled on the first call with that device current

int fail(char* err, int err_len, const char* msg, cudaError_t e = cudaSuccess) {
    if (err != nullptr && err_len > 0) {
        if (e != cudaSuccess) std::snprintf(err, err_len, "%s: %s", msg, cudaGetErrorString(e));
        else std::snprintf(err, err_len, "%s", msg);
    }
    return 1;
}

}  // namespace

extern "C" int ep_dispatch_one_rank_noalloc(const void* x, const void* topk_idx, const float* topk_weights, int num_tokens,
                                            int hidden, int num_topk, int num_experts, int quantize, void* recv_x, float* recv_sf,
                                            void* recv_topk_idx, float* recv_topk_weights, int32_t* recv_src_meta,
                                            int32_t* lane_src, int32_t* plan, int32_t* psum_rank, int32_t* psum_expert,
                                            int32_t* recv_per_expert, int num_sms, void* stream, char* err, int err_len) {
    if (num_experts < 1 || num_experts > EP_MAX_EXPERTS)
        return fail(err, err_len, "num_experts is outside 1..1024, the capacity of the built-in scratch array");
    if (num_topk < 1 || num_topk > EP_MAX_TOPK) return fail(err, err_len, "num_topk is outside 1..16");
    if (num_tokens < 0 || num_tokens >= (1 << 24)) return fail(err, err_len, "num_tokens is outside 0..2^24-1");
    if (num_sms < 1 || num_sms > EP_MAX_CTAS) return fail(err, err_len, "num_sms is outside 1..160, the capacity of the built-in scratch array");
    if (hidden < 16 || hidden % 16 != 0) return fail(err, err_len, "hidden must be a positive multiple of 16");
    if (x == nullptr || topk_idx == nullptr || recv_x == nullptr || recv_topk_idx == nullptr || recv_topk_weights == nullptr ||
        recv_src_meta == nullptr || lane_src == nullptr || plan == nullptr || psum_rank == nullptr || psum_expert == nullptr ||
        recv_per_expert == nullptr || (quantize && recv_sf == nullptr))
        return fail(err, err_len, "a required buffer is null");
    // a misaligned pointer would fault on the GPU instead of returning an error, so every alignment the kernel relies
    // on is checked here: 16 bytes for the rows (bulk copies), 8 for 64-bit ids and the int2 metadata, 4 for the rest
    auto misaligned = [](const void* p, uintptr_t a) { return p != nullptr && reinterpret_cast<uintptr_t>(p) % a != 0; };
    if (misaligned(x, 16) || misaligned(recv_x, 16)) return fail(err, err_len, "x and recv_x must be 16-byte aligned");
    if (misaligned(topk_idx, 8) || misaligned(recv_topk_idx, 8) || misaligned(recv_src_meta, 8))
        return fail(err, err_len, "topk_idx, recv_topk_idx and recv_src_meta must be 8-byte aligned");
    if (misaligned(topk_weights, 4) || misaligned(recv_sf, 4) || misaligned(recv_topk_weights, 4) || misaligned(lane_src, 4) ||
        misaligned(plan, 4) || misaligned(psum_rank, 4) || misaligned(psum_expert, 4) || misaligned(recv_per_expert, 4))
        return fail(err, err_len, "fp32 and int32 buffers must be 4-byte aligned");

    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return fail(err, err_len, "cudaGetDevice", e);
    if (device < 0 || device >= kMaxDevices) return fail(err, err_len, "device index beyond 63");
    unsigned char* base = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (g_scratch_addr[device] == nullptr) {
            // set-up, once per device, with that device current
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_scratch);
            if (e != cudaSuccess || p == nullptr) return fail(err, err_len, "cudaGetSymbolAddress(scratch)", e);
            g_scratch_addr[device] = static_cast<unsigned char*>(p);
        }
        base = g_scratch_addr[device];
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // What must start at zero: the abort flag, the status words, and everything a call that gave up half way may have
    // left behind (token claim counter, CTA arrival counters, count accumulators), so that a failure of an earlier call
    // cannot leak into this one.  Epochs and epoch-tagged words carry over by design.
    struct Span { size_t off, bytes; };
    const Span spans[] = {
        {offsetof(ep::Workspace, abort_flag), sizeof(uint32_t)},
        {offsetof(ep::Workspace, dyn_counter) + EP_CH_DISPATCH * sizeof(uint32_t), sizeof(uint32_t)},
        {offsetof(ep::Workspace, arrive) + EP_CH_DISPATCH * 2 * sizeof(uint32_t), 2 * sizeof(uint32_t)},
        {offsetof(ep::Workspace, tot_rank), sizeof(uint32_t) * EP_MAX_RANKS},
        {offsetof(ep::Workspace, tot_expert), sizeof(uint32_t) * EP_MAX_EXPERTS},
        {kWorkspaceBytes, 8 * sizeof(uint64_t)},
    };
    for (const Span& sp : spans) {
        e = cudaMemsetAsync(base + sp.off, 0, sp.bytes, s);
        if (e != cudaSuccess) return fail(err, err_len, "cudaMemsetAsync(scratch flags)", e);
    }

    DispatchArgs a;
    std::memset(&a, 0, sizeof(a));
    a.ctx.rank = 0;
    a.ctx.num_ranks = 1;
    a.ctx.peer_base[0] = base;
    a.ctx.status = reinterpret_cast<uint64_t*>(base + kWorkspaceBytes);
    a.ctx.timeout_ns = 10ull * 1000 * 1000 * 1000;
    a.x = x;
    a.topk_idx = topk_idx;
    a.topk_weights = topk_weights;
    a.num_tokens = num_tokens;
    a.hidden = hidden;
    a.num_topk = num_topk;
    a.num_experts = num_experts;
    a.idx_is_64 = 1;
    a.quantize = quantize != 0;
    a.expert_alignment = 1;
    a.num_max_tokens = num_tokens > 0 ? num_tokens : 1;
    a.lane_src = lane_src;
    a.plan = plan;
    a.psum_rank = psum_rank;
    a.psum_expert = psum_expert;
    a.recv_per_expert = recv_per_expert;
    // the kernel addresses outputs as (buffer base + byte offset); unsigned wrap-around makes any caller pointer reachable
    auto offset_of = [&](const void* p) { return static_cast<uint64_t>(reinterpret_cast<uintptr_t>(p) - reinterpret_cast<uintptr_t>(base)); };
    a.off_recv_x = offset_of(recv_x);
    a.off_recv_sf = offset_of(recv_sf);
    a.off_recv_idx = offset_of(recv_topk_idx);
    a.off_recv_w = offset_of(recv_topk_weights);
    a.off_recv_meta = offset_of(recv_src_meta);
    a.sf_stride_row = (hidden + 127) / 128;
    a.sf_stride_col = 1;
    a.recv_capacity_rows = num_tokens > 0 ? num_tokens : 1;
    e = ep::launch_dispatch(&a, 1, num_sms, s);
    if (e != cudaSuccess) return fail(err, err_len, "dispatch launch", e);
    return 0;
}

extern "C" int ep_noalloc_last_status(unsigned long long out[6], void* stream, char* err, int err_len) {
    if (out == nullptr) return fail(err, err_len, "out is null");
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return fail(err, err_len, "cudaGetDevice", e);
    if (device < 0 || device >= kMaxDevices) return fail(err, err_len, "device index beyond 63");
    unsigned char* base = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        base = g_scratch_addr[device];
    }
    if (base == nullptr) {   // no dispatch has run on this device yet: nothing to report
        for (int i = 0; i < 6; ++i) out[i] = 0;
        return 0;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    e = cudaMemcpyAsync(out, base + kWorkspaceBytes, 6 * sizeof(uint64_t), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return fail(err, err_len, "reading the status words", e);
    return 0;
}
