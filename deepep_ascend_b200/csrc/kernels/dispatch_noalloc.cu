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
uint64_t g_calls[kMaxDevices] = {};

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
    if (reinterpret_cast<uintptr_t>(x) % 16 != 0 || reinterpret_cast<uintptr_t>(recv_x) % 16 != 0)
        return fail(err, err_len, "x and recv_x must be 16-byte aligned");

    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return fail(err, err_len, "cudaGetDevice", e);
    if (device < 0 || device >= kMaxDevices) return fail(err, err_len, "device index beyond 63");
    unsigned char* base = nullptr;
    uint64_t call_index = 0;
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
        call_index = ++g_calls[device];
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // what must start at zero: the abort flag of the workspace and the status words (a failure of an earlier call
    // must not leak into this one).  Epochs, barrier generations and tagged counters carry over by design.
    e = cudaMemsetAsync(base + offsetof(ep::Workspace, abort_flag), 0, sizeof(uint32_t), s);
    if (e == cudaSuccess) e = cudaMemsetAsync(base + kWorkspaceBytes, 0, 8 * sizeof(uint64_t), s);
    if (e != cudaSuccess) return fail(err, err_len, "cudaMemsetAsync(scratch flags)", e);

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
    (void)call_index;
    e = ep::launch_dispatch(&a, 1, num_sms, s);
    if (e != cudaSuccess) return fail(err, err_len, "dispatch launch", e);
    return 0;
}
