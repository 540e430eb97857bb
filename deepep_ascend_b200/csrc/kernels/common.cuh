// Device-side runtime shared by all kernels: the per-GPU workspace that lives at the start of every symmetric
// buffer, bounded waits that report a status instead of trapping, an in-kernel grid barrier and the
// cross-GPU signal barrier over NVLink.
//
// Failure model: no wait in this library is unbounded and nothing ever traps.  A wait that runs out of time
// records {code, peer, phase, expected, observed} in the buffer's status block (pinned host memory mapped
// into the device), raises the workspace abort flag that every other waiter polls, and returns false; the
// kernel then skips its remaining phases and exits normally.  The host reads the status after the kernel
// and poisons the buffer.
// Parity: replaces deep_ep/include/deep_ep/common/comm.cuh:30-49 (timeout -> trap) and comm.cuh:88-129.
#pragma once
#include "api.h"
#include "ptx.cuh"

namespace ep {

struct GridBarrier {
    uint32_t count;
    uint32_t gen;
};

// Lives at offset 0 of every symmetric buffer; zeroed once when the buffer is created.  All counters are
// monotonic or epoch-tagged, so kernels never have to restore them.
struct Workspace {
    // ---- written only by the owning GPU
    GridBarrier grid_bar[EP_NUM_CHANNELS];
    uint64_t epoch[EP_NUM_CHANNELS];      // completed calls per channel
    uint64_t bar_seq[EP_NUM_CHANNELS];    // cross-GPU barriers executed per channel
    uint32_t abort_flag;
    uint32_t dyn_counter[EP_NUM_CHANNELS];   // next unclaimed work item of the running kernel (dynamic scheduling)
    uint32_t pad0[31 - EP_NUM_CHANNELS];
    // ---- written by peers over NVLink
    alignas(128) uint64_t xbar[EP_NUM_CHANNELS][EP_MAX_RANKS];           // [channel][source]: arrivals
    alignas(128) uint64_t disp_rank_count[EP_MAX_RANKS][EP_MAX_RANKS];   // [source][dest], epoch-tagged
    alignas(128) uint64_t disp_expert_count[EP_MAX_RANKS][EP_MAX_EXPERTS];  // [source][expert], epoch-tagged
    alignas(128) uint64_t disp_done[EP_MAX_RANKS];                         // [source]: dispatch epoch whose rows have all arrived
    alignas(128) uint64_t ll_signal[2][EP_MAX_EXPERTS * EP_MAX_RANKS];    // low-latency count / flag words
    alignas(128) uint64_t pp_signal[4][64];                                // pipeline FIFO credits
    alignas(128) uint64_t tile_flags[EP_MAX_TILE_FLAGS];                   // fused GEMM+collective tile flags
    // ---- local scratch
    alignas(128) uint32_t cta_rank_count[EP_MAX_CTAS][EP_MAX_RANKS];
    alignas(128) uint32_t cta_expert_count[EP_MAX_CTAS][EP_MAX_EXPERTS];
    alignas(128) uint32_t ll_counters[4][EP_MAX_EXPERTS];                  // low-latency slot / finish counters
    alignas(128) uint32_t arrive[EP_NUM_CHANNELS][2];                      // CTAs that finished a phase (arrive_is_last)
    // dispatch layout phase without grid barriers: accumulators of this rank's totals (the last CTA to add reads and
    // clears them) and per-CTA progress words holding the low 32 bits of the dispatch epoch they belong to
    alignas(128) uint32_t tot_rank[EP_MAX_RANKS];
    alignas(128) uint32_t tot_expert[EP_MAX_EXPERTS];
    alignas(128) uint32_t cta_counted[EP_MAX_CTAS];                        // per-CTA counts of that epoch are in cta_*_count
    alignas(128) uint32_t cta_assigned[EP_MAX_CTAS];                       // row numbers of the CTA's tokens are in lane_src / plan
    alignas(128) uint64_t comb_seq;                                        // combine calls completed (entry-barrier sequence)
};
static_assert(sizeof(Workspace) <= EP_WS_HOST_FLAGS_OFFSET, "workspace region too small");
static_assert(EP_NUM_CHANNELS * EP_MAX_RANKS * sizeof(uint64_t) <= EP_WS_HOST_FLAGS_BYTES, "host flag area too small");

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ Workspace* local_ws(const RankCtx& ctx) {
    return reinterpret_cast<Workspace*>(ctx.peer_base[ctx.rank]);
}

__device__ __forceinline__ bool is_aborted(Workspace* ws) {
    return ptx::ld_relaxed_gpu_u32(&ws->abort_flag) != 0;
}

// First error wins; later ones only keep the abort flag up.
static __device__ __noinline__ void report_failure(const RankCtx& ctx, Workspace* ws, uint32_t code, uint32_t phase,
                                            int peer, uint64_t expected, uint64_t observed) {
    // the abort flag lives in device memory, so the race for "first" needs no atomics on host memory
    if (atomicCAS(&ws->abort_flag, 0u, 1u) == 0u) {
        volatile uint64_t* st = ctx.status;
        st[EP_STATUS_PHASE] = phase;
        st[EP_STATUS_PEER] = static_cast<uint64_t>(static_cast<int64_t>(peer));
        st[EP_STATUS_EXPECTED] = expected;
        st[EP_STATUS_OBSERVED] = observed;
        st[EP_STATUS_RANK] = ctx.rank;
        __threadfence_system();
        st[EP_STATUS_CODE] = code;
        __threadfence_system();
    }
    __threadfence();
}

// Spin until pred() or the time limit; returns false on expiry or when someone else already failed.
// `observe()` is what gets recorded as the last value seen.
template <typename Pred, typename Obs>
__device__ __forceinline__ bool bounded_wait(const RankCtx& ctx, Workspace* ws, uint32_t phase, int peer,
                                             uint64_t expected, Pred pred, Obs observe) {
    if (pred()) return true;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (!pred()) {
        if ((++spins & 31u) == 0u) {
            if (is_aborted(ws)) return false;
            if (globaltimer_ns() - t0 > ctx.timeout_ns) {
                report_failure(ctx, ws, EP_ERR_TIMEOUT, phase, peer, expected, observe());
                return false;
            }
        }
    }
    return true;
}

// Barrier over the CTAs of one rank (gridDim.x of them).  Needs co-resident CTAs (cooperative launch).
// Returns false if the wait ran out or the buffer was aborted.
__device__ __forceinline__ bool grid_sync(const RankCtx& ctx, Workspace* ws, int channel, uint32_t phase) {
    __syncthreads();
    int ok = 1;
    if (threadIdx.x == 0) {
        GridBarrier* b = &ws->grid_bar[channel];
        const uint32_t gen = ptx::ld_relaxed_gpu_u32(&b->gen);
        __threadfence();
        const uint32_t arrived = atomicAdd(&b->count, 1u);
        if (arrived == gridDim.x - 1) {
            atomicExch(&b->count, 0u);
            __threadfence();
            ptx::st_release_gpu_u32(&b->gen, gen + 1);
        } else {
            ok = bounded_wait(
                ctx, ws, phase, -1, gen + 1, [&] { return ptx::ld_acquire_gpu_u32(&b->gen) != gen; },
                [&] { return static_cast<uint64_t>(ptx::ld_relaxed_gpu_u32(&b->count)); });
        }
        __threadfence();
    }
    return __syncthreads_and(ok) != 0;
}

// Arrival without waiting: returns true in exactly one CTA of the rank's grid row, the last one to get here; the
// global writes every other CTA made before its own arrival are visible to that CTA.  The counter resets itself, so
// it can be used again by the next phase that is ordered behind this one.  Needs no co-residency.
__device__ __forceinline__ bool arrive_is_last(uint32_t* counter) {
    __shared__ int s_last;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const bool last = atomicAdd(counter, 1u) == gridDim.x - 1;
        if (last) atomicExch(counter, 0u);
        __threadfence();
        s_last = last ? 1 : 0;
    }
    __syncthreads();
    return s_last != 0;
}

// Barrier over all ranks, executed by one whole CTA per rank: every rank adds one arrival to each peer's
// counter for this channel (release) and waits until all its own counters reach this barrier's sequence
// number (acquire).  Writes made before the barrier by this rank (after a grid_sync, by any of its CTAs) are
// visible to every rank after it.
__device__ __forceinline__ bool xgpu_barrier(const RankCtx& ctx, Workspace* ws, int channel, uint32_t phase) {
    __shared__ uint64_t seq_s;
    __syncthreads();
    if (threadIdx.x == 0) {
        seq_s = ws->bar_seq[channel] + 1;
        ws->bar_seq[channel] = seq_s;
    }
    __syncthreads();
    const uint64_t seq = seq_s;
    int ok = 1;
    if (threadIdx.x < ctx.num_ranks) {
        const int peer = threadIdx.x;
        Workspace* pws = reinterpret_cast<Workspace*>(ctx.peer_base[peer]);
        ptx::red_add_release_sys(&pws->xbar[channel][ctx.rank], 1ull);
        const uint64_t* mine = &ws->xbar[channel][peer];
        ok = bounded_wait(
            ctx, ws, phase, peer, seq, [&] { return ptx::ld_acquire_sys(mine) >= seq; },
            [&] { return ptx::ld_relaxed_sys(mine); });
    }
    return __syncthreads_and(ok) != 0;
}

__device__ __forceinline__ uint64_t tag_value(uint64_t epoch, uint32_t value) { return (epoch << 32) | value; }
__device__ __forceinline__ uint32_t count_low32(uint64_t word) { return static_cast<uint32_t>(word & 0xffffffffull); }
__device__ __forceinline__ bool tag_matches(uint64_t word, uint64_t epoch) {
    return (word >> 32) == (epoch & 0xffffffffull);
}

// Bounded wait for an mbarrier phase; all lanes of a warp call it together.
__device__ __forceinline__ bool mbar_wait_bounded(const RankCtx& ctx, Workspace* ws, uint64_t* bar, uint32_t parity,
                                                  uint32_t phase) {
    const bool ok = bounded_wait(
        ctx, ws, phase, -1, parity, [&] { return ptx::mbar_try_wait(bar, parity); }, [&] { return 0ull; });
    return __all_sync(0xffffffffu, ok) != 0;
}

// After a failure: give a bulk load that is still in flight time to land (it must not arrive in shared memory that
// a later CTA owns), without looking at the abort flag.  Returns once the phase completed or `limit_ns` passed.
__device__ __forceinline__ void mbar_drain(uint64_t* bar, uint32_t parity, uint64_t limit_ns) {
    const uint64_t t0 = globaltimer_ns();
    while (!ptx::mbar_try_wait(bar, parity)) {
        if (globaltimer_ns() - t0 > limit_ns) break;
    }
}

}  // namespace ep
