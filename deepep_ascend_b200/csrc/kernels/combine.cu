// Expert-parallel combine for one NVLink domain, as ONE kernel per call: the token's home rank PULLS the rows
// that its experts produced straight out of the expert ranks' symmetric buffers (TMA bulk loads through the
// peer mappings, no multicast) and reduces them in fp32 registers, so the reduction is fused into the gather
// and no intermediate slab is written or re-read.
//
// Work item = (token, column chunk of 32 lanes x 16 B x kUnroll).  Each warp owns kSlots item slots; a slot
// has one chunk buffer per top-k lane and one mbarrier.  While the warp reduces item n, the loads of item
// n + kSlots - 1 are in flight.  The accumulation order is fixed (bias0 + bias1 first, then the plan entries in
// top-k lane order), so results are bitwise reproducible.
//
// Parity: does the work of combine_impl + combine_reduce_epilogue_impl
// (deep_ep/include/deep_ep/impls/combine.cuh:15-243, combine_reduce_epilogue.cuh:12-143) plus the weighted
// reduction of the legacy low-latency combine (csrc/kernels/legacy/internode_ll.cu:1033-1136).
#include <cstdlib>

#include "common.cuh"

namespace ep {

namespace {

constexpr int kCombineMaxWarps = 16;
constexpr int kCombineMaxRing = 32;              // chunk buffers (and mbarriers) per warp
constexpr int kCombineSmemBudget = 208 * 1024;
constexpr int kCombineQueue = 64;                // claimed-token queue per warp (producer -> consumer)

template <int kUnroll>
struct CombineCfg {
    static constexpr int kChunkBytes = 32 * 16 * kUnroll;
};

// Shared-memory plan: [peer table | mbarriers W x ring | chunk buffers W x ring]
struct CombineSmemPlan {
    int num_warps, ring, off_bar, off_queue, off_data, total;
};
__host__ __device__ inline CombineSmemPlan combine_smem_plan(int chunk_bytes, int num_warps) {
    CombineSmemPlan p;
    p.num_warps = num_warps;
    p.off_bar = 128;
    p.off_queue = 128 + num_warps * kCombineMaxRing * 8;
    p.off_data = p.off_queue + num_warps * kCombineQueue * 4;
    p.off_data = (p.off_data + 1023) / 1024 * 1024;
    int ring = (kCombineSmemBudget - p.off_data) / (num_warps * chunk_bytes);
    p.ring = ring > kCombineMaxRing ? kCombineMaxRing : ring;
    p.total = p.off_data + num_warps * p.ring * chunk_bytes;
    return p;
}

// Cursor over the flattened sequence of (work item, source) pairs of one warp.  Lane k holds plan[t][k] of the
// cursor's item; `pending` has one bit per source that is still to be visited, lowest lane first.
struct PullCursor {
    int token;           // >= num_tokens when exhausted
    int chunk;
    int plan_k;
    uint32_t sources;    // lanes of the token's plan that hold a row
    uint32_t pending;    // sources of the current chunk not visited yet
};

template <int kUnroll>
__device__ __forceinline__ void combine_body(const CombineArgs& a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr int kChunk = CombineCfg<kUnroll>::kChunkBytes;
    const RankCtx& ctx = a.ctx;
    Workspace* ws = local_ws(ctx);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int num_warps = blockDim.x >> 5;
    const int K = a.num_topk, T = a.num_tokens;
    const int row_bytes = a.hidden * 2;
    const int num_chunks = (row_bytes + kChunk - 1) / kChunk;
    const CombineSmemPlan sp = combine_smem_plan(kChunk, num_warps);
    const int ring = sp.ring;

    uint8_t** s_peer = reinterpret_cast<uint8_t**>(smem);
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + sp.off_bar) + warp * kCombineMaxRing;
    uint8_t* s_data = smem + sp.off_data + static_cast<size_t>(warp) * ring * kChunk;
    int* s_queue = reinterpret_cast<int*>(smem + sp.off_queue) + warp * kCombineQueue;
    if (blockIdx.x == 0 && tid == 0) atomicExch(&ws->dyn_counter[EP_CH_COMBINE], 0u);   // ordered before its first use by the grid barrier

    if (tid < EP_MAX_RANKS) s_peer[tid] = tid < ctx.num_ranks ? ctx.peer_base[tid] : nullptr;
    if (lane == 0)
        for (int b = 0; b < ring; ++b) ptx::mbar_init(&s_bar[b], 1);
    ptx::mbar_fence_init();
    __syncthreads();
    ptx::fence_proxy_async_smem();

    auto stamp = [&](int i) {
        if (a.prof != nullptr && blockIdx.x == 0 && tid == 0) a.prof[i] = globaltimer_ns();
    };
    stamp(0);
    // every rank's input rows must be in place before anyone pulls
    bool alive = !is_aborted(ws);
    if (blockIdx.x == 0) alive = xgpu_barrier(ctx, ws, EP_CH_COMBINE, EP_PH_COMBINE_ENTRY) && alive;
    alive = grid_sync(ctx, ws, EP_CH_COMBINE, EP_PH_GRID_SYNC) && alive;
    stamp(1);

    // Tokens are claimed dynamically from a counter shared by all CTAs of this rank (SMs that get a smaller share of
    // the NVLink bandwidth claim fewer tokens, so no CTA is left with a tail).  The producer cursor claims; the
    // claimed ids travel through a small per-warp queue to the consumer cursor, which follows in the same order.
    uint32_t claimed = 0, started = 0;     // tokens claimed by the producer / started by the consumer
    auto claim_token = [&]() -> int {
        int tkn = 0;
        if (lane == 0) {
            tkn = static_cast<int>(atomicAdd(&ws->dyn_counter[EP_CH_COMBINE], 1u));
            s_queue[claimed % kCombineQueue] = tkn;
        }
        __syncwarp();
        ++claimed;
        return __shfl_sync(0xffffffffu, tkn, 0);
    };
    auto load_token = [&](PullCursor& c) {
        c.chunk = 0;
        c.plan_k = -1;
        c.sources = 0;
        if (c.token < T) {
            c.plan_k = lane < K ? a.plan[static_cast<int64_t>(c.token) * K + lane] : -1;
            c.sources = __ballot_sync(0xffffffffu, c.plan_k >= 0);
        }
        c.pending = c.sources;
    };
    // producer: move to its next token (claims one); returns false when the queue is too full to claim right now
    auto producer_next_token = [&](PullCursor& c) -> bool {
        if (claimed - started >= static_cast<uint32_t>(kCombineQueue - 8)) return false;
        c.token = c.token < T ? claim_token() : T;
        load_token(c);
        return true;
    };

    if (alive) {
        PullCursor prod{0, 0, -1, 0, 0}, cons{0, 0, -1, 0, 0};
        prod.token = claim_token();
        load_token(prod);
        uint32_t issued = 0, consumed = 0;   // loads issued / consumed by this warp; buffer = counter % ring

        // issue loads in sequence order until the ring is full or the warp's work is exhausted
        auto issue_ahead = [&]() {
            while (issued - consumed < static_cast<uint32_t>(ring) && prod.token < T) {
                if (prod.pending == 0) {
                    if (++prod.chunk == num_chunks) {
                        if (!producer_next_token(prod)) {
                            prod.chunk = num_chunks - 1;   // retry the claim on the next call
                            break;
                        }
                    } else {
                        prod.pending = prod.sources;
                    }
                    continue;
                }
                const int k = __ffs(prod.pending) - 1;
                prod.pending &= prod.pending - 1;
                const int p = __shfl_sync(0xffffffffu, prod.plan_k, k);
                if (lane == 0) {
                    const int c = prod.chunk;
                    const int bytes = min(kChunk, row_bytes - c * kChunk);
                    const int b = issued % ring;
                    const uint8_t* src = s_peer[p >> 24] + a.off_x + static_cast<int64_t>(p & 0xffffff) * row_bytes +
                                         static_cast<int64_t>(c) * kChunk;
                    ptx::mbar_arrive_expect_tx(&s_bar[b], bytes);
                    ptx::bulk_load(s_data + b * kChunk, src, bytes, &s_bar[b]);
                }
                ++issued;
            }
        };

        // consumer: pop the next claimed token (making the producer claim one if it has not run ahead)
        auto consumer_next_token = [&](PullCursor& c) {
            if (started == claimed) {
                // the producer has consumed all its claims too: it sits at the end of its current token
                prod.token = prod.token < T ? claim_token() : T;
                load_token(prod);
            }
            c.token = s_queue[started % kCombineQueue];
            ++started;
            load_token(c);
        };
        consumer_next_token(cons);
        for (; cons.token < T && alive;) {
            const int t = cons.token, c = cons.chunk;
            const int bytes = min(kChunk, row_bytes - c * kChunk);
            const int col0 = c * kChunk;   // byte offset inside the row
            issue_ahead();

            float acc[kUnroll * 8];
#pragma unroll
            for (int i = 0; i < kUnroll * 8; ++i) acc[i] = 0.f;
            // bias0 + bias1 in fp32 first
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                const uint8_t* bias = reinterpret_cast<const uint8_t*>(b == 0 ? a.bias0 : a.bias1);
                if (bias == nullptr) continue;
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    const int off = (u * 32 + lane) * 16;
                    if (off < bytes) {
                        const int4 raw = ptx::ld_nc_v4(bias + static_cast<int64_t>(t) * row_bytes + col0 + off);
                        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 f = __bfloat1622float2(h[j]);
                            acc[u * 8 + 2 * j] += f.x;
                            acc[u * 8 + 2 * j + 1] += f.y;
                        }
                    }
                }
            }
            // weights that travel back with the rows (dispatch backward): one small peer load per lane
            if (c == 0 && a.out_w != nullptr && lane < K) {
                const int ls = a.lane_src[static_cast<int64_t>(t) * K + lane];
                float w = 0.f;
                if (ls >= 0) {
                    const float* wp = reinterpret_cast<const float*>(s_peer[ls >> 24] + a.off_w);
                    const int64_t row = ls & 0xffffff;
                    w = *reinterpret_cast<const volatile float*>(a.w_cols == 1 ? wp + row : wp + row * a.w_cols + lane);
                }
                a.out_w[static_cast<int64_t>(t) * K + lane] = w;
            }
            float mul_k = 1.f;
            if (a.mul_weights != nullptr && lane < K) mul_k = __ldg(a.mul_weights + static_cast<int64_t>(t) * K + lane);

            // sources in top-k lane order; each one sits in the next ring buffer
            uint32_t srcs = cons.pending;
            while (srcs != 0 && alive) {
                const int k = __ffs(srcs) - 1;
                srcs &= srcs - 1;
                const int b = consumed % ring;
                alive = mbar_wait_bounded(ctx, ws, &s_bar[b], (consumed / ring) & 1, EP_PH_COMBINE_LOAD);
                if (!alive) break;
                const float w = __shfl_sync(0xffffffffu, mul_k, k);
                const uint8_t* buf = s_data + b * kChunk;
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    const int off = (u * 32 + lane) * 16;
                    if (off < bytes) {
                        const int4 raw = *reinterpret_cast<const int4*>(buf + off);
                        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 f = __bfloat1622float2(h[j]);
                            acc[u * 8 + 2 * j] = fmaf(w, f.x, acc[u * 8 + 2 * j]);
                            acc[u * 8 + 2 * j + 1] = fmaf(w, f.y, acc[u * 8 + 2 * j + 1]);
                        }
                    }
                }
                // the buffer may be refilled once every lane has read it
                ptx::fence_proxy_async_smem();
                __syncwarp();
                ++consumed;
                issue_ahead();
            }
            if (!alive) break;
            uint8_t* out = reinterpret_cast<uint8_t*>(a.out) + static_cast<int64_t>(t) * row_bytes + col0;
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int off = (u * 32 + lane) * 16;
                if (off < bytes) {
                    int4 raw;
                    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
                    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(acc[u * 8 + 2 * j], acc[u * 8 + 2 * j + 1]);
                    ptx::st_na_v4(out + off, raw);
                }
            }
            if (++cons.chunk == num_chunks) consumer_next_token(cons);
            else cons.pending = cons.sources;
        }
        // loads still in flight belong to nobody once the loop was left early: wait for them (bounded) so that
        // no copy lands in shared memory after the CTA has exited
        while (consumed < issued) {
            if (!bounded_wait(ctx, ws, EP_PH_COMBINE_LOAD, -1, consumed,
                              [&] { return ptx::mbar_try_wait(&s_bar[consumed % ring], (consumed / ring) & 1); }, [&] { return 0ull; }))
                break;
            ++consumed;
        }
    }

    stamp(2);
    // nobody may overwrite its input rows until every rank has finished pulling
    const bool cta_ok = __syncthreads_and(alive ? 1 : 0) != 0;
    alive = grid_sync(ctx, ws, EP_CH_COMBINE, EP_PH_GRID_SYNC) && cta_ok;
    stamp(3);
    if (blockIdx.x == 0) {
        if (alive) xgpu_barrier(ctx, ws, EP_CH_COMBINE, EP_PH_COMBINE_EXIT);
        stamp(4);
        if (tid == 0) ws->epoch[EP_CH_COMBINE] += 1;
    }
}

template <int kUnroll>
__global__ void __launch_bounds__(kCombineMaxWarps * 32, 1) combine_kernel(const __grid_constant__ CombineArgs args) {
    combine_body<kUnroll>(args);
}
template <int kUnroll>
__global__ void __launch_bounds__(kCombineMaxWarps * 32, 1) combine_kernel_multi(const CombineArgs* args) {
    combine_body<kUnroll>(args[blockIdx.y]);
}

inline int env_int(const char* name, int fallback) {
    const char* v = std::getenv(name);
    return v != nullptr && *v != 0 ? std::atoi(v) : fallback;
}

// column chunk = 512 B x unroll; EP_COMBINE_UNROLL overrides the choice when the row divides evenly
inline int pick_unroll(const CombineArgs& a) {
    const int row_bytes = a.hidden * 2;
    const int forced = env_int("EP_COMBINE_UNROLL", 0);
    if ((forced == 7 || forced == 4 || forced == 2 || forced == 1) && row_bytes % (512 * forced) == 0) return forced;
    // larger chunks amortise the per-chunk bookkeeping: 3584 B when the row divides evenly (hidden 7168), else 2048 B
    if (row_bytes % 3584 == 0) return 7;
    return row_bytes % 2048 == 0 ? 4 : (row_bytes % 1024 == 0 ? 2 : (row_bytes >= 2048 ? 4 : 1));
}

}  // namespace

LaunchShape combine_launch_shape(const CombineArgs& a, int num_sms) {
    LaunchShape s;
    s.num_ctas = num_sms < 1 ? 1 : (num_sms > EP_MAX_CTAS ? EP_MAX_CTAS : num_sms);
    int warps = env_int("EP_COMBINE_WARPS", 12);
    warps = warps < 1 ? 1 : (warps > kCombineMaxWarps ? kCombineMaxWarps : warps);
    const CombineSmemPlan p = combine_smem_plan(512 * pick_unroll(a), warps);
    s.num_warps = p.num_warps;
    s.smem_bytes = p.total;
    return s;
}

cudaError_t launch_combine(const CombineArgs* args, int n, int num_sms, cudaStream_t stream) {
    const CombineArgs& a0 = args[0];
    const LaunchShape shape = combine_launch_shape(a0, num_sms);
    if (shape.smem_bytes > 227 * 1024) return cudaErrorInvalidValue;
    const int unroll = pick_unroll(a0);
    const void* fn;
    if (n == 1)
        fn = unroll == 7 ? (const void*)combine_kernel<7> : unroll == 4 ? (const void*)combine_kernel<4>
             : unroll == 2 ? (const void*)combine_kernel<2> : (const void*)combine_kernel<1>;
    else
        fn = unroll == 7 ? (const void*)combine_kernel_multi<7> : unroll == 4 ? (const void*)combine_kernel_multi<4>
             : unroll == 2 ? (const void*)combine_kernel_multi<2> : (const void*)combine_kernel_multi<1>;
    cudaError_t err = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, shape.smem_bytes);
    if (err != cudaSuccess) return err;
    dim3 grid(shape.num_ctas, n, 1), block(shape.num_warps * 32, 1, 1);
    if (n == 1) {
        void* params[] = {const_cast<CombineArgs*>(&a0)};
        return cudaLaunchCooperativeKernel(fn, grid, block, params, shape.smem_bytes, stream);
    }
    CombineArgs* dev = nullptr;
    err = cudaMallocAsync(reinterpret_cast<void**>(&dev), sizeof(CombineArgs) * n, stream);
    if (err != cudaSuccess) return err;
    err = cudaMemcpyAsync(dev, args, sizeof(CombineArgs) * n, cudaMemcpyHostToDevice, stream);
    if (err == cudaSuccess) {
        void* params[] = {&dev};
        err = cudaLaunchCooperativeKernel(fn, grid, block, params, shape.smem_bytes, stream);
    }
    cudaFreeAsync(dev, stream);
    return err;
}

}  // namespace ep
