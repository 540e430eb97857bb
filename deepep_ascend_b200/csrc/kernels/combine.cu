// Expert-parallel combine for one NVLink domain, as ONE kernel per call: the token's home rank PULLS the rows
// that its experts produced straight out of the expert ranks' symmetric buffers (TMA bulk loads through the
// peer mappings, no multicast) and reduces them in fp32 registers, so the reduction is fused into the gather
// and no intermediate slab is written or re-read.
//
// Work item = (token, column chunk of 32 lanes x 16 B x kUnroll).  Items are claimed dynamically by the warps of all
// CTAs from one counter, a whole token's chunks per claim at first and single chunks near the end, so that no warp is
// left with a long tail.  Each warp owns a ring of chunk buffers with one mbarrier each: while it reduces one chunk,
// the loads of the following ones are in flight.  The accumulation order is fixed (bias0 + bias1 first, then the plan
// entries in top-k lane order), so results are bitwise reproducible.
//
// There is no grid-wide barrier and no exit barrier.  Entry: CTA 0 signals every peer, every CTA watches the peers'
// signals itself (all ranks' input rows are in place once all ranks have entered the call).  Exit: the caller
// alternates between two input regions, and a rank can only pass the entry barrier of call n + 1 after every rank has
// entered it, i.e. has finished pulling for call n; so the region of call n is free again when call n + 1 returns.
//
// Parity: does the work of combine_impl + combine_reduce_epilogue_impl
// (deep_ep/include/deep_ep/impls/combine.cuh:15-243, combine_reduce_epilogue.cuh:12-143) plus the weighted
// reduction of the legacy low-latency combine (csrc/kernels/legacy/internode_ll.cu:1033-1136).
#include "common.cuh"

namespace ep {

namespace {

constexpr int kCombineMaxWarps = 12;
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
    p.off_data = p.off_queue + num_warps * kCombineQueue * 8;   // claimed ranges: first item and length
    p.off_data = (p.off_data + 1023) / 1024 * 1024;
    int ring = (kCombineSmemBudget - p.off_data) / (num_warps * chunk_bytes);
    p.ring = ring > kCombineMaxRing ? kCombineMaxRing : ring;
    p.total = p.off_data + num_warps * p.ring * chunk_bytes;
    return p;
}

// Cursor over the flattened sequence of (work item, source) pairs of one warp.  Items are numbered token * num_chunks +
// chunk; a cursor walks a claimed range [item, range_end).  Lane k holds plan[t][k] of the cursor's token; `pending`
// has one bit per source that is still to be visited, lowest lane first.
struct PullCursor {
    int item, range_end;   // current item and end of the claimed range (item == range_end: range used up)
    int token;             // token whose plan is loaded, -1 for none
    int plan_k;
    uint32_t sources;      // lanes of the token's plan that hold a row
    uint32_t pending;      // sources of the current chunk not visited yet
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
    int* s_queue = reinterpret_cast<int*>(smem + sp.off_queue) + warp * 2 * kCombineQueue;
    int* s_qlen = s_queue + kCombineQueue;
    // every CTA reads the entry-barrier sequence before it arrives anywhere; the last CTA to finish writes the new one
    const uint64_t entry_seq = *reinterpret_cast<volatile uint64_t*>(&ws->comb_seq) + 1;

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
    // every rank's input rows must be in place before anyone pulls: CTA 0 tells the peers that this rank has entered
    // the call (stream order puts its rows before the kernel), every CTA waits for all peers' words itself
    bool alive = !is_aborted(ws);
    {
        int ok = alive ? 1 : 0;
        if (alive && tid < ctx.num_ranks) {
            if (blockIdx.x == 0) ptx::red_add_release_sys(&reinterpret_cast<Workspace*>(s_peer[tid])->xbar[EP_CH_COMBINE][ctx.rank], 1ull);
            const uint64_t* mine = &ws->xbar[EP_CH_COMBINE][tid];
            ok = bounded_wait(
                ctx, ws, EP_PH_COMBINE_ENTRY, tid, entry_seq, [&] { return ptx::ld_acquire_sys(mine) >= entry_seq; },
                [&] { return ptx::ld_relaxed_sys(mine); });
        }
        alive = __syncthreads_and(ok) != 0;
    }
    stamp(1);

    // Items are claimed from a counter shared by all CTAs of this rank (SMs that get a smaller share of the NVLink
    // bandwidth claim fewer), which is zero at entry: the last CTA of every call clears it.  The producer cursor
    // claims; the claimed ranges travel through a small per-warp queue to the consumer cursor, which follows in the
    // same order.
    const int total_items = T * num_chunks;
    const int tail_zone = 2 * static_cast<int>(gridDim.x) * num_warps * num_chunks;
    uint32_t claimed = 0, started = 0;     // ranges claimed by the producer / started by the consumer
    int last_base = 0;
    auto claim_range = [&](int& amount) -> int {   // -> first item of the range; base and length also go into the queue
        amount = last_base + tail_zone < total_items ? num_chunks : 1;
        int base = 0;
        if (lane == 0) {
            base = static_cast<int>(atomicAdd(&ws->dyn_counter[EP_CH_COMBINE], static_cast<uint32_t>(amount)));
            s_queue[claimed % kCombineQueue] = base;
            s_qlen[claimed % kCombineQueue] = amount;
        }
        __syncwarp();
        ++claimed;
        base = __shfl_sync(0xffffffffu, base, 0);
        last_base = base;
        return base;
    };
    auto load_token = [&](PullCursor& c) {
        // (re)load the plan of the cursor's current item if it belongs to another token
        const int tkn = c.item < total_items ? c.item / num_chunks : -1;
        if (tkn != c.token) {
            c.token = tkn;
            c.plan_k = -1;
            c.sources = 0;
            if (tkn >= 0) {
                c.plan_k = lane < K ? __ldg(a.plan + static_cast<int64_t>(tkn) * K + lane) : -1;
                c.sources = __ballot_sync(0xffffffffu, c.plan_k >= 0);
            }
        }
        c.pending = c.sources;
    };
    auto set_range = [&](PullCursor& c, int base, int len) {
        c.item = base;
        c.range_end = min(total_items, base + len);
        if (c.item >= c.range_end) c.item = c.range_end = total_items;   // nothing left anywhere
        load_token(c);
    };
    // producer: move to its next range (claims one); returns false when the queue is too full to claim right now
    auto producer_next_range = [&](PullCursor& c) -> bool {
        if (claimed - started >= static_cast<uint32_t>(kCombineQueue - 8)) return false;
        if (c.item >= total_items) return true;   // exhausted: stay there
        int len;
        const int base = claim_range(len);
        set_range(c, base, len);
        return true;
    };

    if (alive) {
        PullCursor prod{0, 0, -1, -1, 0, 0}, cons{0, 0, -1, -1, 0, 0};
        {
            int len;
            const int base = claim_range(len);
            set_range(prod, base, len);
        }
        uint32_t issued = 0, consumed = 0;   // loads issued / consumed by this warp; buffer = counter % ring

        // issue loads in sequence order until the ring is full or the warp's work is exhausted
        auto issue_ahead = [&]() {
            while (issued - consumed < static_cast<uint32_t>(ring) && prod.item < total_items) {
                if (prod.pending == 0) {
                    if (prod.item + 1 >= prod.range_end) {
                        prod.item = prod.range_end;
                        if (!producer_next_range(prod)) {
                            prod.item = prod.range_end - 1;   // retry the claim on the next call
                            break;
                        }
                    } else {
                        ++prod.item;
                        load_token(prod);
                    }
                    continue;
                }
                const int k = __ffs(prod.pending) - 1;
                prod.pending &= prod.pending - 1;
                const int p = __shfl_sync(0xffffffffu, prod.plan_k, k);
                if (lane == 0) {
                    const int c = prod.item % num_chunks;
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

        // consumer: pop the next claimed range (making the producer claim one if it has not run ahead)
        auto consumer_next_range = [&](PullCursor& c) {
            if (started == claimed) {
                // the producer has used up all its claims too: it sits at the end of its current range
                int len;
                const int base = claim_range(len);
                set_range(prod, base, len);
            }
            const int base = s_queue[started % kCombineQueue], len = s_qlen[started % kCombineQueue];
            ++started;
            set_range(c, base, len);
        };
        consumer_next_range(cons);
        for (; cons.item < total_items && alive;) {
            const int t = cons.token, c = cons.item % num_chunks;
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
            if (cons.item + 1 >= cons.range_end) consumer_next_range(cons);
            else {
                ++cons.item;
                load_token(cons);
            }
        }
        // loads still in flight belong to nobody once the loop was left early: give them time to land so that no
        // copy arrives in shared memory after the CTA has exited
        for (; consumed < issued; ++consumed) mbar_drain(&s_bar[consumed % ring], (consumed / ring) & 1, 1000ull * 1000 * 1000);
    }

    stamp(2);
    // the last CTA to finish closes the call: new entry-barrier sequence, claim counter back to zero
    if (!arrive_is_last(&ws->arrive[EP_CH_COMBINE][0])) return;
    if (tid == 0) {
        if (a.prof != nullptr) a.prof[3] = globaltimer_ns();
        atomicExch(&ws->dyn_counter[EP_CH_COMBINE], 0u);
        ws->comb_seq = entry_seq;
        ws->epoch[EP_CH_COMBINE] += 1;
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

// column chunk = 512 B x unroll: larger chunks amortise the per-chunk bookkeeping: 3584 B when the row divides evenly
// (hidden 7168), else 2048 B
inline int pick_unroll(const CombineArgs& a) {
    const int row_bytes = a.hidden * 2;
    if (row_bytes % 3584 == 0) return 7;
    return row_bytes % 2048 == 0 ? 4 : (row_bytes % 1024 == 0 ? 2 : (row_bytes >= 2048 ? 4 : 1));
}

}  // namespace

LaunchShape combine_launch_shape(const CombineArgs& a, int num_sms) {
    LaunchShape s;
    s.num_ctas = num_sms < 1 ? 1 : (num_sms > EP_MAX_CTAS ? EP_MAX_CTAS : num_sms);
    const CombineSmemPlan p = combine_smem_plan(512 * pick_unroll(a), kCombineMaxWarps);
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
        // no CTA waits on another CTA of its own rank, so a plain launch is enough (and can share the GPU with a
        // compute kernel that is already running)
        void* params[] = {const_cast<CombineArgs*>(&a0)};
        return cudaLaunchKernel(fn, grid, block, params, shape.smem_bytes, stream);
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
