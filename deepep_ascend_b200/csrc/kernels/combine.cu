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
#include "common.cuh"

namespace ep {

namespace {

constexpr int kCombineMaxWarps = 12;
constexpr int kCombineSlots = 2;
constexpr int kCombineSmemBudget = 216 * 1024;

template <int kUnroll>
struct CombineCfg {
    static constexpr int kChunkBytes = 32 * 16 * kUnroll;
};

__host__ __device__ inline int combine_slot_bytes(int K, int chunk_bytes) { return K * chunk_bytes; }

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

    uint8_t** s_peer = reinterpret_cast<uint8_t**>(smem);
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + EP_MAX_RANKS * 8) + warp * kCombineSlots;
    uint8_t* s_data = smem + 1024 + static_cast<size_t>(warp) * kCombineSlots * combine_slot_bytes(K, kChunk);

    if (tid < EP_MAX_RANKS) s_peer[tid] = tid < ctx.num_ranks ? ctx.peer_base[tid] : nullptr;
    if (lane == 0)
        for (int s = 0; s < kCombineSlots; ++s) ptx::mbar_init(&s_bar[s], 1);
    ptx::mbar_fence_init();
    __syncthreads();
    ptx::fence_proxy_async_smem();

    // every rank's input rows must be in place before anyone pulls
    bool alive = !is_aborted(ws);
    if (blockIdx.x == 0) alive = xgpu_barrier(ctx, ws, EP_CH_COMBINE, EP_PH_COMBINE_ENTRY) && alive;
    alive = grid_sync(ctx, ws, EP_CH_COMBINE, EP_PH_GRID_SYNC) && alive;

    const int64_t num_items = static_cast<int64_t>(T) * num_chunks;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * num_warps;
    const int64_t first = static_cast<int64_t>(blockIdx.x) * num_warps + warp;

    // issue the loads of item `it` into slot `slot`; returns this lane's plan entry for the item
    auto issue = [&](int64_t it, int slot) -> int {
        const int t = static_cast<int>(it / num_chunks), c = static_cast<int>(it % num_chunks);
        const int p = lane < K ? a.plan[static_cast<int64_t>(t) * K + lane] : -1;
        const int bytes = min(kChunk, row_bytes - c * kChunk);
        const uint32_t srcs = __ballot_sync(0xffffffffu, p >= 0);
        // always arrive (with 0 bytes for an item without sources) so the slot's phase advances once per item
        if (lane == 0) ptx::mbar_arrive_expect_tx(&s_bar[slot], __popc(srcs) * bytes);
        __syncwarp();
        if (p >= 0) {
            const uint8_t* src = s_peer[p >> 24] + a.off_x + static_cast<int64_t>(p & 0xffffff) * row_bytes +
                                 static_cast<int64_t>(c) * kChunk;
            ptx::bulk_load(s_data + (slot * K + lane) * kChunk, src, bytes, &s_bar[slot]);
        }
        return p;
    };

    if (alive) {
        int plan_q[kCombineSlots];   // this lane's plan entry of the item held by each slot
#pragma unroll
        for (int s = 0; s < kCombineSlots - 1; ++s) {
            const int64_t it = first + s * stride;
            plan_q[s] = it < num_items ? issue(it, s) : -1;
        }
        int64_t n = 0;
        for (int64_t it = first; it < num_items && alive; it += stride, ++n) {
            const int slot = static_cast<int>(n % kCombineSlots);
            const uint32_t parity = static_cast<uint32_t>((n / kCombineSlots) & 1);
            // prefetch the item that is kSlots-1 ahead into the slot that was consumed last iteration
            {
                const int64_t ahead = it + (kCombineSlots - 1) * stride;
                const int aslot = static_cast<int>((n + kCombineSlots - 1) % kCombineSlots);
                const int p = ahead < num_items ? issue(ahead, aslot) : -1;
#pragma unroll
                for (int s = 0; s < kCombineSlots; ++s)
                    if (s == aslot) plan_q[s] = p;
            }
            int plan_k = -1;
#pragma unroll
            for (int s = 0; s < kCombineSlots; ++s)
                if (s == slot) plan_k = plan_q[s];
            const int t = static_cast<int>(it / num_chunks), c = static_cast<int>(it % num_chunks);
            const int bytes = min(kChunk, row_bytes - c * kChunk);
            const int col0 = c * kChunk;   // byte offset inside the row

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

            const uint32_t srcs = __ballot_sync(0xffffffffu, plan_k >= 0);
            alive = mbar_wait_bounded(ctx, ws, &s_bar[slot], parity, EP_PH_COMBINE_LOAD);
            if (!alive) break;
            for (int k = 0; k < K; ++k) {
                if (!((srcs >> k) & 1u)) continue;
                const float w = __shfl_sync(0xffffffffu, mul_k, k);
                const uint8_t* buf = s_data + (slot * K + k) * kChunk;
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
            }
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
            ptx::fence_proxy_async_smem();
            __syncwarp();   // every lane is done with this slot before the next iteration refills it
        }
    }

    // nobody may overwrite its input rows until every rank has finished pulling
    const bool cta_ok = __syncthreads_and(alive ? 1 : 0) != 0;
    alive = grid_sync(ctx, ws, EP_CH_COMBINE, EP_PH_GRID_SYNC) && cta_ok;
    if (blockIdx.x == 0) {
        if (alive) xgpu_barrier(ctx, ws, EP_CH_COMBINE, EP_PH_COMBINE_EXIT);
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

inline int pick_unroll(const CombineArgs& a) {
    const int row_bytes = a.hidden * 2;
    return row_bytes % 2048 == 0 ? 4 : (row_bytes % 1024 == 0 ? 2 : (row_bytes >= 2048 ? 4 : 1));
}

}  // namespace

LaunchShape combine_launch_shape(const CombineArgs& a, int num_sms) {
    LaunchShape s;
    s.num_ctas = num_sms < 1 ? 1 : (num_sms > EP_MAX_CTAS ? EP_MAX_CTAS : num_sms);
    const int chunk = 512 * pick_unroll(a);
    const int per_warp = kCombineSlots * combine_slot_bytes(a.num_topk, chunk);
    s.num_warps = kCombineMaxWarps;
    while (s.num_warps > 1 && 1024 + s.num_warps * per_warp > kCombineSmemBudget) --s.num_warps;
    s.smem_bytes = 1024 + s.num_warps * per_warp;
    return s;
}

cudaError_t launch_combine(const CombineArgs* args, int n, int num_sms, cudaStream_t stream) {
    const CombineArgs& a0 = args[0];
    const LaunchShape shape = combine_launch_shape(a0, num_sms);
    if (shape.smem_bytes > 227 * 1024) return cudaErrorInvalidValue;
    const int unroll = pick_unroll(a0);
    const void* fn;
    if (n == 1)
        fn = unroll == 4 ? (const void*)combine_kernel<4> : unroll == 2 ? (const void*)combine_kernel<2> : (const void*)combine_kernel<1>;
    else
        fn = unroll == 4 ? (const void*)combine_kernel_multi<4>
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
