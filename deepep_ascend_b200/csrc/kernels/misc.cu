// Small stand-alone kernels: the cross-GPU barrier, a bounded-wait self test, the routing-layout kernel behind
// get_dispatch_layout, and a stand-alone bf16 -> e4m3 (1x128 scales) cast.
// Parity: barrier_impl (deep_ep/include/deep_ep/impls/barrier.cuh:11-40), get_dispatch_layout
// (csrc/kernels/legacy/layout.cu:10-150), per_token_cast_to_fp8 (deep_ep/utils/math.py:30-39).
#include "common.cuh"

namespace ep {

namespace {

__device__ __forceinline__ void barrier_body(const RankCtx& ctx, int channel) {
    Workspace* ws = local_ws(ctx);
    if (is_aborted(ws)) return;
    xgpu_barrier(ctx, ws, channel, EP_PH_XGPU_BARRIER);
    if (threadIdx.x == 0) ws->epoch[channel] += 1;
}
__global__ void barrier_kernel(const __grid_constant__ RankCtx ctx, uint64_t channel) { barrier_body(ctx, static_cast<int>(channel)); }
__global__ void barrier_kernel_multi(const RankCtx* ctxs, uint64_t channel) { barrier_body(ctxs[blockIdx.y], static_cast<int>(channel)); }

// Waits (bounded) until tile_flags[0] of the local workspace reaches `expected`.  Nothing in the library sets
// that word, so with a short limit this exercises the timeout -> status -> abort path without any fault.
__device__ __forceinline__ void wait_flag_body(const RankCtx& ctx, uint64_t expected) {
    Workspace* ws = local_ws(ctx);
    const uint64_t* flag = &ws->tile_flags[0];
    if (threadIdx.x == 0)
        bounded_wait(
            ctx, ws, EP_PH_TEST_FLAG, ctx.rank, expected, [&] { return ptx::ld_acquire_sys(flag) >= expected; },
            [&] { return ptx::ld_relaxed_sys(flag); });
}
__global__ void wait_flag_kernel(const __grid_constant__ RankCtx ctx, uint64_t expected) { wait_flag_body(ctx, expected); }
__global__ void wait_flag_kernel_multi(const RankCtx* ctxs, uint64_t expected) { wait_flag_body(ctxs[blockIdx.y], expected); }

// One thread per token; block-level shared histograms, then one global atomic per (block, bin).
__global__ void layout_kernel(const LayoutArgs a) {
    extern __shared__ uint32_t hist[];   // [E + R]
    const int E = a.num_experts, R = a.num_ranks, K = a.num_topk, El = E / R;
    for (int i = threadIdx.x; i < E + R; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < a.num_tokens) {
        uint32_t rank_mask = 0;
        for (int k = 0; k < K; ++k) {
            const int64_t i = static_cast<int64_t>(t) * K + k;
            const int e = a.idx_is_64 ? static_cast<int>(reinterpret_cast<const long long*>(a.topk_idx)[i])
                                      : reinterpret_cast<const int*>(a.topk_idx)[i];
            if (e >= 0 && e < E) {
                atomicAdd(&hist[e], 1u);
                rank_mask |= 1u << (e / El);
            }
        }
        for (int r = 0; r < R; ++r) {
            const bool in = (rank_mask >> r) & 1u;
            a.is_token_in_rank[static_cast<int64_t>(t) * R + r] = in;
            if (in) atomicAdd(&hist[E + r], 1u);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < E + R; i += blockDim.x) {
        const uint32_t n = hist[i];
        if (n == 0) continue;
        if (i < E) atomicAdd(reinterpret_cast<unsigned int*>(a.num_tokens_per_expert) + i, n);
        else atomicAdd(reinterpret_cast<unsigned int*>(a.num_tokens_per_rank) + (i - E), n);
    }
}

// One warp per token row; 16 lanes share one 128-channel scale.
__global__ void quant_kernel(const QuantArgs a) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= a.num_tokens) return;
    const int H = a.hidden;
    const uint8_t* in = reinterpret_cast<const uint8_t*>(a.x) + static_cast<int64_t>(t) * H * 2;
    uint8_t* out = reinterpret_cast<uint8_t*>(a.q) + static_cast<int64_t>(t) * H;
    const int iters = (H + 255) / 256;
    for (int i = 0; i < iters; ++i) {
        const int elem = (i * 32 + lane) * 8;
        const bool in_range = elem < H;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.f;
        if (in_range) {
            const int4 raw = ptx::ld_nc_v4(in + elem * 2);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(h[j]);
                v[2 * j] = f.x;
                v[2 * j + 1] = f.y;
            }
        }
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
        amax = fmaxf(ptx::warp_max_16(amax), 1e-4f);
        float scale, sf;
        if (a.round_scale || a.use_ue8m0) {
            // dequantization factor rounded up to a power of two
            const float raw = __fdiv_rn(amax, 448.f);
            const int exp = static_cast<int>((__float_as_uint(raw) >> 23) & 0xff) + ((__float_as_uint(raw) & 0x7fffff) ? 1 : 0);
            sf = __uint_as_float(static_cast<uint32_t>(exp) << 23);
            scale = __uint_as_float(static_cast<uint32_t>(254 - exp) << 23);
        } else {
            scale = __fmul_rn(448.f, __frcp_rn(amax));   // what PyTorch computes for `448.0 / amax`
            sf = __fdiv_rn(amax, 448.f);
        }
        if (in_range) {
            uint32_t packed[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j] * scale, v[4 * j + 1] * scale),
                                                              __NV_SATFINITE, __NV_E4M3);
                const uint32_t hi = __nv_cvt_float2_to_fp8x2(
                    make_float2(v[4 * j + 2] * scale, v[4 * j + 3] * scale), __NV_SATFINITE, __NV_E4M3);
                packed[j] = lo | (hi << 16);
            }
            *reinterpret_cast<uint2*>(out + elem) = make_uint2(packed[0], packed[1]);
            if ((lane & 15) == 0) {
                const int g = elem / 128;
                if (a.use_ue8m0) {
                    uint8_t* p = reinterpret_cast<uint8_t*>(a.sf) + (static_cast<int64_t>(t) * a.sf_stride_row + (g / 4) * a.sf_stride_col) * 4 + (g & 3);
                    *p = static_cast<uint8_t>(__float_as_uint(sf) >> 23);
                } else {
                    a.sf[static_cast<int64_t>(t) * a.sf_stride_row + g * a.sf_stride_col] = sf;
                }
            }
        }
    }
}

// Engram fetch: one warp per requested entry; the entry is pulled from its owner's storage (TMA bulk load through
// the peer mapping, or from the owner's CPU segment, no multicast) into shared memory and bulk-stored into the local
// output row.  Parity: deep_ep/include/deep_ep/impls/engram_fetch.cuh:46-82 (payload get + local scale gather).
__device__ __forceinline__ void engram_fetch_body(const EngramFetchArgs& a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const RankCtx& ctx = a.ctx;
    Workspace* ws = local_ws(ctx);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, num_warps = blockDim.x >> 5;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem) + warp * 2;
    const int stage_bytes = (a.entry_bytes + 127) / 128 * 128;
    uint8_t* stage = smem + 1024 + static_cast<size_t>(warp) * 2 * stage_bytes;
    if (lane == 0) {
        ptx::mbar_init(&bars[0], 1);
        ptx::mbar_init(&bars[1], 1);
    }
    ptx::mbar_fence_init();
    __syncthreads();
    ptx::fence_proxy_async_smem();
    bool alive = !is_aborted(ws);
    uint32_t n = 0;
    for (int i = blockIdx.x * num_warps + warp; i < a.num_fetches && alive; i += gridDim.x * num_warps, ++n) {
        const int id = a.indices[i];
        const int owner = id / a.entries_per_rank, local = id - owner * a.entries_per_rank;
        const int st = n & 1;
        ptx::bulk_wait_read<1>();   // the stage was the source of the store issued two entries ago
        __syncwarp();
        if (owner < 0 || owner >= ctx.num_ranks) {
            if (lane == 0) report_failure(ctx, ws, EP_ERR_BOUNDS, EP_PH_TILE_FLAG, owner, ctx.num_ranks, id);
            alive = false;
            break;
        }
        if (lane == 0) {
            ptx::mbar_arrive_expect_tx(&bars[st], a.entry_bytes);
            ptx::bulk_load(stage + st * stage_bytes, a.storage[owner] + static_cast<int64_t>(local) * a.entry_bytes, a.entry_bytes, &bars[st]);
        }
        if (a.sf_table != nullptr) {
            // the scales of the entry come from the local copy of the replicated table while the payload is in flight
            const int token = i / a.entries_per_token, entry = i - token * a.entries_per_token;
            for (int p = lane; p < a.sf_packs; p += 32)
                a.fetched_sf[token * a.sf_token_stride + static_cast<int64_t>(entry * a.sf_packs + p) * a.sf_pack_stride] =
                    __ldg(a.sf_table + static_cast<int64_t>(id) * a.sf_packs + p);
        }
        alive = mbar_wait_bounded(ctx, ws, &bars[st], (n >> 1) & 1, EP_PH_COMBINE_LOAD);
        if (!alive) break;
        if (lane == 0)
            ptx::bulk_store(reinterpret_cast<uint8_t*>(a.out) + static_cast<int64_t>(i) * a.entry_bytes, stage + st * stage_bytes, a.entry_bytes);
        ptx::bulk_commit();
    }
    ptx::bulk_commit();
    ptx::bulk_wait<0>();
}
__global__ void engram_fetch_kernel(const __grid_constant__ EngramFetchArgs a) { engram_fetch_body(a); }
__global__ void engram_fetch_kernel_multi(const EngramFetchArgs* a) { engram_fetch_body(a[blockIdx.y]); }

// out[i] = sum over slots of slots[s][i], accumulated in fp32 in slot order
__global__ void reduce_slots_kernel(const ReduceSlotsArgs a) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < a.n; i += stride) {
        float acc = 0.f;
        for (int s = 0; s < a.num_slots; ++s)
            acc += a.is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.slots)[s * a.n + i])
                             : reinterpret_cast<const float*>(a.slots)[s * a.n + i];
        if (a.is_bf16) reinterpret_cast<__nv_bfloat16*>(a.out)[i] = __float2bfloat16_rn(acc);
        else reinterpret_cast<float*>(a.out)[i] = acc;
    }
}

template <typename T>
cudaError_t launch_small(const void* single, const void* multi, const T* items, int n, dim3 block, cudaStream_t stream,
                         uint64_t extra, bool has_extra) {
    if (n == 1) {
        void* params[] = {const_cast<T*>(items), &extra};
        return cudaLaunchKernel(single, dim3(1, 1, 1), block, params, 0, stream);
    }
    T* dev = nullptr;
    cudaError_t err = cudaMallocAsync(reinterpret_cast<void**>(&dev), sizeof(T) * n, stream);
    if (err != cudaSuccess) return err;
    err = cudaMemcpyAsync(dev, items, sizeof(T) * n, cudaMemcpyHostToDevice, stream);
    if (err == cudaSuccess) {
        void* params[] = {&dev, &extra};
        // the n single-CTA virtual ranks wait on one another: cooperative launch keeps them co-resident
        err = cudaLaunchCooperativeKernel(multi, dim3(1, n, 1), block, params, 0, stream);
    }
    cudaFreeAsync(dev, stream);
    (void)has_extra;
    return err;
}

}  // namespace

cudaError_t launch_barrier(const RankCtx* ctxs, int n, int channel, cudaStream_t stream) {
    if (channel < 0 || channel >= EP_NUM_CHANNELS) return cudaErrorInvalidValue;
    return launch_small<RankCtx>((const void*)barrier_kernel, (const void*)barrier_kernel_multi, ctxs, n, dim3(32, 1, 1),
                                 stream, static_cast<uint64_t>(channel), true);
}

cudaError_t launch_wait_flag_test(const RankCtx* ctxs, int n, uint64_t expected, cudaStream_t stream) {
    return launch_small<RankCtx>((const void*)wait_flag_kernel, (const void*)wait_flag_kernel_multi, ctxs, n,
                                 dim3(32, 1, 1), stream, expected, true);
}

cudaError_t launch_engram_fetch(const EngramFetchArgs* args, int n, int num_sms, cudaStream_t stream) {
    const int warps = 4;
    const int stage_bytes = (args[0].entry_bytes + 127) / 128 * 128;
    const int smem = 1024 + warps * 2 * stage_bytes;
    if (smem > 200 * 1024 || args[0].entry_bytes % 16 != 0) return cudaErrorInvalidValue;
    const void* fn = n == 1 ? (const void*)engram_fetch_kernel : (const void*)engram_fetch_kernel_multi;
    cudaError_t err = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return err;
    dim3 grid(num_sms < 1 ? 1 : num_sms, n, 1), block(warps * 32, 1, 1);
    if (n == 1) {
        void* params[] = {const_cast<EngramFetchArgs*>(args)};
        return cudaLaunchKernel(fn, grid, block, params, smem, stream);
    }
    EngramFetchArgs* dev = nullptr;
    err = cudaMallocAsync(reinterpret_cast<void**>(&dev), sizeof(EngramFetchArgs) * n, stream);
    if (err != cudaSuccess) return err;
    err = cudaMemcpyAsync(dev, args, sizeof(EngramFetchArgs) * n, cudaMemcpyHostToDevice, stream);
    if (err == cudaSuccess) {
        void* params[] = {&dev};
        err = cudaLaunchKernel(fn, grid, block, params, smem, stream);
    }
    cudaFreeAsync(dev, stream);
    return err;
}

cudaError_t launch_reduce_slots(const ReduceSlotsArgs& a, cudaStream_t stream) {
    if (a.n == 0) return cudaSuccess;
    const int threads = 256;
    const int64_t want = (a.n + threads - 1) / threads;
    const int blocks = static_cast<int>(want < 148 * 8 ? want : 148 * 8);
    reduce_slots_kernel<<<blocks, threads, 0, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_layout(const LayoutArgs& a, cudaStream_t stream) {
    const int threads = 256;
    const int blocks = (a.num_tokens + threads - 1) / threads;
    if (blocks == 0) return cudaSuccess;
    layout_kernel<<<blocks, threads, (a.num_experts + a.num_ranks) * sizeof(uint32_t), stream>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_quant(const QuantArgs& a, cudaStream_t stream) {
    const int warps = 8;
    const int blocks = (a.num_tokens + warps - 1) / warps;
    if (blocks == 0) return cudaSuccess;
    quant_kernel<<<blocks, warps * 32, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace ep
