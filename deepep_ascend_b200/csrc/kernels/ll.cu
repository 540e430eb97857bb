// Low-latency dispatch / combine for decode-sized batches (graph-capturable: no host sync, no allocation, all
// protocol state lives in device memory and is epoch-tagged so nothing has to be cleaned between calls).
//
// Dispatch:  SEND  - one token per CTA iteration: all warps cast the token bf16 -> e4m3 (1x128 scales; fp32,
//                    power-of-two or UE8M0) into a message {16 B header, payload, scales} in shared memory, then
//                    warp k claims a slot for expert topk[k] and bulk-stores the message into the slab
//                    [local expert][source rank][slot] of the expert's rank through its peer mapping;
//                    the last CTA to have its stores acknowledged sends the per-expert counts as epoch-tagged words.
//            RECV  - every CTA waits for all counts, forms one prefix sum over the received messages and copies an
//                    equal share of them into [local expert, ranks * max_tokens, hidden] (+ column-major scales,
//                    source info, ranges).
// Combine:   SEND  - the packed rows of all local experts form one list shared evenly by the staging warps of all
//                    CTAs: every row is bulk-copied into the slot [source token][top-k lane] of the token's home
//                    rank; the last CTA to finish raises one epoch-tagged flag per rank pair.
//            RECV  - wait for all ranks' flags, then out[t] = sum_k w[t,k] * slot[t,k] in fp32 -> bf16.
// No CTA waits for another CTA of its own rank (no grid barrier): phases end with an arrival counter whose last
// arriver does the publishing.
// SEND and RECV can be launched separately (phases argument) so that no SM is held while data is in flight.
//
// Parity: csrc/kernels/legacy/internode_ll.cu:128-554 (dispatch) and 714-1238 (combine) of the reference.
#include "common.cuh"
#include "logfmt.cuh"

namespace ep {

namespace {

constexpr int kLLThreads = 512;
constexpr int kLLWarps = kLLThreads / 32;
constexpr int kLLCombineSmemBudget = 200 * 1024;

// warps of a CTA that stage combine rows (two bf16 rows of shared memory each, plus one word per 128 channels for the
// range headers of the LogFMT coding)
__host__ __device__ inline int ll_combine_hdr_bytes(int hidden) { return ((hidden + 127) / 128 * 4 + 15) / 16 * 16; }
__host__ __device__ inline int ll_combine_send_warps(int hidden) {
    const int w = (kLLCombineSmemBudget - 1024) / (2 * hidden * 2 + ll_combine_hdr_bytes(hidden));
    return w < 1 ? 1 : (w > kLLWarps ? kLLWarps : w);
}

__device__ __forceinline__ int ll_load_idx(const void* p, int is64, int64_t i) {
    return is64 ? static_cast<int>(__ldg(reinterpret_cast<const long long*>(p) + i)) : __ldg(reinterpret_cast<const int*>(p) + i);
}

__device__ __forceinline__ bool rank_masked(const int32_t* mask, int r) {
    return mask != nullptr && *reinterpret_cast<const volatile int32_t*>(mask + r) != 0;
}

// 8 bf16 values held by each lane -> 8 e4m3 bytes + the dequantization scale of the lane's 128-channel group
__device__ __forceinline__ uint2 cast_8(const float (&v)[8], int round_scale, float& sf) {
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    amax = fmaxf(ptx::warp_max_16(amax), 1e-4f);
    float scale;
    if (round_scale) {
        const float raw = __fdiv_rn(amax, 448.f);
        const int exp = static_cast<int>((__float_as_uint(raw) >> 23) & 0xff) + ((__float_as_uint(raw) & 0x7fffff) ? 1 : 0);
        sf = __uint_as_float(static_cast<uint32_t>(exp) << 23);
        scale = __uint_as_float(static_cast<uint32_t>(254 - exp) << 23);
    } else {
        scale = __fmul_rn(448.f, __frcp_rn(amax));
        sf = __fdiv_rn(amax, 448.f);
    }
    uint32_t packed[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j] * scale, v[4 * j + 1] * scale), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j + 2] * scale, v[4 * j + 3] * scale), __NV_SATFINITE, __NV_E4M3);
        packed[j] = lo | (hi << 16);
    }
    return make_uint2(packed[0], packed[1]);
}

// In-place exclusive prefix sum of data[0, n) in shared memory (n <= 2 * blockDim.x); data[n] receives the total.
// Called by all threads of the CTA.
__device__ __forceinline__ void block_exclusive_scan(uint32_t* data, int n) {
    __shared__ uint32_t s_warp_total[kLLWarps];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t v0 = 2 * tid < n ? data[2 * tid] : 0u, v1 = 2 * tid + 1 < n ? data[2 * tid + 1] : 0u;
    uint32_t incl = v0 + v1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 31) s_warp_total[warp] = incl;
    __syncthreads();
    uint32_t base = 0;
    for (int w = 0; w < warp; ++w) base += s_warp_total[w];
    const uint32_t excl = base + incl - (v0 + v1);
    if (2 * tid < n) data[2 * tid] = excl;
    if (2 * tid + 1 < n) data[2 * tid + 1] = excl + v0;
    if (tid == blockDim.x - 1) data[n] = base + incl;
    __syncthreads();
}

// index of the segment that holds item g: largest p with pref[p] <= g (pref is an exclusive prefix sum of n counts)
__device__ __forceinline__ int find_segment(const uint32_t* pref, int n, uint32_t g) {
    int lo = 0, hi = n;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (pref[mid] <= g) lo = mid;
        else hi = mid;
    }
    return lo;
}

// Shrink mode: wait for a tagged word until the time limit; like every other wait it also gives up when the buffer has
// been aborted.  Returns whether the word arrived; running out of time is not an error here (the caller masks the rank).
__device__ __forceinline__ bool shrink_wait(const RankCtx& ctx, Workspace* ws, const uint64_t* sig, uint64_t epoch, uint64_t t0) {
    uint32_t spins = 0;
    while (!tag_matches(ptx::ld_acquire_sys(sig), epoch)) {
        if ((++spins & 31u) == 0u && (is_aborted(ws) || globaltimer_ns() - t0 > ctx.timeout_ns)) return false;
    }
    return true;
}

__device__ __forceinline__ void ll_dispatch_body(const LLDispatchArgs& a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const RankCtx& ctx = a.ctx;
    Workspace* ws = local_ws(ctx);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int R = ctx.num_ranks, me = ctx.rank, E = a.num_experts, El = E / R, K = a.num_topk, H = a.hidden;
    const int M = a.num_max_tokens, G = (H + 127) / 128;
    const uint64_t epoch = ws->epoch[EP_CH_LL_DISPATCH] + 1;
    const int set = static_cast<int>(epoch & 1);
    const int payload = a.use_fp8 ? H : 2 * H;
    __shared__ uint8_t* s_peer[EP_MAX_RANKS];
    __shared__ uint32_t s_pref[EP_MAX_EXPERTS + 1];   // counts, then exclusive prefix, of the (local expert, source) pairs
    if (tid < EP_MAX_RANKS) s_peer[tid] = tid < R ? ctx.peer_base[tid] : nullptr;
    __syncthreads();
    bool alive = !is_aborted(ws);
    uint32_t* slot_counter = ws->ll_counters[0];
    auto stamp = [&](int i) {
        if (a.prof != nullptr && blockIdx.x == 0 && tid == 0) a.prof[i] = globaltimer_ns();
    };
    stamp(0);

    if (a.phases & EP_LL_SEND) {
        if (blockIdx.x == 0)
            for (int j = tid; j < El; j += blockDim.x) a.packed_count[j] = 0;
        const uint8_t* xb = reinterpret_cast<const uint8_t*>(a.x);
        int n = 0;
        for (int t = blockIdx.x; t < a.num_tokens; t += gridDim.x, ++n) {
            uint8_t* msg = smem + (n & 1) * a.msg_bytes;
            // the message buffer about to be rewritten was the source of the stores issued two tokens ago
            ptx::bulk_wait_read<1>();
            __syncthreads();
            if (a.use_fp8) {
                float* sf_out = reinterpret_cast<float*>(msg + 16 + H);
                for (int i = warp; i * 256 < H; i += kLLWarps) {
                    const int elem = (i * 32 + lane) * 8;
                    float v[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = 0.f;
                    if (elem < H) {
                        const int4 raw = ptx::ld_nc_v4(xb + (static_cast<int64_t>(t) * H + elem) * 2);
                        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 f = __bfloat1622float2(h[j]);
                            v[2 * j] = f.x;
                            v[2 * j + 1] = f.y;
                        }
                    }
                    float sf;
                    const uint2 q = cast_8(v, a.round_scale | a.use_ue8m0, sf);
                    if (elem < H) {
                        *reinterpret_cast<uint2*>(msg + 16 + elem) = q;
                        if ((lane & 15) == 0) sf_out[elem / 128] = sf;
                    }
                }
            } else {
                for (int off = tid * 16; off < payload; off += blockDim.x * 16)
                    *reinterpret_cast<int4*>(msg + 16 + off) = ptx::ld_nc_v4(xb + static_cast<int64_t>(t) * payload + off);
            }
            ptx::fence_proxy_async_smem();
            __syncthreads();
            if (warp < K && lane == 0) {
                const int e = ll_load_idx(a.topk_idx, a.idx_is_64, static_cast<int64_t>(t) * K + warp);
                if (e >= 0 && e < E && !rank_masked(a.mask, e / El)) {
                    const uint32_t slot = atomicAdd(&slot_counter[e], 1u);
                    if (slot < static_cast<uint32_t>(M)) {
                        uint8_t* dst = s_peer[e / El] + a.off_slab[set] +
                                       ((static_cast<int64_t>(e % El) * R + me) * M + slot) * a.msg_bytes;
                        // header word 1 carries the top-k lane; it differs per destination, so it goes out as a
                        // separate 16-byte store after the bulk copy of the shared message body
                        ptx::bulk_store(dst + 16, msg + 16, a.msg_bytes - 16);
                        *reinterpret_cast<int4*>(dst) = make_int4(t, warp, 0, 0);
                    } else {
                        report_failure(ctx, ws, EP_ERR_BOUNDS, EP_PH_LL_RECV_COUNT, e / El, M, slot);
                    }
                }
                ptx::bulk_commit();
            }
        }
        ptx::bulk_commit();
        stamp(1);
        ptx::bulk_wait<0>();
        __threadfence_system();
        stamp(2);
        // No grid barrier: the last CTA of this rank to finish its sends publishes how many messages every expert got
        // from this rank (a tagged zero means "none"); the others go straight on to the receive phase.
        if (arrive_is_last(&ws->arrive[EP_CH_LL_DISPATCH][0]) && !is_aborted(ws)) {
            for (int e = tid; e < E; e += blockDim.x) {
                const uint32_t n_sent = min(__ldcg(&slot_counter[e]), static_cast<uint32_t>(M));
                __stcg(&slot_counter[e], 0u);
                if (!rank_masked(a.mask, e / El)) {
                    Workspace* pws = reinterpret_cast<Workspace*>(s_peer[e / El]);
                    ptx::st_release_sys(&pws->ll_signal[0][(e % El) * R + me], tag_value(epoch, n_sent));
                }
            }
            if (a.prof != nullptr && tid == 0) a.prof[3] = globaltimer_ns();
        }
    }

    if (a.phases & EP_LL_RECV) {
        const uint8_t* slab = s_peer[me] + a.off_slab[set];
        const int64_t rows_per_expert = static_cast<int64_t>(R) * M;
        // Every CTA waits for the counts of all (local expert, source rank) pairs, turns them into one prefix sum over
        // all received messages and then takes an equal share of the (message, 2 KB piece) copy items, so no CTA is left
        // with a long pair.  The packed position of a source's messages inside its expert is the sum of the counts of
        // the lower sources.
        const int P = El * R;
        int ok = alive ? 1 : 0;
        for (int p = tid; p < P && alive; p += blockDim.x) {
            const int src = p % R;
            uint32_t n_recv = 0;
            if (!rank_masked(a.mask, src)) {
                const uint64_t* sig = &ws->ll_signal[0][p];
                const uint64_t t0 = globaltimer_ns();
                if (a.shrink) {
                    // shrink mode: a source that stays silent is masked out instead of failing the call
                    const bool got = shrink_wait(ctx, ws, sig, epoch, t0);
                    if (!got && !is_aborted(ws)) atomicExch(a.mask + src, 1);
                    if (got) n_recv = count_low32(ptx::ld_relaxed_sys(sig));
                } else {
                    const int got = bounded_wait(
                        ctx, ws, EP_PH_LL_RECV_COUNT, src, epoch, [&] { return tag_matches(ptx::ld_acquire_sys(sig), epoch); },
                        [&] { return ptx::ld_relaxed_sys(sig); });
                    if (got) n_recv = count_low32(ptx::ld_relaxed_sys(sig));
                    else ok = 0;
                }
                if (a.wait_stats != nullptr && blockIdx.x == 0)
                    atomicAdd(reinterpret_cast<unsigned long long*>(a.wait_stats + src), globaltimer_ns() - t0);
            }
            s_pref[p] = n_recv;
        }
        alive = __syncthreads_and(ok) != 0;
        stamp(4);
        if (alive) {
            block_exclusive_scan(s_pref, P);
            if (blockIdx.x == 0) {
                for (int p = tid; p < P; p += blockDim.x) {
                    const int j = p / R;
                    a.layout_range[p] = (static_cast<int64_t>(s_pref[p] - s_pref[j * R]) << 32) | (s_pref[p + 1] - s_pref[p]);
                    if (p % R == 0) {
                        const uint32_t total = s_pref[(j + 1) * R] - s_pref[j * R];
                        a.packed_count[j] = total;
                        if (a.stats != nullptr) a.stats[j] += total;
                    }
                }
            }
            const uint32_t pieces = (payload + 2047) / 2048;
            const uint32_t items = s_pref[P] * pieces;
            for (uint32_t u = blockIdx.x * kLLWarps + warp; u < items; u += gridDim.x * kLLWarps) {
                const uint32_t g = u / pieces, c = u - g * pieces;
                const int p = find_segment(s_pref, P, g);
                const int j = p / R;
                const uint32_t i = g - s_pref[p], begin = s_pref[p] - s_pref[j * R];
                const uint8_t* m = slab + (static_cast<int64_t>(p) * M + i) * a.msg_bytes;
                const int64_t pos = static_cast<int64_t>(j) * rows_per_expert + begin + i;
                uint8_t* out = reinterpret_cast<uint8_t*>(a.packed_x) + pos * payload;
                {
                    const int off = c * 2048 + lane * 16;
                    int4 v[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (off + q * 512 < payload) v[q] = __ldcg(reinterpret_cast<const int4*>(m + 16 + off + q * 512));
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (off + q * 512 < payload) *reinterpret_cast<int4*>(out + off + q * 512) = v[q];
                }
                if (c == 0 && lane == 0) {
                    const int4 hdr = __ldcg(reinterpret_cast<const int4*>(m));
                    a.packed_src_info[pos] = (hdr.y << 20) | hdr.x;
                }
                if (a.use_fp8 && c == pieces - 1) {
                    const float* sf = reinterpret_cast<const float*>(m + 16 + H);
                    if (a.use_ue8m0) {
                        // four exponents per int32, groups along the slow axis: [E_local, ceil(G/4), R*M]
                        uint8_t* dst = reinterpret_cast<uint8_t*>(a.packed_sf);
                        const int64_t G4 = (G + 3) / 4;
                        for (int gi = lane; gi < G; gi += 32)
                            dst[((static_cast<int64_t>(j) * G4 + gi / 4) * rows_per_expert + begin + i) * 4 + (gi & 3)] =
                                static_cast<uint8_t>(__float_as_uint(__ldcg(sf + gi)) >> 23);
                    } else {
                        float* dst = reinterpret_cast<float*>(a.packed_sf);
                        for (int gi = lane; gi < G; gi += 32)
                            dst[(static_cast<int64_t>(j) * G + gi) * rows_per_expert + begin + i] = __ldcg(sf + gi);
                    }
                }
            }
        }
        stamp(5);
        // the call is complete when the last CTA gets here (every CTA read the epoch before it arrived)
        if (arrive_is_last(&ws->arrive[EP_CH_LL_DISPATCH][1]) && tid == 0) {
            ws->epoch[EP_CH_LL_DISPATCH] = epoch;
            if (a.prof != nullptr) a.prof[6] = globaltimer_ns();
        }
    }
}


__device__ __forceinline__ void ll_combine_body(const LLCombineArgs& a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const RankCtx& ctx = a.ctx;
    Workspace* ws = local_ws(ctx);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int R = ctx.num_ranks, me = ctx.rank, E = a.num_experts, El = E / R, K = a.num_topk, H = a.hidden;
    const int M = a.num_max_tokens;
    const int row_bytes = 2 * H;
    const uint64_t epoch = ws->epoch[EP_CH_LL_COMBINE] + 1;
    const int set = static_cast<int>(epoch & 1);
    __shared__ uint8_t* s_peer[EP_MAX_RANKS];
    __shared__ uint32_t s_pref[EP_MAX_EXPERTS + 1], s_begin[EP_MAX_EXPERTS];
    if (tid < EP_MAX_RANKS) s_peer[tid] = tid < R ? ctx.peer_base[tid] : nullptr;
    // per warp: two staging rows and two mbarriers
    const int send_warps = ll_combine_send_warps(H);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem) + warp * 2;
    uint8_t* stage = smem + 1024 + static_cast<size_t>(warp < send_warps ? warp : 0) * 2 * row_bytes;
    uint32_t* hdr_scratch = reinterpret_cast<uint32_t*>(smem + 1024 + static_cast<size_t>(send_warps) * 2 * row_bytes +
                                                        static_cast<size_t>(warp < send_warps ? warp : 0) * ll_combine_hdr_bytes(H));
    const int wire_bytes = a.use_logfmt ? logfmt::wire_bytes(H) : row_bytes;   // what one row puts on the wire
    if (lane == 0) {
        ptx::mbar_init(&bars[0], 1);
        ptx::mbar_init(&bars[1], 1);
    }
    ptx::mbar_fence_init();
    __syncthreads();
    ptx::fence_proxy_async_smem();
    bool alive = !is_aborted(ws);
    auto stamp = [&](int i) {
        if (a.prof != nullptr && blockIdx.x == 0 && tid == 0) a.prof[i] = globaltimer_ns();
    };
    stamp(0);

    if (a.phases & EP_LL_SEND) {
        const uint8_t* xb = reinterpret_cast<const uint8_t*>(a.x);
        const int64_t rows_per_expert = static_cast<int64_t>(R) * M;
        uint32_t n_loaded = 0;   // loads issued by this warp so far (selects stage and mbarrier parity)
        // all packed rows of this rank form one list (prefix sum over the (local expert, source rank) pairs) that the
        // staging warps of all CTAs share evenly
        const int P = El * R;
        for (int p = tid; p < P; p += blockDim.x) {
            const int64_t lr = a.layout_range[p];
            s_pref[p] = rank_masked(a.mask, p % R) ? 0u : static_cast<uint32_t>(lr & 0xffffffffll);
            s_begin[p] = static_cast<uint32_t>(lr >> 32);
        }
        __syncthreads();
        block_exclusive_scan(s_pref, P);
        const uint32_t total = s_pref[P];
        // one row load is always in flight ahead of the row being stored
        const uint32_t g_stride = gridDim.x * send_warps;
        int next_src = 0;   // source rank of the row whose load was issued last
        auto issue_load = [&](uint32_t g, uint32_t n) {
            const int p = find_segment(s_pref, P, g);
            next_src = p % R;
            const int64_t pos = static_cast<int64_t>(p / R) * rows_per_expert + s_begin[p] + (g - s_pref[p]);
            if (lane == 0) {
                ptx::mbar_arrive_expect_tx(&bars[n & 1], row_bytes);
                ptx::bulk_load(stage + (n & 1) * row_bytes, xb + pos * row_bytes, row_bytes, &bars[n & 1]);
            }
            return pos;
        };
        uint32_t g = blockIdx.x * send_warps + warp;
        int64_t pos = 0;
        if (warp < send_warps && g < total && alive) pos = issue_load(g, 0);
        for (; warp < send_warps && g < total && alive; g += g_stride) {
            const int s = next_src;
            const int info = a.src_info[pos];
            const int t = info & 0xfffff, k = info >> 20;
            const int st = n_loaded & 1;
            int64_t next_pos = 0;
            if (g + g_stride < total) {
                // the other stage was the source of the previous row's store
                ptx::bulk_wait_read<0>();
                __syncwarp();
                next_pos = issue_load(g + g_stride, n_loaded + 1);
            }
            alive = mbar_wait_bounded(ctx, ws, &bars[st], (n_loaded >> 1) & 1, EP_PH_COMBINE_LOAD);
            ++n_loaded;
            if (!alive) break;
            if (a.use_logfmt) {
                // re-code the row in place: 10 bits per channel plus one range per 128 channels
                logfmt::encode_row_in_place(stage + st * row_bytes, hdr_scratch, H);
                ptx::fence_proxy_async_smem();
                __syncwarp();
            }
            if (lane == 0) {
                uint8_t* dst = s_peer[s] + a.off_slab[set] + (static_cast<int64_t>(t) * K + k) * row_bytes;
                ptx::bulk_store(dst, stage + st * row_bytes, wire_bytes);
            }
            ptx::bulk_commit();
            pos = next_pos;
        }
        ptx::bulk_commit();
        stamp(1);
        ptx::bulk_wait<0>();
        __threadfence_system();
        stamp(2);
        // the last CTA of this rank to finish its stores raises this rank's flag at every peer (no grid barrier)
        if (arrive_is_last(&ws->arrive[EP_CH_LL_COMBINE][0]) && !is_aborted(ws)) {
            if (tid < R && !rank_masked(a.mask, tid)) {
                Workspace* pws = reinterpret_cast<Workspace*>(s_peer[tid]);
                ptx::st_release_sys(&pws->ll_signal[1][me], tag_value(epoch, 1));
            }
            if (a.prof != nullptr && tid == 0) a.prof[3] = globaltimer_ns();
        }
    }

    if (a.phases & EP_LL_RECV) {
        int ok = alive ? 1 : 0;
        if (alive && tid < R && !rank_masked(a.mask, tid)) {
            const uint64_t* sig = &ws->ll_signal[1][tid];
            const uint64_t t0 = globaltimer_ns();
            if (a.shrink) {
                if (!shrink_wait(ctx, ws, sig, epoch, t0) && !is_aborted(ws)) atomicExch(a.mask + tid, 1);
            } else {
                ok = bounded_wait(
                    ctx, ws, EP_PH_LL_COMBINE_FLAG, tid, epoch, [&] { return tag_matches(ptx::ld_acquire_sys(sig), epoch); },
                    [&] { return ptx::ld_relaxed_sys(sig); });
            }
            if (a.wait_stats != nullptr && blockIdx.x == 0)
                atomicAdd(reinterpret_cast<unsigned long long*>(a.wait_stats + tid), globaltimer_ns() - t0);
        }
        alive = __syncthreads_and(ok) != 0;
        stamp(4);
        if (alive && a.use_logfmt) {
            // out[t] = sum_k w[t, k] * decode(slot[t, k]); work item = (token, 512 channels), one warp each; a lane decodes
            // 16 channels (five words of codes) of every source row, eight lanes share a range header
            const uint8_t* slab = s_peer[me] + a.off_slab[set];
            const int steps = (H + logfmt::kStepChannels - 1) / logfmt::kStepChannels;
            const int groups = H / logfmt::kGroup;
            const int64_t items = static_cast<int64_t>(a.num_tokens) * steps;
            for (int64_t it = static_cast<int64_t>(blockIdx.x) * kLLWarps + warp; it < items; it += static_cast<int64_t>(gridDim.x) * kLLWarps) {
                const int t = static_cast<int>(it / steps), c = static_cast<int>(it % steps);
                const int ch = c * logfmt::kStepChannels + lane * logfmt::kLaneChannels;
                const bool in_row = ch < H;
                int e_k = -1;
                float w_k = 0.f;
                if (lane < K) {
                    e_k = ll_load_idx(a.topk_idx, a.idx_is_64, static_cast<int64_t>(t) * K + lane);
                    w_k = __ldg(a.topk_weights + static_cast<int64_t>(t) * K + lane);
                    if (e_k >= 0 && rank_masked(a.mask, e_k / El)) e_k = -1;
                }
                const uint32_t srcs = __ballot_sync(0xffffffffu, e_k >= 0 && e_k < E);
                float acc[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[i] = 0.f;
                // the codes of up to eight source rows are requested together, so that an item costs one memory round
                // trip (as in the bf16 path), then decoded and accumulated in top-k lane order
                for (int k0 = 0; k0 < K; k0 += 8) {
                    uint32_t wds[8][5], hdr[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int k = k0 + j;
                        if (k < K && ((srcs >> k) & 1u) && in_row) {
                            const uint8_t* row = slab + (static_cast<int64_t>(t) * K + k) * row_bytes;
                            const uint32_t* codes = reinterpret_cast<const uint32_t*>(row + (ch / logfmt::kLaneChannels) * 20);
#pragma unroll
                            for (int q = 0; q < 5; ++q) wds[j][q] = __ldcg(codes + q);
                            hdr[j] = __ldcg(reinterpret_cast<const uint32_t*>(row + groups * logfmt::kCodeBytesPerGroup) + ch / logfmt::kGroup);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int k = k0 + j;
                        if (k < K && ((srcs >> k) & 1u)) {      // warp-uniform
                            const float w = __shfl_sync(0xffffffffu, w_k, k);
                            if (in_row) {
                                const float2 mm = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&hdr[j]));   // (amax, amin)
                                if (mm.x > 0.f) {
                                    uint32_t cds[16];
                                    logfmt::unpack16(wds[j], cds);
                                    const logfmt::Range r = logfmt::make_range(mm.x, mm.y);
#pragma unroll
                                    for (int i = 0; i < 16; ++i) acc[i] = fmaf(w, logfmt::decode_one(cds[i], r), acc[i]);
                                }
                            }
                        }
                    }
                }
                if (in_row) {
                    int4 o[2];
                    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(o);
#pragma unroll
                    for (int q = 0; q < 8; ++q) h[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
                    int4* dst = reinterpret_cast<int4*>(reinterpret_cast<uint8_t*>(a.out) + static_cast<int64_t>(t) * row_bytes + ch * 2);
                    dst[0] = o[0];
                    dst[1] = o[1];
                }
            }
        } else if (alive) {
            // out[t] = sum_k w[t, k] * slot[t, k]; work item = (token, 512-byte column chunk), one warp each: every lane
            // has the 16-byte loads of all top-k rows in flight at once, so an item costs one memory round trip
            const uint8_t* slab = s_peer[me] + a.off_slab[set];
            constexpr int kChunk = 32 * 16;
            const int num_chunks = (row_bytes + kChunk - 1) / kChunk;
            const int64_t items = static_cast<int64_t>(a.num_tokens) * num_chunks;
            for (int64_t it = static_cast<int64_t>(blockIdx.x) * kLLWarps + warp; it < items; it += static_cast<int64_t>(gridDim.x) * kLLWarps) {
                const int t = static_cast<int>(it / num_chunks), c = static_cast<int>(it % num_chunks);
                const int off = c * kChunk + lane * 16;
                const bool in_row = off < row_bytes;
                int e_k = -1;
                float w_k = 0.f;
                if (lane < K) {
                    e_k = ll_load_idx(a.topk_idx, a.idx_is_64, static_cast<int64_t>(t) * K + lane);
                    w_k = __ldg(a.topk_weights + static_cast<int64_t>(t) * K + lane);
                    if (e_k >= 0 && rank_masked(a.mask, e_k / El)) e_k = -1;
                }
                const uint32_t srcs = __ballot_sync(0xffffffffu, e_k >= 0 && e_k < E);
                const uint8_t* rows = slab + static_cast<int64_t>(t) * K * row_bytes + off;
                int4 raw[EP_MAX_TOPK];
#pragma unroll
                for (int k = 0; k < EP_MAX_TOPK; ++k)
                    if (k < K && ((srcs >> k) & 1u) && in_row) raw[k] = __ldcg(reinterpret_cast<const int4*>(rows + static_cast<int64_t>(k) * row_bytes));
                float acc[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
                for (int k = 0; k < EP_MAX_TOPK; ++k) {
                    if (k < K && ((srcs >> k) & 1u)) {
                        const float w = __shfl_sync(0xffffffffu, w_k, k);
                        if (in_row) {
                            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[k]);
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const float2 f = __bfloat1622float2(h[q]);
                                acc[2 * q] = fmaf(w, f.x, acc[2 * q]);
                                acc[2 * q + 1] = fmaf(w, f.y, acc[2 * q + 1]);
                            }
                        }
                    }
                }
                if (in_row) {
                    int4 outv;
                    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&outv);
#pragma unroll
                    for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
                    *reinterpret_cast<int4*>(reinterpret_cast<uint8_t*>(a.out) + static_cast<int64_t>(t) * row_bytes + off) = outv;
                }
            }
        }
        stamp(5);
        if (arrive_is_last(&ws->arrive[EP_CH_LL_COMBINE][1]) && tid == 0) {
            ws->epoch[EP_CH_LL_COMBINE] = epoch;
            if (a.prof != nullptr) a.prof[6] = globaltimer_ns();
        }
    }
}

__global__ void __launch_bounds__(kLLThreads, 1) ll_dispatch_kernel(const __grid_constant__ LLDispatchArgs a) { ll_dispatch_body(a); }
// n virtual ranks on one device: the argument structs travel as ONE kernel parameter (no allocation, no copy), which
// keeps the launch capturable in a CUDA graph
template <typename Args>
struct MultiArgs {
    Args a[EP_MAX_RANKS];
};
__global__ void __launch_bounds__(kLLThreads, 1) ll_dispatch_kernel_multi(const __grid_constant__ MultiArgs<LLDispatchArgs> m) { ll_dispatch_body(m.a[blockIdx.y]); }
__global__ void __launch_bounds__(kLLThreads, 1) ll_combine_kernel(const __grid_constant__ LLCombineArgs a) { ll_combine_body(a); }
__global__ void __launch_bounds__(kLLThreads, 1) ll_combine_kernel_multi(const __grid_constant__ MultiArgs<LLCombineArgs> m) { ll_combine_body(m.a[blockIdx.y]); }

template <typename Args>
cudaError_t launch_ll(const void* single, const void* multi, const Args* args, int n, int num_sms, int smem, cudaStream_t stream) {
    // A launch that both sends and receives must have all its CTAs resident: the counts a CTA waits for are published by
    // the LAST CTA of the peer to finish sending, which may be one that only starts when a waiting CTA leaves.  The
    // halves of the hook mode have no such dependency (the send half waits for nothing, the receive half only for peers'
    // send halves), so they are plain launches that can share the GPU with a compute kernel.
    const bool both_phases = (args[0].phases & (EP_LL_SEND | EP_LL_RECV)) == (EP_LL_SEND | EP_LL_RECV);
    const void* fn = n == 1 ? single : multi;
    cudaError_t err = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return err;
    const int ctas = num_sms < 1 ? 1 : (num_sms > EP_MAX_CTAS ? EP_MAX_CTAS : num_sms);
    dim3 grid(ctas, n, 1), block(kLLThreads, 1, 1);
    if (n == 1) {
        void* params[] = {const_cast<Args*>(args)};
        if (both_phases) return cudaLaunchCooperativeKernel(fn, grid, block, params, smem, stream);
        return cudaLaunchKernel(fn, grid, block, params, smem, stream);
    }
    if (n > EP_MAX_RANKS) return cudaErrorInvalidValue;
    MultiArgs<Args> multi_args;
    for (int i = 0; i < n; ++i) multi_args.a[i] = args[i];
    void* params[] = {&multi_args};
    // the virtual ranks wait on one another: all their CTAs must be resident
    return cudaLaunchCooperativeKernel(fn, grid, block, params, smem, stream);
}

}  // namespace

cudaError_t launch_ll_dispatch(const LLDispatchArgs* args, int n, int num_sms, cudaStream_t stream) {
    const int smem = 2 * args[0].msg_bytes;
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    return launch_ll<LLDispatchArgs>((const void*)ll_dispatch_kernel, (const void*)ll_dispatch_kernel_multi, args, n, num_sms, smem, stream);
}

cudaError_t launch_ll_combine(const LLCombineArgs* args, int n, int num_sms, cudaStream_t stream) {
    const int smem = 1024 + ll_combine_send_warps(args[0].hidden) * (2 * args[0].hidden * 2 + ll_combine_hdr_bytes(args[0].hidden));
    if (smem > 227 * 1024) return cudaErrorInvalidValue;
    if (args[0].use_logfmt && args[0].hidden % 128 != 0) return cudaErrorInvalidValue;
    return launch_ll<LLCombineArgs>((const void*)ll_combine_kernel, (const void*)ll_combine_kernel_multi, args, n, num_sms, smem, stream);
}

}  // namespace ep
