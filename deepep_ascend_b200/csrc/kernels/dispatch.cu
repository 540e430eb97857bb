// Expert-parallel dispatch for one NVLink domain, as ONE kernel per call with no grid-wide barrier inside:
//
//   1. count    - every CTA counts, for its slice of tokens, the rows it will send to each rank (a token counts once
//                 per rank) and the selections of each expert, publishes its own counts (for the CTAs above it) and
//                 adds them to this rank's totals with atomics;
//   2. exchange - the last CTA to add publishes the totals into every peer's workspace as epoch-tagged words; every
//                 CTA waits for all ranks' totals itself (this is also the entry barrier: a peer's totals arrive only
//                 once the peer has entered the same call);
//   3. assign   - prefix sums over (lower source ranks, lower CTAs, lower warps) turn the counts into FINAL row numbers in
//                 the receivers' output tensors, in (source rank, token) order, so the result is deterministic and needs
//                 no second pass; a CTA then flags its slice as assigned;
//   4. scatter  - tokens are claimed dynamically by the warps of all CTAs (a claimer waits for the flag of the CTA that
//                 owns the token); per token: optional fused bf16 -> e4m3 cast with 1x128 scales (register batches
//                 straight from global memory) or a TMA bulk load, then per destination rank one bulk store of the row
//                 straight into that rank's recv_x through its peer mapping, one of the scales and one of a tail record
//                 (expert ids already relative to the receiver, weights, source token and sending lane);
//   5. finish   - every CTA drains its bulk stores and arrives; the last one tells every peer "my rows have arrived",
//                 waits for the peers' words and closes the call.  All other CTAs leave as soon as they are drained.
//
// Parity: does the work of dispatch_impl + dispatch_copy_epilogue_impl
// (deep_ep/include/deep_ep/impls/dispatch.cuh:17-409, dispatch_copy_epilogue.cuh:11-323, zero padding :231-322) and of
// the fused FP8 cast of the legacy low-latency kernel (csrc/kernels/legacy/internode_ll.cu:212-250).
#include <cstdlib>

#include "common.cuh"

namespace ep {

namespace {

constexpr int kDispatchMaxWarps = 12;
constexpr int kDispatchMaxStages = 4;
constexpr int kDispatchSmemBudget = 222 * 1024;

struct DispatchSmemPlan {
    int off_peer;       // uint8_t* [EP_MAX_RANKS]
    int off_tot;        // uint32 [E]   expert totals over sources
    int off_before;     // uint32 [E]   selections from lower source ranks (and lower CTAs)
    int off_start;      // uint32 [E]   first row of each expert at its rank
    int off_prefix;     // uint32 [R]   rows of lower ranks / CTAs per destination
    int off_wc_rank;    // uint32 [W][R]
    int off_wc_expert;  // uint32 [W][E] (expand layout) or [E] shared by the CTA
    int off_bar;        // uint64 [W][3]
    int off_sf;         // float  [W][n_side][sf_floats]
    int off_tail;       // bytes  [W][n_side][max_dst][tail_bytes] tail records being sent
    int off_stage;      // per warp: stage buffers
    int sf_floats, max_dst, n_side;
    int in_bytes, out_bytes, n_in, n_out, warp_stage_bytes;
    int total;
};

__host__ __device__ inline int align_int(int x, int a) { return (x + a - 1) / a * a; }

__host__ __device__ inline DispatchSmemPlan make_smem_plan(const DispatchArgs& a, int num_warps, int num_stages) {
    DispatchSmemPlan p;
    const int E = a.num_experts, R = a.ctx.num_ranks;
    const int G = (a.hidden + 127) / 128;
    p.sf_floats = align_int(G, 4);
    p.max_dst = a.num_topk < R ? a.num_topk : R;
    // staging buffers of the small pieces follow the payload stages: a buffer is reused once the bulk stores of the
    // token that last used it have read their sources
    p.n_side = a.quantize ? num_stages : 2;
    int off = 0;
    p.off_peer = off;       off += EP_MAX_RANKS * 8;
    p.off_tot = off;        off += align_int(E * 4, 16);
    p.off_before = off;     off += align_int(E * 4, 16);
    p.off_start = off;      off += align_int(E * 4, 16);
    p.off_prefix = off;     off += EP_MAX_RANKS * 4;
    p.off_wc_rank = off;    off += align_int(num_warps * R * 4, 16);
    p.off_wc_expert = off;  off += align_int((a.do_expand ? num_warps : 1) * E * 4, 16);
    p.off_bar = off;        off += align_int(num_warps * 3 * 8, 16);   // keeps everything behind it 16-byte aligned (bulk copy sources)
    p.off_sf = off;         off += num_warps * p.n_side * p.sf_floats * 4;
    p.off_tail = off;       off += a.side_packed ? num_warps * p.n_side * p.max_dst * a.tail_bytes : 0;
    off = align_int(off, 128);
    p.off_stage = off;
    const int in_row = a.hidden * (a.x_is_fp8 ? 1 : 2);
    p.in_bytes = align_int(in_row, 128);
    if (a.quantize) {
        // the cast reads global memory directly; `num_stages` output stages (the stores of earlier tokens may still be
        // reading their stages while the next token is cast)
        p.out_bytes = align_int(a.hidden, 128);
        p.n_in = 0;
        p.n_out = num_stages;
    } else {
        // the input stage is also the store source: three stages keep one load and one store in flight
        p.out_bytes = 0;
        p.n_in = 3;
        p.n_out = 0;
    }
    p.warp_stage_bytes = p.n_in * p.in_bytes + p.n_out * p.out_bytes;
    p.total = off + num_warps * p.warp_stage_bytes;
    return p;
}

__device__ __forceinline__ int load_idx(const DispatchArgs& a, int t, int k) {
    const int64_t i = static_cast<int64_t>(t) * a.num_topk + k;
    return a.idx_is_64 ? static_cast<int>(__ldg(reinterpret_cast<const long long*>(a.topk_idx) + i))
                       : __ldg(reinterpret_cast<const int*>(a.topk_idx) + i);
}

struct Slice {
    int begin, end;
};

// Contiguous token slice of (cta, warp); warp slices are multiples of the tokens handled per layout step.
__device__ __forceinline__ Slice warp_slice(int T, int K, int num_warps, int warp) {
    const int chunk = (T + gridDim.x - 1) / gridDim.x;
    const int cta_begin = min(T, static_cast<int>(blockIdx.x) * chunk);
    const int cta_end = min(T, cta_begin + chunk);
    const int tps = 32 / K;
    int sub = (chunk + num_warps - 1) / num_warps;
    sub = (sub + tps - 1) / tps * tps;
    Slice s;
    s.begin = min(cta_end, cta_begin + warp * sub);
    s.end = min(cta_end, s.begin + sub);
    return s;
}

// One pass over the warp's tokens, `32 / K` tokens per step with lane = (token_in_step, top-k lane).
// kAssign == false: count into the warp's private counters.
// kAssign == true : the counters hold the first row for this warp; hand out rows in (token, lane) order.
template <bool kAssign>
__device__ __forceinline__ void layout_pass(const DispatchArgs& a, Slice sl, uint32_t* wc_rank, uint32_t* wc_expert) {
    const int K = a.num_topk, R = a.ctx.num_ranks, E = a.num_experts, El = E / R;
    const int lane = ptx::lane_id();
    const int tps = 32 / K;
    const int ts = lane / K, k = lane - ts * K;
    const uint32_t lt = ptx::lanemask_lt();
    for (int t0 = sl.begin; t0 < sl.end; t0 += tps) {
        const int t = t0 + ts;
        const bool active = ts < tps && t < sl.end;
        const int e = active ? load_idx(a, t, k) : -1;
        const bool valid = e >= 0 && e < E;
        const int r = valid ? e / El : -1;
        const uint32_t peers_tr = __match_any_sync(0xffffffffu, valid ? (ts * EP_MAX_RANKS + r) : (1024 + lane));
        const int master = 31 - __clz(peers_tr);
        const bool is_last = valid && lane == master;
        if (!kAssign) {
            if (valid) atomicAdd(&wc_expert[e], 1u);
            if (is_last) atomicAdd(&wc_rank[r], 1u);
        } else {
            int packed;
            if (a.do_expand) {
                const uint32_t peers = __match_any_sync(0xffffffffu, valid ? e : (0x10000 + lane));
                const int leader = __ffs(peers) - 1;
                uint32_t old = 0;
                if (valid && lane == leader) {
                    old = wc_expert[e];
                    wc_expert[e] = old + __popc(peers);
                }
                old = __shfl_sync(0xffffffffu, old, leader);
                const uint32_t row = old + __popc(peers & lt);
                packed = valid ? static_cast<int>((static_cast<uint32_t>(r) << 24) | row) : -1;
                if (active) {
                    a.lane_src[static_cast<int64_t>(t) * K + k] = packed;
                    a.plan[static_cast<int64_t>(t) * K + k] = packed;
                }
            } else {
                const uint32_t peers = __match_any_sync(0xffffffffu, is_last ? r : (1024 + lane));
                const int leader = __ffs(peers) - 1;
                uint32_t old = 0;
                if (is_last && lane == leader) {
                    old = wc_rank[r];
                    wc_rank[r] = old + __popc(peers);
                }
                old = __shfl_sync(0xffffffffu, old, leader);
                uint32_t row = old + __popc(peers & lt);
                row = __shfl_sync(0xffffffffu, row, master);
                packed = valid ? static_cast<int>((static_cast<uint32_t>(r) << 24) | row) : -1;
                if (active) {
                    a.lane_src[static_cast<int64_t>(t) * K + k] = packed;
                    a.plan[static_cast<int64_t>(t) * K + k] = is_last ? packed : -1;
                }
            }
            __syncwarp();
        }
    }
    __syncwarp();
}

__device__ __forceinline__ uint32_t count_of(uint64_t word) { return static_cast<uint32_t>(word & 0xffffffffull); }

// Fused cast: a row is processed in register batches of kCastSteps x 256 channels.  All 16-byte loads of a batch
// are issued back to back straight from global memory, the next batch is requested before the current one is
// converted, and the unrolled conversions of a batch are independent of one another, so neither the memory
// latency nor the shuffle / reciprocal latency chains of one 128-channel group are exposed.
// q = x * (448 / max(amax, 1e-4)) rounded to nearest even, scale = max(amax, 1e-4) / 448.
// The correctly rounded division amax / 448 costs ~20 instructions that only two lanes of a step would use, so the steps
// leave the clamped amax in the staging row and scales_from_amax divides all groups of the row at once, one group per lane.
constexpr int kCastSteps = 7;

struct RowBatch {
    int4 v[kCastSteps];
};

__device__ __forceinline__ void load_batch(RowBatch& b, const uint8_t* row, int H, int batch) {
    const int lane = ptx::lane_id();
#pragma unroll
    for (int i = 0; i < kCastSteps; ++i) {
        const int elem = ((batch * kCastSteps + i) * 32 + lane) * 8;
        b.v[i] = elem < H ? ptx::ld_nc_v4(row + elem * 2) : make_int4(0, 0, 0, 0);
    }
}

__device__ __forceinline__ void scales_from_amax(float* sf, int num_groups) {
    __syncwarp();
    for (int g = ptx::lane_id(); g < num_groups; g += 32) sf[g] = __fdiv_rn(sf[g], 448.f);
}

__device__ __forceinline__ void cast_batch(const RowBatch& b, uint8_t* out, float* sf, int H, int batch) {
    const int lane = ptx::lane_id();
#pragma unroll
    for (int i = 0; i < kCastSteps; ++i) {
        const int elem = ((batch * kCastSteps + i) * 32 + lane) * 8;
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&b.v[i]);
        float v[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            v[2 * j] = f.x;
            v[2 * j + 1] = f.y;
        }
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
        amax = fmaxf(ptx::warp_max_16(amax), 1e-4f);
        // 448 * (1 / amax), each step correctly rounded: bit-identical to the PyTorch expression `448.0 / amax`
        const float scale = __fmul_rn(448.f, __frcp_rn(amax));
        if (elem < H) {
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
            if ((lane & 15) == 0) sf[elem / 128] = amax;      // divided by 448 once per row, see scales_from_amax
        }
    }
}

// sources of all but the `pending` most recent bulk groups of this thread have been read
__device__ __forceinline__ void bulk_wait_read_n(int pending) {
    switch (pending) {
        case 1: ptx::bulk_wait_read<1>(); break;
        case 2: ptx::bulk_wait_read<2>(); break;
        case 3: ptx::bulk_wait_read<3>(); break;
        default: ptx::bulk_wait_read<0>(); break;
    }
}

template <bool kQuant>
__device__ __forceinline__ void dispatch_body(const DispatchArgs& a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const RankCtx& ctx = a.ctx;
    Workspace* ws = local_ws(ctx);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int num_warps = blockDim.x >> 5, nthreads = blockDim.x;
    const int cta = blockIdx.x, num_ctas = gridDim.x;
    const int R = ctx.num_ranks, me = ctx.rank, E = a.num_experts, El = E / R, K = a.num_topk, T = a.num_tokens;
    const int G = (a.hidden + 127) / 128;
    const DispatchSmemPlan sp = make_smem_plan(a, num_warps, a.tune_stages);

    uint8_t** s_peer = reinterpret_cast<uint8_t**>(smem + sp.off_peer);
    uint32_t* s_tot = reinterpret_cast<uint32_t*>(smem + sp.off_tot);
    uint32_t* s_before = reinterpret_cast<uint32_t*>(smem + sp.off_before);
    uint32_t* s_start = reinterpret_cast<uint32_t*>(smem + sp.off_start);
    uint32_t* s_prefix = reinterpret_cast<uint32_t*>(smem + sp.off_prefix);
    uint32_t* s_wc_rank = reinterpret_cast<uint32_t*>(smem + sp.off_wc_rank);
    uint32_t* s_wc_expert = reinterpret_cast<uint32_t*>(smem + sp.off_wc_expert);
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + sp.off_bar) + warp * 3;
    float* s_sf = reinterpret_cast<float*>(smem + sp.off_sf) + warp * sp.n_side * sp.sf_floats;
    uint8_t* s_tail = smem + sp.off_tail + warp * sp.n_side * sp.max_dst * a.tail_bytes;
    uint8_t* s_stage = smem + sp.off_stage + warp * sp.warp_stage_bytes;
    const int expert_sets = a.do_expand ? num_warps : 1;   // private expert counters per warp only where row order needs them

    // every CTA reads the call number before it arrives anywhere; the last CTA to finish writes the new one
    const uint64_t epoch = *reinterpret_cast<volatile uint64_t*>(&ws->epoch[EP_CH_DISPATCH]) + 1;
    const uint32_t epoch32 = static_cast<uint32_t>(epoch);
    const uint64_t entry_seq = *reinterpret_cast<volatile uint64_t*>(&ws->bar_seq[EP_CH_DISPATCH]) + 1;
    if (tid < EP_MAX_RANKS) s_peer[tid] = tid < R ? ctx.peer_base[tid] : nullptr;
    if (lane == 0) {
        ptx::mbar_init(&s_bar[0], 1);
        ptx::mbar_init(&s_bar[1], 1);
        ptx::mbar_init(&s_bar[2], 1);
    }
    ptx::mbar_fence_init();
    for (int i = tid; i < num_warps * R; i += nthreads) s_wc_rank[i] = 0;
    for (int i = tid; i < expert_sets * E; i += nthreads) s_wc_expert[i] = 0;
    __syncthreads();
    ptx::fence_proxy_async_smem();

    const Slice sl = warp_slice(T, K, num_warps, warp);
    const int own_chunk = max(1, (T + num_ctas - 1) / num_ctas);
    bool alive = !is_aborted(ws);
    auto stamp = [&](int i) {
        if (a.prof != nullptr && cta == 0 && tid == 0) a.prof[i] = globaltimer_ns();
    };
    stamp(0);
    const bool bookkeeper = cta == num_ctas - 1;   // writes what this rank receives (handle tensors, host counters); its tokens are claimed last
    const bool need_experts = a.do_expand || bookkeeper;

    if (!a.cached) {
        // ---------------------------------------------------------------- 1. count
        layout_pass<false>(a, sl, s_wc_rank + warp * R, s_wc_expert + (a.do_expand ? warp * E : 0));
        __syncthreads();
        for (int i = tid; i < E + R; i += nthreads) {
            uint32_t tot = 0;
            if (i < E) {
                for (int w = 0; w < expert_sets; ++w) tot += s_wc_expert[w * E + i];
                if (a.do_expand) __stcg(&ws->cta_expert_count[cta][i], tot);
                if (tot) atomicAdd(&ws->tot_expert[i], tot);
            } else {
                for (int w = 0; w < num_warps; ++w) tot += s_wc_rank[w * R + (i - E)];
                __stcg(&ws->cta_rank_count[cta][i - E], tot);
                if (tot) atomicAdd(&ws->tot_rank[i - E], tot);
            }
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) ptx::st_release_gpu_u32(&ws->cta_counted[cta], epoch32);
        const bool last_to_count = arrive_is_last(&ws->arrive[EP_CH_DISPATCH][0]);
        stamp(1);

        // ---------------------------------------------------------------- 2. exchange
        if (last_to_count && alive) {
            // every CTA of this rank has added its counts: publish the totals to all ranks (this rank included) and
            // clear the accumulators for the next call
            for (int i = tid; i < E + R; i += nthreads) {
                uint32_t* acc = i < E ? &ws->tot_expert[i] : &ws->tot_rank[i - E];
                const uint32_t tot = __ldcg(acc);
                __stcg(acc, 0u);
                const uint64_t word = tag_value(epoch, tot);
                for (int p = 0; p < R; ++p) {
                    Workspace* pws = reinterpret_cast<Workspace*>(s_peer[p]);
                    ptx::st_relaxed_sys(i < E ? &pws->disp_expert_count[me][i] : &pws->disp_rank_count[me][i - E], word);
                }
            }
        }
        int ok = alive ? 1 : 0;
        if (alive) {
            for (int i = tid; i < R * R && ok; i += nthreads) {
                const uint64_t* slot = &ws->disp_rank_count[i / R][i % R];
                ok = bounded_wait(
                    ctx, ws, EP_PH_COUNT_EXCHANGE, i / R, epoch,
                    [&] { return tag_matches(ptx::ld_relaxed_sys(slot), epoch); },
                    [&] { return ptx::ld_relaxed_sys(slot); });
            }
            // counts of the CTAs below this one
            for (int c = tid; c < cta && ok; c += nthreads) {
                const uint32_t* flag = &ws->cta_counted[c];
                ok = bounded_wait(
                    ctx, ws, EP_PH_CTA_COUNTS, c, epoch32, [&] { return ptx::ld_acquire_gpu_u32(flag) == epoch32; },
                    [&] { return static_cast<uint64_t>(ptx::ld_relaxed_gpu_u32(flag)); });
            }
            if (need_experts) {
                for (int i = tid; i < R * E && ok; i += nthreads) {
                    const uint64_t* slot = &ws->disp_expert_count[i / E][i % E];
                    ok = bounded_wait(
                        ctx, ws, EP_PH_COUNT_EXCHANGE, i / E, epoch,
                        [&] { return tag_matches(ptx::ld_relaxed_sys(slot), epoch); },
                        [&] { return ptx::ld_relaxed_sys(slot); });
                }
            }
        }
        alive = __syncthreads_and(ok) != 0;
        stamp(2);

        // ---------------------------------------------------------------- 3. assign: counts -> first rows
        if (alive) {
            const uint32_t A = max(1, a.expert_alignment);
            if (tid < R) s_prefix[tid] = 0;
            __syncthreads();
            if (!a.do_expand) {
                // rows of lower source ranks and of lower CTAs of this rank, summed by all threads in parallel
                for (int p = tid; p < (me + cta) * R; p += nthreads) {
                    const int d = p % R, i = p / R;
                    const uint32_t n = i < me ? count_of(ptx::ld_relaxed_sys(&ws->disp_rank_count[i][d])) : __ldcg(&ws->cta_rank_count[i - me][d]);
                    if (n) atomicAdd(&s_prefix[d], n);
                }
                __syncthreads();
                if (tid < R) {
                    uint32_t running = s_prefix[tid];
                    for (int w = 0; w < num_warps; ++w) {
                        const uint32_t n = s_wc_rank[w * R + tid];
                        s_wc_rank[w * R + tid] = running;
                        running += n;
                    }
                }
            }
            if (need_experts) {
                for (int e = tid; e < E; e += nthreads) {
                    uint32_t tot = 0, before = 0;
                    for (int s = 0; s < R; ++s) {
                        const uint32_t n = count_of(ptx::ld_relaxed_sys(&ws->disp_expert_count[s][e]));
                        tot += n;
                        if (s < me) before += n;
                    }
                    s_tot[e] = tot;
                    s_before[e] = before;
                }
                __syncthreads();
                // first row of every expert at its rank = exclusive prefix sum of the aligned totals of that rank
                // (every segment start is a multiple of the alignment); one warp scans one rank
                for (int d = warp; d < R; d += num_warps) {
                    uint32_t carry = 0;
                    for (int base = 0; base < El; base += 32) {
                        const int j = base + lane;
                        const uint32_t al = j < El ? (s_tot[d * El + j] + A - 1) / A * A : 0;
                        uint32_t incl = al;
#pragma unroll
                        for (int o = 1; o < 32; o <<= 1) {
                            const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
                            if (lane >= o) incl += up;
                        }
                        if (j < El) s_start[d * El + j] = carry + incl - al;
                        carry += __shfl_sync(0xffffffffu, incl, 31);
                    }
                }
                if (a.do_expand) {
                    // selections of lower CTAs of this rank
                    for (int p = tid; p < cta * E; p += nthreads) {
                        const uint32_t n = __ldcg(&ws->cta_expert_count[p / E][p % E]);
                        if (n) atomicAdd(&s_before[p % E], n);
                    }
                }
                __syncthreads();
                if (a.do_expand) {
                    for (int e = tid; e < E; e += nthreads) {
                        uint32_t running = s_start[e] + s_before[e];
                        for (int w = 0; w < num_warps; ++w) {
                            const uint32_t n = s_wc_expert[w * E + e];
                            s_wc_expert[w * E + e] = running;
                            running += n;
                        }
                    }
                }
                if (bookkeeper) {
                    // what this rank receives: handle tensors + host-visible counters (each word carries its own
                    // epoch tag, so the host needs no ordering between them)
                    volatile uint64_t* st = ctx.status;
                    for (int j = tid; j < El; j += nthreads) {
                        const uint32_t n = s_tot[me * El + j], start = s_start[me * El + j];
                        a.recv_per_expert[j] = n;
                        a.psum_expert[j] = a.do_expand ? start + n : start + (n + A - 1) / A * A;
                        if (a.stats != nullptr) a.stats[j] += n;
                        st[EP_STATUS_EXPERT_BASE + j] = tag_value(epoch, n);
                    }
                    if (tid == 0) {
                        uint32_t psum = 0;
                        for (int s = 0; s < R; ++s) {
                            psum += count_of(ptx::ld_relaxed_sys(&ws->disp_rank_count[s][me]));
                            a.psum_rank[s] = psum;
                        }
                        const uint32_t last = me * El + El - 1;
                        const uint32_t expanded = s_start[last] + (s_tot[last] + A - 1) / A * A;
                        st[EP_STATUS_NUM_EXPANDED] = tag_value(epoch, a.do_expand ? expanded : 0);
                        st[EP_STATUS_NUM_RECV] = tag_value(epoch, psum);
                    }
                }
            }
            __syncthreads();
            layout_pass<true>(a, sl, s_wc_rank + warp * R, s_wc_expert + (a.do_expand ? warp * E : 0));
        }
        // the row numbers of this CTA's slice are in global memory: any warp of the rank may now send those tokens
        __threadfence();
        __syncthreads();
        if (tid == 0 && alive) ptx::st_release_gpu_u32(&ws->cta_assigned[cta], epoch32);
    } else {
        // cached layout: only the entry barrier (receivers must be done with the previous contents); CTA 0 signals the
        // peers, every CTA watches the peers' arrivals itself
        int ok = alive ? 1 : 0;
        if (alive && tid < R) {
            if (cta == 0) ptx::red_add_release_sys(&reinterpret_cast<Workspace*>(s_peer[tid])->xbar[EP_CH_DISPATCH][me], 1ull);
            const uint64_t* mine = &ws->xbar[EP_CH_DISPATCH][tid];
            ok = bounded_wait(
                ctx, ws, EP_PH_XGPU_BARRIER, tid, entry_seq, [&] { return ptx::ld_acquire_sys(mine) >= entry_seq; },
                [&] { return ptx::ld_relaxed_sys(mine); });
        }
        alive = __syncthreads_and(ok) != 0;
    }
    stamp(3);

    // -------------------------------------------------------------------- 3b. zero padding of the expand layout
    if (alive && a.do_expand && a.do_zero_padding && a.expert_alignment > 1) {
        // rows between the end of a local expert's segment and its aligned end are written by nobody: zero them here
        // (payload and scales), one expert per warp
        const uint32_t A = a.expert_alignment;
        const int out_row = (kQuant || a.x_is_fp8) ? a.hidden : a.hidden * 2;
        const bool has_sf = kQuant || a.sf != nullptr;
        uint8_t* base = s_peer[me];
        for (int j = cta * num_warps + warp; j < El; j += num_ctas * num_warps) {
            uint32_t end;
            if (a.cached) end = static_cast<uint32_t>(__ldcg(a.psum_expert + j));
            else end = s_start[me * El + j] + s_tot[me * El + j];
            uint32_t aligned_end = (end + A - 1) / A * A;
            if (aligned_end > static_cast<uint32_t>(a.recv_capacity_rows)) aligned_end = a.recv_capacity_rows;
            for (uint32_t row = end; row < aligned_end; ++row) {
                uint8_t* dst = base + a.off_recv_x + static_cast<int64_t>(row) * out_row;
                for (int off = lane * 16; off < out_row; off += 32 * 16) ptx::st_na_v4(dst + off, make_int4(0, 0, 0, 0));
                if (has_sf) {
                    float* sfp = reinterpret_cast<float*>(base + a.off_recv_sf);
                    for (int g = lane; g < G; g += 32) sfp[static_cast<int64_t>(row) * a.sf_stride_row + g * a.sf_stride_col] = 0.f;
                }
            }
        }
    }

    // -------------------------------------------------------------------- 4. scatter
    if (alive) {
        const int in_row = a.hidden * (a.x_is_fp8 ? 1 : 2);
        const int out_row = kQuant ? a.hidden : in_row;
        const int idx_bytes = a.idx_is_64 ? 8 : 4;
        const bool has_sf = kQuant || a.sf != nullptr;
        uint8_t* in_stage = s_stage;
        uint8_t* out_stage = s_stage + sp.n_in * sp.in_bytes;
        const uint8_t* xb = reinterpret_cast<const uint8_t*>(a.x);
        const int S_in = kQuant ? 1 : sp.n_in;
        const int S_side = sp.n_side;
        const int num_batches = ((a.hidden + 255) / 256 + kCastSteps - 1) / kCastSteps;
        const uint32_t lt = ptx::lanemask_lt();
        // Tokens are claimed dynamically from a counter shared by all CTAs of this rank: SMs that get a smaller share of
        // the NVLink bandwidth simply claim fewer tokens.  Two tokens per claim, one near the end so that no warp is
        // left with a long tail.  The counter is zero at entry: the last CTA of every call clears it.
        const int tail_zone = 4 * num_ctas * num_warps;
        int last_base = 0;
        auto claim = [&](int& amount) -> int {
            amount = last_base + tail_zone < T ? 2 : 1;
            int b = 0;
            if (lane == 0) b = static_cast<int>(atomicAdd(&ws->dyn_counter[EP_CH_DISPATCH], static_cast<uint32_t>(amount)));
            b = __shfl_sync(0xffffffffu, b, 0);
            last_base = b;
            return b;
        };
        int chunk_n = 0, next_n = 0;
        int chunk_base = claim(chunk_n), next_base = claim(next_n), in_chunk = 0;
        auto next_token = [&]() -> int {
            if (in_chunk == chunk_n) {
                chunk_base = next_base;
                chunk_n = next_n;
                if (chunk_base < T) next_base = claim(next_n);
                else next_base = T, next_n = 1;
                in_chunk = 0;
            }
            const int t = chunk_base + in_chunk++;
            return t < T ? t : -1;
        };
        // row numbers of tokens outside this CTA's own slice were written by another CTA: wait for its flag once
        int known_lo = a.cached ? 0 : cta * own_chunk, known_hi = a.cached ? T : min(T, known_lo + own_chunk);
        auto rows_assigned = [&](int t) -> bool {
            if (t >= known_lo && t < known_hi) return true;
            const int owner = t / own_chunk;
            int ok = 1;
            if (lane == 0) {
                const uint32_t* flag = &ws->cta_assigned[owner];
                ok = bounded_wait(
                    ctx, ws, EP_PH_DISPATCH_ASSIGN, owner, epoch32, [&] { return ptx::ld_acquire_gpu_u32(flag) == epoch32; },
                    [&] { return static_cast<uint64_t>(ptx::ld_relaxed_gpu_u32(flag)); });
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            __syncwarp();
            known_lo = owner * own_chunk;
            known_hi = min(T, known_lo + own_chunk);
            return ok != 0;
        };
        int t = next_token(), t_next = next_token();
        int loads_issued = 0, loads_waited = 0;   // bulk loads of the pass-through path (token i uses stage i % S_in)
        RowBatch cur;
        if (kQuant) {
            if (t >= 0) load_batch(cur, xb + static_cast<int64_t>(t) * in_row, a.hidden, 0);
        } else if (t >= 0) {
            if (lane == 0) {
                ptx::mbar_arrive_expect_tx(&s_bar[0], in_row);
                ptx::bulk_load(in_stage, xb + static_cast<int64_t>(t) * in_row, in_row, &s_bar[0]);
            }
            loads_issued = 1;
        }
        for (int n = 0; t >= 0 && alive; ++n, t = t_next, t_next = next_token()) {
            const int st = n % S_in;
            const uint32_t parity = (n / S_in) & 1;
            // the staging buffers about to be overwritten were last read by the stores of token n - S_side
            bulk_wait_read_n(S_side - 1);
            __syncwarp();
            if (!kQuant) {
                // prefetch the next token; its stage was the source of the bulk stores of token n-2
                if (t_next >= 0) {
                    if (lane == 0) {
                        const int ns = (n + 1) % S_in;
                        ptx::mbar_arrive_expect_tx(&s_bar[ns], in_row);
                        ptx::bulk_load(in_stage + ns * sp.in_bytes, xb + static_cast<int64_t>(t_next) * in_row, in_row, &s_bar[ns]);
                    }
                    ++loads_issued;
                }
            }
            if (!rows_assigned(t)) {
                alive = false;
                break;
            }
            int e_k = -1, plan_k = -1;
            float w_k = 0.f;
            if (lane < K) {
                e_k = load_idx(a, t, lane);
                plan_k = __ldcg(a.plan + static_cast<int64_t>(t) * K + lane);
                if (a.topk_weights != nullptr) w_k = __ldg(a.topk_weights + static_cast<int64_t>(t) * K + lane);
            }
            const int side_slot = n % S_side;
            float* sf_cur = s_sf + side_slot * sp.sf_floats;
            uint8_t* tail_cur = s_tail + side_slot * sp.max_dst * a.tail_bytes;
            if (!kQuant && has_sf)
                for (int j = lane; j < G; j += 32) sf_cur[j] = __ldg(a.sf + static_cast<int64_t>(t) * G + j);
            const uint8_t* src_smem;
            if (kQuant) {
                uint8_t* o = out_stage + side_slot * sp.out_bytes;
                const uint8_t* row = xb + static_cast<int64_t>(t) * in_row;
                for (int b = 0; b < num_batches; ++b) {
                    RowBatch nxt;
                    if (b + 1 < num_batches) load_batch(nxt, row, a.hidden, b + 1);
                    else if (t_next >= 0) load_batch(nxt, xb + static_cast<int64_t>(t_next) * in_row, a.hidden, 0);   // first batch of the next token
                    cast_batch(cur, o, sf_cur, a.hidden, b);
                    cur = nxt;
                }
                scales_from_amax(sf_cur, G);
                src_smem = o;
            } else {
                alive = mbar_wait_bounded(ctx, ws, &s_bar[st], parity, EP_PH_DISPATCH_LOAD);
                if (!alive) break;
                ++loads_waited;
                src_smem = in_stage + st * sp.in_bytes;
            }
            const uint32_t sends = __ballot_sync(0xffffffffu, plan_k >= 0);   // lanes that own a destination row
            if (a.side_packed) {
                // one tail record per destination: expert ids relative to THAT rank's first expert (-1 for experts of
                // other ranks), the weights, the source token and the lane that sends the row
                int j = 0;
                for (uint32_t m = sends; m != 0; m &= m - 1, ++j) {
                    const int k = __ffs(m) - 1;
                    const int d = __shfl_sync(0xffffffffu, plan_k, k) >> 24;
                    uint8_t* rec = tail_cur + j * a.tail_bytes;
                    if (lane < K) {
                        const int lo = d * El;
                        const int local = (e_k >= lo && e_k < lo + El) ? e_k - lo : -1;
                        if (a.idx_is_64) reinterpret_cast<long long*>(rec)[lane] = local;
                        else reinterpret_cast<int*>(rec)[lane] = local;
                        reinterpret_cast<float*>(rec + a.tail_off_w)[lane] = w_k;
                    }
                    if (lane == 0) *reinterpret_cast<int2*>(rec + a.tail_off_meta) = make_int2(me * a.num_max_tokens + t, me * K + k);
                }
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            // bulk stores of a destination row are issued by the lane that owns the plan entry
            if (plan_k >= 0) {
                const int d = plan_k >> 24, row = plan_k & 0xffffff;
                if (row < a.recv_capacity_rows) {
                    uint8_t* base = s_peer[d];
                    ptx::bulk_store(base + a.off_recv_x + static_cast<int64_t>(row) * out_row, src_smem, out_row);
                    if (a.side_packed) {
                        if (has_sf) ptx::bulk_store(base + a.off_recv_sf + static_cast<int64_t>(row) * a.sf_stride_row * 4, sf_cur, G * 4);
                        const int j = __popc(sends & lt);
                        ptx::bulk_store(base + a.off_recv_tail + static_cast<int64_t>(row) * a.tail_pitch, tail_cur + j * a.tail_bytes, a.tail_bytes);
                    }
                } else {
                    report_failure(ctx, ws, EP_ERR_BOUNDS, EP_PH_DISPATCH_LOAD, d, a.recv_capacity_rows, row);
                    plan_k = -1;
                }
            }
            ptx::bulk_commit();
            if (!a.side_packed) {
                // small per-row pieces go out as plain peer stores
                uint32_t m = __ballot_sync(0xffffffffu, plan_k >= 0);
                while (m) {
                    const int k = __ffs(m) - 1;
                    m &= m - 1;
                    const int p = __shfl_sync(0xffffffffu, plan_k, k);
                    const int d = p >> 24;
                    const int64_t row = p & 0xffffff;
                    uint8_t* base = s_peer[d];
                    if (has_sf) {
                        float* dst = reinterpret_cast<float*>(base + a.off_recv_sf);
                        for (int j = lane; j < G; j += 32) dst[row * a.sf_stride_row + j * a.sf_stride_col] = sf_cur[j];
                    }
                    if (a.do_expand) {
                        const float w = __shfl_sync(0xffffffffu, w_k, k);
                        if (lane == 0) {
                            if (a.topk_weights != nullptr) reinterpret_cast<float*>(base + a.off_recv_w)[row] = w;
                            reinterpret_cast<int2*>(base + a.off_recv_meta)[row] = make_int2(me * a.num_max_tokens + t, me * K + k);
                        }
                    } else {
                        if (lane < K) {
                            const int lo = d * El;
                            const int local = (e_k >= lo && e_k < lo + El) ? e_k - lo : -1;
                            uint8_t* ip = base + a.off_recv_idx + (row * K + lane) * idx_bytes;
                            if (a.idx_is_64) *reinterpret_cast<long long*>(ip) = local;
                            else *reinterpret_cast<int*>(ip) = local;
                            if (a.topk_weights != nullptr) reinterpret_cast<float*>(base + a.off_recv_w)[row * K + lane] = w_k;
                        }
                        if (lane == 0)
                            reinterpret_cast<int2*>(base + a.off_recv_meta)[row] = make_int2(me * a.num_max_tokens + t, me * K + k);
                    }
                }
            }
        }
        // left early after a failure: loads still in flight must land before this CTA gives up its shared memory
        for (; loads_waited < loads_issued; ++loads_waited)
            mbar_drain(&s_bar[loads_waited % S_in], (loads_waited / S_in) & 1, 1000ull * 1000 * 1000);
    }

    // ------------------------------------------------------------------------ 5. finish
    ptx::bulk_commit();
    ptx::bulk_wait<0>();
    __threadfence_system();
    stamp(4);
    // Every CTA arrives once its own stores are complete; only the last one stays: it tells every peer "all rows of my
    // dispatch number `epoch` have arrived", waits for the same word from every peer (the kernel must not end before
    // this rank's received rows are in place) and closes the call.
    if (!arrive_is_last(&ws->arrive[EP_CH_DISPATCH][1])) return;
    auto stamp_last = [&](int i) {
        if (a.prof != nullptr && tid == 0) a.prof[i] = globaltimer_ns();
    };
    stamp_last(5);
    alive = !is_aborted(ws);
    {
        int ok = alive ? 1 : 0;
        if (alive && tid < R) {
            ptx::st_release_sys(&reinterpret_cast<Workspace*>(s_peer[tid])->disp_done[me], epoch);
            const uint64_t* word = &ws->disp_done[tid];
            ok = bounded_wait(
                ctx, ws, EP_PH_DISPATCH_DONE, tid, epoch, [&] { return ptx::ld_acquire_sys(word) >= epoch; },
                [&] { return ptx::ld_relaxed_sys(word); });
        }
        alive = __syncthreads_and(ok) != 0;
    }
    stamp_last(6);
    if (tid == 0) {
        atomicExch(&ws->dyn_counter[EP_CH_DISPATCH], 0u);
        if (a.cached) ws->bar_seq[EP_CH_DISPATCH] = entry_seq;
        ws->epoch[EP_CH_DISPATCH] = epoch;
    }
    stamp_last(7);
}

template <bool kQuant>
__global__ void __launch_bounds__(kDispatchMaxWarps * 32, 1) dispatch_kernel(const __grid_constant__ DispatchArgs args) {
    dispatch_body<kQuant>(args);
}

// n virtual ranks on one device: blockIdx.y selects the rank
template <bool kQuant>
__global__ void __launch_bounds__(kDispatchMaxWarps * 32, 1) dispatch_kernel_multi(const DispatchArgs* args) {
    dispatch_body<kQuant>(args[blockIdx.y]);
}

}  // namespace

LaunchShape dispatch_launch_shape(const DispatchArgs& a, int num_sms) {
    LaunchShape s;
    s.num_ctas = num_sms < 1 ? 1 : (num_sms > EP_MAX_CTAS ? EP_MAX_CTAS : num_sms);
    // staging buffers per warp of the fused-cast path (two unless the caller asks for more), then as many warps (each
    // with its own staging ring) as fit in shared memory; the token-per-step layout needs at least one warp
    s.num_stages = a.tune_stages >= 2 && a.tune_stages <= kDispatchMaxStages ? a.tune_stages : 2;
    s.num_warps = a.tune_warps >= 1 && a.tune_warps <= kDispatchMaxWarps ? a.tune_warps : kDispatchMaxWarps;
    while (s.num_warps > 1 && make_smem_plan(a, s.num_warps, s.num_stages).total > kDispatchSmemBudget) --s.num_warps;
    s.smem_bytes = make_smem_plan(a, s.num_warps, s.num_stages).total;
    return s;
}

cudaError_t launch_dispatch(const DispatchArgs* args_in, int n, int num_sms, cudaStream_t stream) {
    const LaunchShape shape = dispatch_launch_shape(args_in[0], num_sms);
    if (shape.smem_bytes > 227 * 1024 || n < 1 || n > EP_MAX_RANKS) return cudaErrorInvalidValue;
    // the kernel derives its shared-memory plan from the resolved shape
    DispatchArgs args[EP_MAX_RANKS];
    for (int i = 0; i < n; ++i) {
        args[i] = args_in[i];
        args[i].tune_warps = shape.num_warps;
        args[i].tune_stages = shape.num_stages;
    }
    const DispatchArgs& a0 = args[0];
    const void* fn;
    if (n == 1) fn = a0.quantize ? (const void*)dispatch_kernel<true> : (const void*)dispatch_kernel<false>;
    else fn = a0.quantize ? (const void*)dispatch_kernel_multi<true> : (const void*)dispatch_kernel_multi<false>;
    cudaError_t err = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, shape.smem_bytes);
    if (err != cudaSuccess) return err;
    dim3 grid(shape.num_ctas, n, 1), block(shape.num_warps * 32, 1, 1);
    // cooperative: the CTAs of a rank (and of all virtual ranks) wait on one another, so they must be co-resident
    if (n == 1) {
        void* params[] = {const_cast<DispatchArgs*>(&a0)};
        return cudaLaunchCooperativeKernel(fn, grid, block, params, shape.smem_bytes, stream);
    }
    DispatchArgs* dev = nullptr;
    err = cudaMallocAsync(reinterpret_cast<void**>(&dev), sizeof(DispatchArgs) * n, stream);
    if (err != cudaSuccess) return err;
    err = cudaMemcpyAsync(dev, args, sizeof(DispatchArgs) * n, cudaMemcpyHostToDevice, stream);
    if (err == cudaSuccess) {
        void* params[] = {&dev};
        err = cudaLaunchCooperativeKernel(fn, grid, block, params, shape.smem_bytes, stream);
    }
    cudaFreeAsync(dev, stream);
    return err;
}

}  // namespace ep
