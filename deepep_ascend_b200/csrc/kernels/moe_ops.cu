// Element-wise pieces of the MoE expert FFN that sit between the two grouped GEMMs: SwiGLU fused with the
// e4m3 (1x128 scales) cast of the second GEMM's input, so the activation is written once in FP8 instead of being
// written in bf16 and re-read by a separate quantisation kernel; and the element-wise kernels of the backward pass,
// which also emit the transposed operands of the weight-gradient GEMMs.
#include <cuda_fp8.h>

#include "common.cuh"

namespace ep {

namespace {

// one warp per row; each step covers 256 channels (two 128-channel scale groups).  The loads of two steps are issued
// before the arithmetic of the first, the sigmoid uses the fast reciprocal (the activation is rounded to bf16 right
// after), and the correctly rounded amax / 448 of a group is computed once per 16 steps by the lane that kept that amax
// (all lanes divide at once) instead of by two lanes in every step.
struct SwigluStep {
    int4 gate, up;
};
__device__ __forceinline__ SwigluStep swiglu_load(const uint8_t* gate, const uint8_t* up, int elem, int I) {
    SwigluStep s;
    if (elem < I) {
        s.gate = ptx::ld_nc_v4(gate + elem * 2);
        s.up = ptx::ld_nc_v4(up + elem * 2);
    } else {
        s.gate = s.up = make_int4(0, 0, 0, 0);
    }
    return s;
}

__global__ void swiglu_quant_kernel(const SwigluQuantArgs a) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= a.rows) return;
    const int I = a.inter;
    const uint8_t* gate = reinterpret_cast<const uint8_t*>(a.h) + static_cast<int64_t>(row) * a.ldh * 2;
    const uint8_t* up = gate + static_cast<int64_t>(I) * 2;
    uint8_t* q = reinterpret_cast<uint8_t*>(a.q) + static_cast<int64_t>(row) * I;
    float* sf_row = a.sf + static_cast<int64_t>(row) * a.sf_stride_row;
    const int iters = (I + 255) / 256, num_groups = (I + 127) / 128;
    float kept = 0.f;                 // amax of the group this lane will divide: step (lane & 15) of the current 16, half lane >> 4
    auto flush_scales = [&](int first_step) {
        const int group = (first_step + (lane & 15)) * 2 + (lane >> 4);
        if (group < num_groups && first_step + (lane & 15) < iters) sf_row[group * a.sf_stride_col] = __fdiv_rn(kept, 448.f);
    };
    SwigluStep cur = swiglu_load(gate, up, lane * 8, I);
    for (int i = 0; i < iters; ++i) {
        const int elem = (i * 32 + lane) * 8;
        const bool in_range = elem < I;
        const SwigluStep nxt = swiglu_load(gate, up, i + 1 < iters ? elem + 256 : I, I);
        float v[8];
        {
            const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&cur.gate);
            const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&cur.up);
            int4 act_raw;
            __nv_bfloat162* ah = reinterpret_cast<__nv_bfloat162*>(&act_raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 gf = __bfloat1622float2(gh[j]), uf = __bfloat1622float2(uh[j]);
                const float a0 = __fdividef(gf.x, 1.f + __expf(-gf.x)) * uf.x, a1 = __fdividef(gf.y, 1.f + __expf(-gf.y)) * uf.y;
                // the activation is rounded to bf16 first so that the FP8 cast sees the same values as a bf16 pipeline
                ah[j] = __floats2bfloat162_rn(a0, a1);
                const float2 r = __bfloat1622float2(ah[j]);
                v[2 * j] = r.x;
                v[2 * j + 1] = r.y;
            }
            if (in_range && a.act_bf16 != nullptr)
                *reinterpret_cast<int4*>(reinterpret_cast<uint8_t*>(a.act_bf16) + (static_cast<int64_t>(row) * I + elem) * 2) = act_raw;
        }
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
        amax = fmaxf(ptx::warp_max_16(amax), 1e-4f);
        const float scale = __fmul_rn(448.f, __frcp_rn(amax));
        if ((lane & 15) == (i & 15)) kept = amax;
        if (in_range) {
            uint32_t packed[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j] * scale, v[4 * j + 1] * scale), __NV_SATFINITE, __NV_E4M3);
                const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j + 2] * scale, v[4 * j + 3] * scale), __NV_SATFINITE, __NV_E4M3);
                packed[j] = lo | (hi << 16);
            }
            *reinterpret_cast<uint2*>(q + elem) = make_uint2(packed[0], packed[1]);
        }
        if ((i & 15) == 15) flush_scales(i - 15);
        cur = nxt;
    }
    if ((iters & 15) != 0) flush_scales(iters & ~15);
}

// ---------------------------------------------------------------------------------------------- backward pass
// 64 x 64 tiles, 256 threads: thread (pair = tid / 8, c8 = tid % 8) owns rows 2 * pair, 2 * pair + 1 and the eight
// columns c8 * 8 ...  Results are written row-major straight from registers and, through a transposed
// shared-memory tile, column-major in 128-byte runs.
constexpr int kTile = 64, kTileThreads = 256;
constexpr int kTStride = 66;   // bf16 elements per transposed tile row (132 bytes: 4-byte aligned, 2-way bank conflicts at most)

struct TileT {
    __nv_bfloat16 v[kTile][kTStride];
};

// stash the two rows' values of column `col` (rows 2 * pair and 2 * pair + 1 of the tile) as one 4-byte word
__device__ __forceinline__ void stash_pair(TileT& t, int col, int pair, float lo, float hi) {
    *reinterpret_cast<__nv_bfloat162*>(&t.v[col][2 * pair]) = __floats2bfloat162_rn(lo, hi);
}
// write the tile transposed: out_t[(col0 + c) * ld + row0 + 0..63], one 128-byte run per warp instruction
__device__ __forceinline__ void flush_transposed(const TileT& t, void* out_t, int64_t ld, int col0, int row0) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int i = 0; i < kTile / (kTileThreads / 32); ++i) {
        const int c = warp * (kTile / (kTileThreads / 32)) + i;
        const uint32_t word = *reinterpret_cast<const uint32_t*>(&t.v[c][2 * lane]);
        *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(out_t) + ((col0 + c) * ld + row0 + 2 * lane) * 2) = word;
    }
}
__device__ __forceinline__ void unpack8(const int4& raw, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 v = __bfloat1622float2(h[j]);
        f[2 * j] = v.x;
        f[2 * j + 1] = v.y;
    }
}
__device__ __forceinline__ int4 pack8(const float (&f)[8]) {
    int4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
    return raw;
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// grid (rows / 64, ceil(H / kPrepCols)): one CTA = 64 rows x kPrepCols columns; the per-row dot product of its columns goes
// to row_dot[blockIdx.y * rows + row] and the caller adds the column blocks up (fixed order, so the result is deterministic)
constexpr int kPrepCols = 512;

__global__ void __launch_bounds__(kTileThreads) moe_bwd_prep_kernel(const MoeBwdArgs a) {
    __shared__ TileT tile;
    const int pair = threadIdx.x >> 3, c8 = threadIdx.x & 7;
    const int row0 = blockIdx.x * kTile;
    const int H = a.cols;
    const int col_begin = blockIdx.y * kPrepCols, col_end = min(H, col_begin + kPrepCols);
    const uint8_t* gb = reinterpret_cast<const uint8_t*>(a.g);
    const uint8_t* yb = reinterpret_cast<const uint8_t*>(a.y);
    uint8_t* ob = reinterpret_cast<uint8_t*>(a.out);
    float dot[2] = {0.f, 0.f}, w[2];
    bool ok[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row0 + 2 * pair + r;
        ok[r] = a.valid[row] != 0;
        w[r] = ok[r] ? a.w[row] : 0.f;
    }
    for (int col0 = col_begin; col0 < col_end; col0 += kTile) {
        float res[2][8];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int64_t off = (static_cast<int64_t>(row0 + 2 * pair + r) * H + col0 + c8 * 8) * 2;
            float g[8], y[8];
            if (ok[r]) {
                unpack8(ptx::ld_nc_v4(gb + off), g);
                if (yb != nullptr) unpack8(ptx::ld_nc_v4(yb + off), y);
                else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) y[j] = 0.f;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) g[j] = y[j] = 0.f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                dot[r] = fmaf(g[j], y[j], dot[r]);
                res[r][j] = round_bf16(g[j] * w[r]);
            }
            if (ob != nullptr) *reinterpret_cast<int4*>(ob + off) = pack8(res[r]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) stash_pair(tile, c8 * 8 + j, pair, res[0][j], res[1][j]);
        __syncthreads();
        flush_transposed(tile, a.out_t, a.rows, col0, row0);
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float d = dot[r];
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        d += __shfl_xor_sync(0xffffffffu, d, 2);
        d += __shfl_xor_sync(0xffffffffu, d, 4);
        if (c8 == 0 && a.row_dot != nullptr) a.row_dot[static_cast<int64_t>(blockIdx.y) * a.rows + row0 + 2 * pair + r] = d;
    }
}

// grid (rows / 64, I / 64)
__global__ void __launch_bounds__(kTileThreads) moe_bwd_swiglu_kernel(const MoeBwdArgs a) {
    __shared__ TileT t_gate, t_up, t_act;
    const int pair = threadIdx.x >> 3, c8 = threadIdx.x & 7;
    const int row0 = blockIdx.x * kTile, col0 = blockIdx.y * kTile;
    const int I = a.cols;
    const uint8_t* db = reinterpret_cast<const uint8_t*>(a.g);
    const uint8_t* hb = reinterpret_cast<const uint8_t*>(a.y);
    uint8_t* ob = reinterpret_cast<uint8_t*>(a.out);
    float dg[2][8], du[2][8], act[2][8], dot[2] = {0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row0 + 2 * pair + r;
        const int col = col0 + c8 * 8;
        if (a.valid[row] != 0) {
            float d[8], gate[8], up[8];
            unpack8(ptx::ld_nc_v4(db + (static_cast<int64_t>(row) * I + col) * 2), d);
            const float wr = a.w != nullptr ? a.w[row] : 1.f;
            unpack8(ptx::ld_nc_v4(hb + (static_cast<int64_t>(row) * 2 * I + col) * 2), gate);
            unpack8(ptx::ld_nc_v4(hb + (static_cast<int64_t>(row) * 2 * I + I + col) * 2), up);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float sig = 1.f / (1.f + __expf(-gate[j]));
                act[r][j] = round_bf16(gate[j] * sig * up[j]);
                // d[j] is the gradient w.r.t. the UNWEIGHTED activation when a row weight is given: its product with the
                // activation is d loss / d weight, and the weight enters the gradients that flow on
                dot[r] = fmaf(d[j], act[r][j], dot[r]);
                const float dj = d[j] * wr;
                du[r][j] = round_bf16(dj * gate[j] * sig);
                dg[r][j] = round_bf16(dj * up[j] * sig * (1.f + gate[j] * (1.f - sig)));
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) act[r][j] = du[r][j] = dg[r][j] = 0.f;
        }
        *reinterpret_cast<int4*>(ob + (static_cast<int64_t>(row) * 2 * I + col) * 2) = pack8(dg[r]);
        *reinterpret_cast<int4*>(ob + (static_cast<int64_t>(row) * 2 * I + I + col) * 2) = pack8(du[r]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        stash_pair(t_gate, c8 * 8 + j, pair, dg[0][j], dg[1][j]);
        stash_pair(t_up, c8 * 8 + j, pair, du[0][j], du[1][j]);
        stash_pair(t_act, c8 * 8 + j, pair, act[0][j], act[1][j]);
    }
    __syncthreads();
    flush_transposed(t_gate, a.out_t, a.rows, col0, row0);
    flush_transposed(t_up, a.out_t, a.rows, I + col0, row0);
    flush_transposed(t_act, a.out2_t, a.rows, col0, row0);
    if (a.row_dot != nullptr) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float d = dot[r];
            d += __shfl_xor_sync(0xffffffffu, d, 1);
            d += __shfl_xor_sync(0xffffffffu, d, 2);
            d += __shfl_xor_sync(0xffffffffu, d, 4);
            if (c8 == 0) a.row_dot[static_cast<int64_t>(blockIdx.y) * a.rows + row0 + 2 * pair + r] = d;
        }
    }
}

// grid (rows / 64, H / 64)
__global__ void __launch_bounds__(kTileThreads) moe_bwd_dequant_t_kernel(const MoeBwdArgs a) {
    __shared__ TileT tile;
    const int pair = threadIdx.x >> 3, c8 = threadIdx.x & 7;
    const int row0 = blockIdx.x * kTile, col0 = blockIdx.y * kTile;
    const int H = a.cols;
    const uint8_t* qb = reinterpret_cast<const uint8_t*>(a.y);
    float x[2][8];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row0 + 2 * pair + r;
        const int col = col0 + c8 * 8;
        if (a.valid[row] != 0) {
            const uint2 raw = *reinterpret_cast<const uint2*>(qb + static_cast<int64_t>(row) * H + col);
            const float sf = __ldg(a.w + row * a.sf_stride_row + (col / 128) * a.sf_stride_col);
            const __nv_fp8x2_storage_t* p = reinterpret_cast<const __nv_fp8x2_storage_t*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(p[j], __NV_E4M3);
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
                x[r][2 * j] = f.x * sf;
                x[r][2 * j + 1] = f.y * sf;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) x[r][j] = 0.f;
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) stash_pair(tile, c8 * 8 + j, pair, x[0][j], x[1][j]);
    __syncthreads();
    flush_transposed(tile, a.out_t, a.rows, col0, row0);
}


// Expand-layout bookkeeping of a grouped GEMM in one launch: from the inclusive segment ends (segment e starts at
// align(end[e - 1], alignment) and holds end[e] - start rows) -> the weights group of every 128-row tile (-1: no token
// in the tile), one validity byte per row (0: alignment padding) and the aligned segment boundaries [G + 1].
constexpr int kSegThreads = 256;
__global__ void __launch_bounds__(kSegThreads) expert_segments_kernel(const ExpertSegmentsArgs a) {
    extern __shared__ int s_seg[];                    // aligned ends [G]
    for (int e = threadIdx.x; e < a.num_groups; e += kSegThreads)
        s_seg[e] = (__ldg(a.psum_ends + e) + a.alignment - 1) / a.alignment * a.alignment;
    __syncthreads();
    if (blockIdx.x == 0 && a.seg_off != nullptr) {
        for (int e = threadIdx.x; e <= a.num_groups; e += kSegThreads) a.seg_off[e] = e == 0 ? 0 : s_seg[e - 1];
    }
    const int padded_rows = (a.num_rows + 127) / 128 * 128;
    for (int row = blockIdx.x * kSegThreads + threadIdx.x; row < padded_rows; row += gridDim.x * kSegThreads) {
        // first segment whose aligned end lies beyond the row
        int lo = 0, hi = a.num_groups;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (s_seg[mid] > row) hi = mid;
            else lo = mid + 1;
        }
        const bool in_segment = lo < a.num_groups && row < __ldg(a.psum_ends + lo);
        if (row < a.num_rows && a.valid_row != nullptr) a.valid_row[row] = in_segment ? 1 : 0;
        if ((row & 127) == 0 && a.tile_group != nullptr) a.tile_group[row >> 7] = in_segment ? lo : -1;
    }
}

// ------------------------------------------------------------------------------------------------ local expansion
// PLAN, two launches that each read the ids once.  The (row, k) pairs are cut into one contiguous share per warp
// (kPlanWarps warps per CTA).  COUNT: every warp counts its pairs per expert.  ASSIGN: a warp's first number for expert e
// is the segment start plus the counts of all warps before it, and inside its share the warp numbers the pairs in
// order (match_any groups the lanes of a step by expert), so the rows of an expert segment are ordered by received
// row: the same result on every run.
constexpr int kPlanWarps = 8;
__device__ __forceinline__ int plan_id(const LocalExpandPlanArgs& a, int i, int total) {   // rows * K < 2^31
    if (i >= total) return -1;
    const int row = i / a.num_topk;
    const int64_t at = static_cast<int64_t>(row) * a.idx_pitch + (i - row * a.num_topk);
    const long long id = a.idx_is_64 ? __ldg(reinterpret_cast<const long long*>(a.recv_idx) + at)
                                     : static_cast<long long>(__ldg(reinterpret_cast<const int*>(a.recv_idx) + at));
    return id >= 0 && id < a.num_local_experts ? static_cast<int>(id) : -1;
}
// share of warp `w` of the grid: multiples of 32 pairs
__device__ __forceinline__ void plan_share(const LocalExpandPlanArgs& a, int w, int num_warps, int& lo, int& hi) {
    const int total = a.num_rows * a.num_topk;
    const int share = ((total + num_warps * 32 - 1) / (num_warps * 32)) * 32;
    lo = min(w * share, total);
    hi = min(lo + share, total);
}
__global__ void __launch_bounds__(kPlanWarps * 32) local_expand_count_kernel(const LocalExpandPlanArgs a) {
    extern __shared__ int s_plan[];                    // [kPlanWarps][El]
    const int El = a.num_local_experts, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int* mine = s_plan + warp * El;
    for (int e = lane; e < El; e += 32) mine[e] = 0;
    __syncwarp();
    int lo, hi;
    plan_share(a, blockIdx.x * kPlanWarps + warp, gridDim.x * kPlanWarps, lo, hi);
    constexpr int kBatch = 4;
    for (int first = lo; first < hi; first += 32 * kBatch) {
        int id[kBatch];
#pragma unroll
        for (int j = 0; j < kBatch; ++j) id[j] = plan_id(a, first + j * 32 + lane, hi);
#pragma unroll
        for (int j = 0; j < kBatch; ++j)
            if (id[j] >= 0) atomicAdd(mine + id[j], 1);
    }
    __syncthreads();
    // per-warp counts and, for the prefix over CTAs, their sum
    int* out = a.warp_counts + static_cast<int64_t>(blockIdx.x * kPlanWarps + warp) * El;
    for (int e = lane; e < El; e += 32) out[e] = mine[e];
    for (int e = threadIdx.x; e < El; e += kPlanWarps * 32) {
        int sum = 0;
        for (int w = 0; w < kPlanWarps; ++w) sum += s_plan[w * El + e];
        a.cta_counts[static_cast<int64_t>(blockIdx.x) * El + e] = sum;
    }
}
__global__ void __launch_bounds__(kPlanWarps * 32) local_expand_assign_kernel(const LocalExpandPlanArgs a) {
    extern __shared__ int s_plan[];                    // [kPlanWarps][El] next number of every expert for each warp
    const int El = a.num_local_experts, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int me = blockIdx.x * kPlanWarps + warp, num_warps = gridDim.x * kPlanWarps;
    int* next = s_plan + warp * El;
    for (int e = lane; e < El; e += 32) {
        int before = e == 0 ? 0 : __ldg(a.seg_end_aligned + e - 1), all = before;
        for (int b = 0; b < static_cast<int>(gridDim.x); ++b) {
            const int c = __ldg(a.cta_counts + static_cast<int64_t>(b) * El + e);
            before += b < static_cast<int>(blockIdx.x) ? c : 0;
            all += c;
        }
        for (int w = 0; w < warp; ++w) before += __ldg(a.warp_counts + static_cast<int64_t>(blockIdx.x * kPlanWarps + w) * El + e);
        next[e] = before;
        if (me == 0) a.seg_end[e] = all;
    }
    __syncwarp();
    int lo, hi;
    plan_share(a, me, num_warps, lo, hi);
    constexpr int kBatch = 4;
    for (int first = lo; first < hi; first += 32 * kBatch) {
        int id[kBatch];
#pragma unroll
        for (int j = 0; j < kBatch; ++j) id[j] = plan_id(a, first + j * 32 + lane, hi);
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
            // lanes with the same expert: the lowest takes the numbers for all of them
            const uint32_t peers = __match_any_sync(0xffffffffu, id[j]);
            if (id[j] >= 0) {
                const int leader = __ffs(peers) - 1;
                int base = 0;
                if (lane == leader) {
                    base = next[id[j]];
                    next[id[j]] = base + __popc(peers);
                }
                base = __shfl_sync(peers, base, leader);
                a.pos[first + j * 32 + lane] = base + __popc(peers & ptx::lanemask_lt());
            }
            __syncwarp();
        }
    }
}

// COPY: one warp per received row; every 512-byte piece is read once and written to each expert row of the row.
constexpr int kExpandWarps = 8, kMaxExpandTopk = 32;
__global__ void __launch_bounds__(kExpandWarps * 32) local_expand_copy_kernel(const LocalExpandCopyArgs a) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * kExpandWarps + (threadIdx.x >> 5);
    if (row >= a.num_rows) return;
    const int my_pos = lane < a.num_topk ? __ldg(a.pos + static_cast<int64_t>(row) * a.num_topk + lane) : -1;
    uint32_t dests = __ballot_sync(0xffffffffu, my_pos >= 0);
    if (dests == 0) return;
    if (a.w_src != nullptr && my_pos >= 0) a.w_dst[my_pos] = __ldg(a.w_src + static_cast<int64_t>(row) * a.w_pitch + lane);
    const uint8_t* src = reinterpret_cast<const uint8_t*>(a.src) + static_cast<int64_t>(row) * a.src_pitch;
    uint8_t* dst = reinterpret_cast<uint8_t*>(a.dst);
    const int pieces = a.row_bytes / 16;
    for (int p0 = 0; p0 < pieces; p0 += 128) {
        int4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int p = p0 + j * 32 + lane;
            v[j] = p < pieces ? ptx::ld_nc_v4(src + p * 16) : make_int4(0, 0, 0, 0);
        }
        for (uint32_t m = dests; m != 0; m &= m - 1) {
            const int64_t to = __shfl_sync(0xffffffffu, my_pos, __ffs(m) - 1);
            uint8_t* out = dst + to * a.row_bytes;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int p = p0 + j * 32 + lane;
                if (p < pieces) *reinterpret_cast<int4*>(out + p * 16) = v[j];
            }
        }
    }
    if (a.sf_src != nullptr) {
        for (int c = lane; c < a.sf_cols; c += 32) {
            const float f = __ldg(a.sf_src + static_cast<int64_t>(row) * a.sf_stride_row + c * a.sf_stride_col);
            for (uint32_t m = dests; m != 0; m &= m - 1) {
                const int64_t to = __shfl_sync(0xffffffffu, my_pos, __ffs(m) - 1);
                a.sf_dst[to * a.sf_cols + c] = f;
            }
        }
    }
}

// REDUCE: one warp per received row; fp32 sum of its expert rows (in top-k order), optionally weighted, rounded once to bf16.
__global__ void __launch_bounds__(kExpandWarps * 32) local_reduce_kernel(const LocalReduceArgs a) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * kExpandWarps + (threadIdx.x >> 5);
    if (row >= a.num_rows) return;
    const int my_pos = lane < a.num_topk ? __ldg(a.pos + static_cast<int64_t>(row) * a.num_topk + lane) : -1;
    const float my_w = (a.w != nullptr && my_pos >= 0) ? __ldg(a.w + my_pos) : 1.f;
    const uint32_t srcs = __ballot_sync(0xffffffffu, my_pos >= 0);
    const uint8_t* src = reinterpret_cast<const uint8_t*>(a.src);
    uint8_t* out = reinterpret_cast<uint8_t*>(a.dst) + static_cast<int64_t>(row) * a.cols * 2;
    const int pieces = a.cols / 8;            // 16-byte pieces of 8 bf16
    constexpr int kPer = 4;                   // pieces per lane and step: the loads of a step are issued together
    for (int p0 = 0; p0 < pieces; p0 += 32 * kPer) {
        float acc[kPer][8];
#pragma unroll
        for (int j = 0; j < kPer; ++j)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[j][i] = 0.f;
        for (uint32_t m = srcs; m != 0; m &= m - 1) {
            const int k = __ffs(m) - 1;
            const int64_t from = __shfl_sync(0xffffffffu, my_pos, k);
            const float w = __shfl_sync(0xffffffffu, my_w, k);
            const uint8_t* in = src + from * a.cols * 2;
            int4 v[kPer];
#pragma unroll
            for (int j = 0; j < kPer; ++j) {
                const int p = p0 + j * 32 + lane;
                v[j] = p < pieces ? ptx::ld_nc_v4(in + p * 16) : make_int4(0, 0, 0, 0);
            }
#pragma unroll
            for (int j = 0; j < kPer; ++j) {
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[j]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(h[i]);
                    acc[j][2 * i] = fmaf(w, f.x, acc[j][2 * i]);
                    acc[j][2 * i + 1] = fmaf(w, f.y, acc[j][2 * i + 1]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
            const int p = p0 + j * 32 + lane;
            if (p < pieces) {
                int4 o;
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(acc[j][2 * i], acc[j][2 * i + 1]);
                *reinterpret_cast<int4*>(out + p * 16) = o;
            }
        }
    }
}
}  // namespace

int moe_bwd_prep_col_blocks(int cols) { return (cols + kPrepCols - 1) / kPrepCols; }

cudaError_t launch_moe_bwd(const MoeBwdArgs& a, cudaStream_t stream) {
    if (a.rows == 0) return cudaSuccess;
    if (a.rows % kTile != 0 || a.cols % kTile != 0) return cudaErrorInvalidValue;
    if (a.op == EP_MOE_BWD_PREP) moe_bwd_prep_kernel<<<dim3(a.rows / kTile, (a.cols + kPrepCols - 1) / kPrepCols), kTileThreads, 0, stream>>>(a);
    else if (a.op == EP_MOE_BWD_SWIGLU) moe_bwd_swiglu_kernel<<<dim3(a.rows / kTile, a.cols / kTile), kTileThreads, 0, stream>>>(a);
    else if (a.op == EP_MOE_BWD_DEQUANT_T) moe_bwd_dequant_t_kernel<<<dim3(a.rows / kTile, a.cols / kTile), kTileThreads, 0, stream>>>(a);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

cudaError_t launch_local_expand_plan(const LocalExpandPlanArgs& a, cudaStream_t stream) {
    if (a.num_local_experts < 1 || a.num_topk < 1 || a.num_topk > kMaxExpandTopk || a.num_rows < 0) return cudaErrorInvalidValue;
    if (a.num_ctas < 1 || a.num_local_experts > 1024 || a.warp_counts == nullptr || a.cta_counts == nullptr) return cudaErrorInvalidValue;
    const size_t smem = static_cast<size_t>(kPlanWarps) * a.num_local_experts * sizeof(int);
    local_expand_count_kernel<<<a.num_ctas, kPlanWarps * 32, smem, stream>>>(a);
    local_expand_assign_kernel<<<a.num_ctas, kPlanWarps * 32, smem, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_local_expand_copy(const LocalExpandCopyArgs& a, cudaStream_t stream) {
    if (a.num_rows == 0) return cudaSuccess;
    if (a.num_topk < 1 || a.num_topk > kMaxExpandTopk || a.row_bytes % 16 != 0 || a.src_pitch % 16 != 0 ||
        reinterpret_cast<uintptr_t>(a.src) % 16 != 0 || reinterpret_cast<uintptr_t>(a.dst) % 16 != 0)
        return cudaErrorInvalidValue;
    local_expand_copy_kernel<<<(a.num_rows + kExpandWarps - 1) / kExpandWarps, kExpandWarps * 32, 0, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_local_reduce(const LocalReduceArgs& a, cudaStream_t stream) {
    if (a.num_rows == 0) return cudaSuccess;
    if (a.num_topk < 1 || a.num_topk > kMaxExpandTopk || a.cols % 8 != 0 || reinterpret_cast<uintptr_t>(a.src) % 16 != 0 ||
        reinterpret_cast<uintptr_t>(a.dst) % 16 != 0)
        return cudaErrorInvalidValue;
    local_reduce_kernel<<<(a.num_rows + kExpandWarps - 1) / kExpandWarps, kExpandWarps * 32, 0, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_expert_segments(const ExpertSegmentsArgs& a, cudaStream_t stream) {
    if (a.num_groups < 1 || a.num_groups > 8192 || a.alignment < 128 || a.alignment % 128 != 0 || a.num_rows < 0) return cudaErrorInvalidValue;
    const int blocks = max(1, min(1024, (a.num_rows + kSegThreads - 1) / kSegThreads));
    expert_segments_kernel<<<blocks, kSegThreads, a.num_groups * sizeof(int), stream>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_swiglu_quant(const SwigluQuantArgs& a, cudaStream_t stream) {
    if (a.rows == 0) return cudaSuccess;
    const int warps = 8;
    swiglu_quant_kernel<<<(a.rows + warps - 1) / warps, warps * 32, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace ep
