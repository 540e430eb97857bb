// Persistent tcgen05 GEMM for sm_100a: C[M, N] (bf16) = A[M, K] * B[g][N, K]^T.
//
//   warp 0   : TMA producer - 2-D tiled loads of 128 x 128-byte A and B tiles (128B swizzle) into a ring of
//              shared-memory stages, completion counted on mbarriers; optionally waits for an "A rows are ready"
//              flag per M tile (all-gather fused into the loads)
//   warp 1   : MMA issuer   - one elected thread issues tcgen05.mma (kind::f16 for bf16, kind::f8f6f4 for e4m3)
//              with fp32 accumulators in tensor memory; tcgen05.commit releases stages and publishes accumulators
//   warps 2-5 (2-9 for e4m3): epilogue - tcgen05.ld the accumulator (each warp its 32 TMEM lanes), scale / convert, store bf16
//
// bf16 operands: one accumulator per output tile, two TMEM buffers so the epilogue of tile i overlaps the MMAs of
// tile i+1.  e4m3 operands with fp32 block scales (A: per row x 128 channels, B: per 128 x 128 block): every
// 128-channel block is accumulated into its own TMEM buffer and promoted into fp32 registers with its scale by
// EIGHT epilogue warps (two per TMEM lane quadrant, 64 columns each, both tcgen05.ld of a block in flight before one
// wait); four TMEM buffers let the MMAs run up to three blocks ahead of the promotion.
// Grouped (MoE) use: `tile_group[m_tile]` selects the expert whose weights multiply that 128-row tile.
// Every pipeline wait is bounded; on expiry the kernel raises `*error`, leaves its loops and frees its TMEM.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "gemm_sm100.cuh"

namespace ep {

namespace {

constexpr int kBlockM = 128, kTileBytes = 128 * 128;   // A tile: 128 rows x 128 bytes; B tile: kBlockN rows x 128 bytes
constexpr int kMaxStages = 7;
constexpr int kEpiRowBytes = 128 * 2 + 16;              // one staged bf16 output row (128 columns), padded against bank conflicts
constexpr int kEpiStageBytes = 4 * 32 * kEpiRowBytes;   // four epilogue warps x 32 rows
// shared memory: [A stages | B stages | barriers (1 KB) | epilogue staging]
__host__ __device__ constexpr int stage_bytes(int block_n) { return kTileBytes + block_n * 128; }
// e4m3 tiles carry half the math per byte of bf16 tiles, so that kernel keeps as many bytes in flight as fit (7 stages)
__host__ __device__ constexpr int num_stages(int block_n, bool fp8) { return block_n == 256 ? 4 : (fp8 ? 7 : 5); }
__host__ __device__ constexpr int gemm_smem_bytes(int block_n, bool fp8) {
    return num_stages(block_n, fp8) * stage_bytes(block_n) + 1024 + (block_n == 128 && !fp8 ? kEpiStageBytes : 0);
}
constexpr int kMaxCopyWarps = 6;
// copy warps of a copier CTA (all-gather fusion): each owns two 16 KB staging buffers in the shared memory that the tensor-core
// CTAs use for their operand stages: 160 KB with 128-column tiles (five warps), at least 192 KB with wider tiles (all six warps)
__host__ __device__ constexpr int copy_warps(int block_n) { return block_n == 128 ? 5 : 6; }
constexpr int kGemmThreads = 192;        // bf16: TMA warp, MMA warp, 4 epilogue warps
constexpr int kGemmThreadsFp8 = 320;     // e4m3, 128-column tiles: TMA warp, MMA warp, 8 epilogue warps
constexpr int kGemmThreadsFp8Wide = 384; // e4m3, 256-column tiles: one producer warpgroup (TMA, MMA, two idle warps) that gives its
                                         // registers to the two epilogue warpgroups (128 fp32 sums + 64 loaded values per thread)
__host__ __device__ constexpr int gemm_threads(bool fp8, int block_n) {
    return fp8 ? (block_n == 256 ? kGemmThreadsFp8Wide : kGemmThreadsFp8) : kGemmThreads;
}
template <int kRegs>
__device__ __forceinline__ void reg_alloc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void reg_dealloc() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}
constexpr int kMaxAccBufs = 4;
constexpr uint64_t kDefaultWaitLimitNs = 4ull * 1000 * 1000 * 1000;   // when the caller gives no limit

struct GemmSmem {
    uint64_t full[kMaxStages], empty[kMaxStages], tmem_full[kMaxAccBufs], tmem_empty[kMaxAccBufs];
    uint64_t copy_bar[kMaxCopyWarps][2];
    uint32_t tmem_base;
    int failed;
};

__device__ __forceinline__ uint64_t gemm_timer() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint64_t wait_limit_ns(const GemmArgs& g) { return g.timeout_ns != 0 ? g.timeout_ns : kDefaultWaitLimitNs; }

// A pipeline wait ran out: stop this CTA's loops, raise the per-device flag and, when the caller gave the status block of
// a communication buffer, record the failure there too, so that the buffer's check_status() reports it and poisons the
// buffer like any other failed device wait.  `code`: 1 = empty stage, 2 = free accumulator, 3 = rows-ready flag,
// 4 = full stage, 5 = finished accumulator, 7 = all-gather copy.
__device__ __noinline__ void gemm_fail(const GemmArgs& g, GemmSmem* sm, int code) {
    sm->failed = code;
    if (g.error != nullptr && atomicCAS(g.error, 0, code) == 0 && g.status != nullptr) {
        volatile uint64_t* st = g.status;
        st[EP_STATUS_PHASE] = EP_PH_GEMM_PIPE;
        st[EP_STATUS_PEER] = static_cast<uint64_t>(-1ll);
        st[EP_STATUS_EXPECTED] = static_cast<uint64_t>(code);
        st[EP_STATUS_OBSERVED] = blockIdx.x;
        st[EP_STATUS_RANK] = static_cast<uint64_t>(g.status_rank);
        __threadfence_system();
        st[EP_STATUS_CODE] = EP_ERR_TIMEOUT;
        __threadfence_system();
    }
}

// bounded mbarrier wait; returns false (and raises the failure flags) when the limit runs out
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, GemmSmem* sm, const GemmArgs& g, int code) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = gemm_timer();
    uint32_t spins = 0;
    while (!ptx::mbar_try_wait(bar, parity)) {
        if ((++spins & 63u) == 0u) {
            if (*reinterpret_cast<volatile int*>(&sm->failed)) return false;
            if (gemm_timer() - t0 > wait_limit_ns(g)) {
                gemm_fail(g, sm, code);
                return false;
            }
        }
    }
    return true;
}

// Tile order: M tiles are walked in groups of `group_m`; inside a group consecutive tiles step through M first, so
// the tiles that run at the same time share few distinct A and B tiles and stay in L2.
struct TileCoord {
    int m, n;
};
__device__ __forceinline__ TileCoord tile_coord(int tile, int num_m, int num_n, int group_m, int m_offset) {
    const int per_group = group_m * num_n;
    const int grp = tile / per_group, in_grp = tile - grp * per_group;
    const int first_m = grp * group_m;
    const int gm = min(group_m, num_m - first_m);
    TileCoord c;
    c.m = (first_m + in_grp % gm + m_offset) % num_m;
    c.n = in_grp / gm;
    return c;
}

// What one tile index means: output tile (m, n), weights group of B, K blocks [kb0, kb1), first output row of its group.
struct TileWork {
    int m, n, grp, kb0, kb1;
    int64_t c_row0;
};
__device__ __forceinline__ TileWork tile_work(const GemmArgs& g, int tile, int num_m, int num_n, int num_k, int group_m, int block_k) {
    TileWork w;
    int e = 0;
    if (g.k_group_off != nullptr) {
        e = tile / (num_m * num_n);
        tile -= e * num_m * num_n;
    }
    const TileCoord tc = tile_coord(tile, num_m, num_n, group_m, g.m_tile_offset);
    w.m = tc.m;
    w.n = tc.n;
    if (g.k_group_off != nullptr) {
        w.grp = 0;
        w.kb0 = __ldg(g.k_group_off + e) / block_k;
        w.kb1 = __ldg(g.k_group_off + e + 1) / block_k;
        w.c_row0 = static_cast<int64_t>(e) * g.M;
    } else {
        w.grp = g.tile_group != nullptr ? __ldg(g.tile_group + tc.m) : 0;
        w.kb0 = 0;
        w.kb1 = num_k;
        w.c_row0 = 0;
    }
    return w;
}

template <int kStages>
struct PipeState {
    int stage = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void advance() {
        if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
        }
    }
};

template <bool kFp8, int kBlockN>
__global__ void __launch_bounds__(gemm_threads(kFp8, kBlockN), 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmArgs g) {
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr int kStages = num_stages(kBlockN, kFp8);
    constexpr int kTileBytesB = kBlockN * 128;
    constexpr int kAccBufs = (kFp8 && kBlockN == 128) ? 4 : 2;   // accumulator buffers of kBlockN fp32 columns in tensor memory
    constexpr int kEpiWarps = kFp8 ? 8 : 4;
    constexpr bool kWide = kFp8 && kBlockN == 256;   // register re-allocation between warpgroups
    constexpr int kEpiWarp0 = kWide ? 4 : 2;         // first epilogue warp
    constexpr int kTmemColumns = kAccBufs * kBlockN <= 256 ? 256 : 512;   // allocations are powers of two
    static_assert(kBlockN % 32 == 0 && kBlockN >= 32 && kBlockN <= 256 && kAccBufs * kBlockN <= 512, "tile width");
    uint8_t* s_a = smem;
    uint8_t* s_b = smem + kStages * kTileBytes;
    GemmSmem* sm = reinterpret_cast<GemmSmem*>(smem + kStages * (kTileBytes + kTileBytesB));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int kBlockK = kFp8 ? 128 : 64;          // elements per 128-byte row
    constexpr int kUmmaK = kFp8 ? 32 : 16;            // elements per tcgen05.mma (32 bytes of K)
    constexpr uint32_t kIdesc = umma::make_instr_desc(kBlockM, kBlockN, kFp8 ? umma::kFormatE4M3 : umma::kFormatBF16);
    const int num_m = (g.M + kBlockM - 1) / kBlockM, num_n = (g.N + kBlockN - 1) / kBlockN;
    const int num_k = (g.K + kBlockK - 1) / kBlockK;
    const int num_tiles = num_m * num_n * (g.k_group_off != nullptr ? g.num_groups : 1);
    const int gemm_ctas = static_cast<int>(gridDim.x) - g.num_copy_ctas;
    const bool is_copier = static_cast<int>(blockIdx.x) >= gemm_ctas;
    uint8_t* s_epi = smem + kStages * (kTileBytes + kTileBytesB) + 1024;   // present only in the 128-column variant
    Workspace* ws = g.fuse != EP_GEMM_FUSE_NONE ? local_ws(g.ctx) : nullptr;
    const uint64_t epoch = ws != nullptr ? ws->epoch[EP_CH_GEMM] + 1 : 0;
    const int tiles_per_shard = g.fuse != EP_GEMM_FUSE_NONE ? num_m / g.ctx.num_ranks : num_m;
    // all-gather fusion wants the M tiles in arrival order, so its groups never span two shards
    const int group_m = g.fuse == EP_GEMM_FUSE_ALL_GATHER ? min(8, tiles_per_shard) : 16;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; ++i) {
            ptx::mbar_init(&sm->full[i], 1);
            ptx::mbar_init(&sm->empty[i], 1);
        }
        for (int i = 0; i < kAccBufs; ++i) {
            ptx::mbar_init(&sm->tmem_full[i], 1);
            ptx::mbar_init(&sm->tmem_empty[i], kEpiWarps);
        }
        sm->failed = 0;
        ptx::mbar_fence_init();
        umma::prefetch_tensormap(&map_a);
        umma::prefetch_tensormap(&map_b);
    }
    if (warp == 1) {
        umma::tmem_alloc(&sm->tmem_base, kTmemColumns);
        umma::tmem_relinquish();
    }
    umma::fence_before_thread_sync();
    __syncthreads();
    umma::fence_after_thread_sync();
    const uint32_t tmem_base = sm->tmem_base;

    if (warp < kEpiWarp0) {
        // ---------------------------------------------------------------------- producer warps
        // wide e4m3 kernel: warps 0-3 (TMA, MMA, two idle) keep 40 registers each so that the epilogue warps can take 232
        if (kWide) reg_dealloc<40>();
        if (warp == 0) {
            // ------------------------------------------------------------------ TMA producer
            if (lane == 0) {
                PipeState<kStages> p;
                bool ok = true;
                for (int tile = blockIdx.x; !is_copier && tile < num_tiles && ok; tile += gemm_ctas) {
                    const TileWork tw = tile_work(g, tile, num_m, num_n, num_k, group_m, kBlockK);
                    const int m_blk = tw.m, n_blk = tw.n, grp = tw.grp;
                    if (grp < 0 || tw.kb1 <= tw.kb0) continue;
                    if (g.fuse == EP_GEMM_FUSE_ALL_GATHER && m_blk / tiles_per_shard != g.ctx.rank) {
                        // rows of a remote shard: wait until a copier CTA of this kernel has landed the tile locally
                        const uint64_t* flag = &ws->tile_flags[m_blk];
                        const uint64_t t0 = gemm_timer();
                        while (ptx::ld_acquire_sys(flag) < epoch) {
                            if (gemm_timer() - t0 > wait_limit_ns(g) || *reinterpret_cast<volatile int*>(&sm->failed)) {
                                gemm_fail(g, sm, 3);
                                ok = false;
                                break;
                            }
                        }
                        if (!ok) break;
                        ptx::fence_proxy_async_all();   // the tile was written through the async proxy of another SM
                    }
                    if (g.a_ready_flags != nullptr) {
                        // rows of this M tile arrive from another rank: wait (bounded) for their flag
                        const uint64_t* flag = g.a_ready_flags + (g.a_flag_of_tile != nullptr ? g.a_flag_of_tile[m_blk] : m_blk);
                        const uint64_t t0 = gemm_timer();
                        while (ptx::ld_acquire_sys(flag) < g.a_ready_value) {
                            if (gemm_timer() - t0 > wait_limit_ns(g) || *reinterpret_cast<volatile int*>(&sm->failed)) {
                                gemm_fail(g, sm, 3);
                                ok = false;
                                break;
                            }
                        }
                        if (!ok) break;
                    }
                    for (int kb = tw.kb0; kb < tw.kb1 && ok; ++kb) {
                        ok = wait_bar(&sm->empty[p.stage], p.phase ^ 1, sm, g, 1);
                        if (!ok) break;
                        ptx::mbar_arrive_expect_tx(&sm->full[p.stage], kTileBytes + kTileBytesB);
                        umma::tma_load_2d(s_a + p.stage * kTileBytes, &map_a, kb * kBlockK, m_blk * kBlockM, &sm->full[p.stage]);
                        umma::tma_load_2d(s_b + p.stage * kTileBytesB, &map_b, kb * kBlockK, grp * g.N + n_blk * kBlockN, &sm->full[p.stage]);
                        p.advance();
                    }
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------------------------ MMA issuer
            if (lane == 0) {
                PipeState<kStages> p;
                int acc = 0;
                uint32_t acc_phase = 0;
                bool ok = true;
                for (int tile = blockIdx.x; !is_copier && tile < num_tiles && ok; tile += gemm_ctas) {
                    const TileWork tw = tile_work(g, tile, num_m, num_n, num_k, group_m, kBlockK);
                    if (tw.grp < 0 || tw.kb1 <= tw.kb0) continue;
                    if (!kFp8) {
                        ok = wait_bar(&sm->tmem_empty[acc], acc_phase ^ 1, sm, g, 2);
                        if (!ok) break;
                        umma::fence_after_thread_sync();
                    }
                    for (int kb = tw.kb0; kb < tw.kb1 && ok; ++kb) {
                        if (kFp8) {
                            ok = wait_bar(&sm->tmem_empty[acc], acc_phase ^ 1, sm, g, 2);
                            if (!ok) break;
                        }
                        ok = wait_bar(&sm->full[p.stage], p.phase, sm, g, 4);
                        if (!ok) break;
                        umma::fence_after_thread_sync();
                        const uint64_t desc_a = umma::make_smem_desc_sw128(s_a + p.stage * kTileBytes);
                        const uint64_t desc_b = umma::make_smem_desc_sw128(s_b + p.stage * kTileBytesB);
#pragma unroll
                        for (int k = 0; k < kBlockK / kUmmaK; ++k) {
                            const uint32_t accumulate = kFp8 ? (k != 0) : (kb != tw.kb0 || k != 0);
                            umma::mma_ss<kFp8>(tmem_base + acc * kBlockN, umma::advance_desc_k(desc_a, k * 32), umma::advance_desc_k(desc_b, k * 32),
                                               kIdesc, accumulate);
                        }
                        umma::mma_commit(&sm->empty[p.stage]);       // the stage may be refilled once these MMAs are done
                        p.advance();
                        if (kFp8) {
                            umma::mma_commit(&sm->tmem_full[acc]);   // one 128-channel block is ready for promotion
                            if (++acc == kAccBufs) {
                                acc = 0;
                                acc_phase ^= 1;
                            }
                        }
                    }
                    if (!kFp8 && ok) {
                        umma::mma_commit(&sm->tmem_full[acc]);
                        if (++acc == kAccBufs) {
                            acc = 0;
                            acc_phase ^= 1;
                        }
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (32 TMEM lanes per warp)
        if (kWide) reg_alloc<232>();
        const int quad = warp & 3;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        uint8_t* cb = reinterpret_cast<uint8_t*>(g.c);
        for (int tile = blockIdx.x; !is_copier && tile < num_tiles && ok; tile += gemm_ctas) {
            const TileWork tw = tile_work(g, tile, num_m, num_n, num_k, group_m, kBlockK);
            const int m_blk = tw.m, n_blk = tw.n, grp = tw.grp;
            if (grp < 0) continue;
            const int row = m_blk * kBlockM + quad * 32 + lane;
            const int n0 = n_blk * kBlockN;
            if (tw.kb1 <= tw.kb0) {
                // empty K range (an expert without tokens): the product is zero
                if (row < g.M)
                    for (int col = n0; col < min(n0 + kBlockN, g.N); col += 8)
                        *reinterpret_cast<int4*>(cb + ((tw.c_row0 + row) * g.ldc + col) * 2) = make_int4(0, 0, 0, 0);
                continue;
            }
            const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
            if (!kFp8) {
                ok = wait_bar(&sm->tmem_full[acc], acc_phase, sm, g, 5);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                umma::fence_after_thread_sync();
                const bool to_peer = kBlockN == 128 && g.fuse == EP_GEMM_FUSE_REDUCE_SCATTER;
                uint8_t* my_stage = s_epi + (quad * 32 + lane) * kEpiRowBytes;
                if (to_peer) {
                    ptx::bulk_wait_read<0>();     // the staging rows were the source of the previous tile's stores
                    __syncwarp();
                }
#pragma unroll
                for (int c = 0; c < kBlockN / 32; ++c) {
                    uint32_t r[32];
                    umma::tmem_ld_32x32(tmem_base + lane_addr + acc * kBlockN + c * 32, r);
                    umma::tmem_ld_wait();
                    if (row < g.M) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            const int col = n0 + c * 32 + v * 8;
                            if (col + 8 <= g.N) {
                                int4 out;
                                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                                for (int j = 0; j < 4; ++j)
                                    h[j] = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]));
                                if (to_peer) *reinterpret_cast<int4*>(my_stage + (c * 32 + v * 8) * 2) = out;
                                else *reinterpret_cast<int4*>(cb + ((tw.c_row0 + row) * g.ldc + col) * 2) = out;
                            }
                        }
                    }
                }
                if (to_peer) {
                    // GEMM -> reduce-scatter: this row of the partial result goes to the rank that owns it, into the
                    // slot reserved for this source rank (one 256-byte bulk store per row over NVLink)
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    const int rows_per_rank = g.M / g.ctx.num_ranks;
                    const int owner = row / rows_per_rank, local_row = row - owner * rows_per_rank;
                    uint8_t* dst = g.ctx.peer_base[owner] + g.off_slots + (epoch & 1) * g.slot_set_bytes +
                                   ((static_cast<int64_t>(g.ctx.rank) * rows_per_rank + local_row) * g.N + n0) * 2;
                    ptx::bulk_store(dst, my_stage, kBlockN * 2);
                    ptx::bulk_commit();
                }
                umma::fence_before_thread_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&sm->tmem_empty[acc]);
                if (++acc == kAccBufs) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            } else {
                // this warp promotes one half of the tile's columns for its 32 rows
                constexpr int kCols = kBlockN / 2;
                const int col_half = (warp - kEpiWarp0) >> 2;
                uint64_t sum2[kCols / 2];   // fp32 pairs (columns 2i, 2i + 1)
#pragma unroll
                for (int i = 0; i < kCols / 2; ++i) sum2[i] = 0ull;
                const int num_kb_sf = (g.K + 127) / 128, num_nb_sf = (g.N + 127) / 128;
                // the B scale block of this warp's columns (a half tile never straddles two 128-column blocks)
                const int nb_sf = min((n0 + col_half * kCols) / 128, num_nb_sf - 1);
                const float* sfb = g.sfb + (static_cast<int64_t>(grp) * num_nb_sf + nb_sf) * num_kb_sf;
                float scale_next = (row < g.M ? __ldg(g.sfa + row * g.sfa_stride_row) : 0.f) * __ldg(sfb);
                for (int kb = 0; kb < num_k && ok; ++kb) {
                    const uint64_t scale2 = umma::pack_f32x2(__float_as_uint(scale_next), __float_as_uint(scale_next));
                    if (kb + 1 < num_k)
                        scale_next = (row < g.M ? __ldg(g.sfa + row * g.sfa_stride_row + (kb + 1) * g.sfa_stride_kb) : 0.f) * __ldg(sfb + kb + 1);
                    ok = wait_bar(&sm->tmem_full[acc], acc_phase, sm, g, 5);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    umma::fence_after_thread_sync();
                    const uint32_t taddr = tmem_base + lane_addr + acc * kBlockN + col_half * kCols;
                    if (kCols == 64) {
                        uint32_t r0[32], r1[32];
                        umma::tmem_ld_32x32(taddr, r0);
                        umma::tmem_ld_32x32(taddr + 32, r1);
                        umma::tmem_ld_wait();
                        // the values are in registers: hand the buffer back before the arithmetic
                        umma::fence_before_thread_sync();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(&sm->tmem_empty[acc]);
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            umma::fma_f32x2(sum2[i], umma::pack_f32x2(r0[2 * i], r0[2 * i + 1]), scale2);
                            umma::fma_f32x2(sum2[16 + i], umma::pack_f32x2(r1[2 * i], r1[2 * i + 1]), scale2);
                        }
                    } else {
                        // 128 columns in two steps of two loads each (64 loaded values live at a time)
#pragma unroll
                        for (int c = 0; c < kCols / 64; ++c) {
                            uint32_t r0[32], r1[32];
                            umma::tmem_ld_32x32(taddr + c * 64, r0);
                            umma::tmem_ld_32x32(taddr + c * 64 + 32, r1);
                            umma::tmem_ld_wait();
                            if (c == kCols / 64 - 1) {
                                umma::fence_before_thread_sync();
                                __syncwarp();
                                if (lane == 0) ptx::mbar_arrive(&sm->tmem_empty[acc]);
                            }
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                umma::fma_f32x2(sum2[c * 32 + i], umma::pack_f32x2(r0[2 * i], r0[2 * i + 1]), scale2);
                                umma::fma_f32x2(sum2[c * 32 + 16 + i], umma::pack_f32x2(r1[2 * i], r1[2 * i + 1]), scale2);
                            }
                        }
                    }
                    if (++acc == kAccBufs) {
                        acc = 0;
                        acc_phase ^= 1;
                    }
                }
                if (ok && row < g.M) {
#pragma unroll
                    for (int v = 0; v < kCols / 8; ++v) {
                        const int col = n0 + col_half * kCols + v * 8;
                        if (col + 8 <= g.N) {
                            int4 out;
                            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                float lo, hi;
                                umma::unpack_f32x2(sum2[v * 4 + j], lo, hi);
                                h[j] = __floats2bfloat162_rn(lo, hi);
                            }
                            *reinterpret_cast<int4*>(cb + (static_cast<int64_t>(row) * g.ldc + col) * 2) = out;
                        }
                    }
                }
            }
        }
    }
    constexpr int kCopyWarps = copy_warps(kBlockN);
    static_assert(kFp8 || kCopyWarps * 2 * 16384 <= num_stages(kBlockN, false) * stage_bytes(kBlockN), "copy staging must fit in front of the barriers");
    if (!kFp8 && g.fuse == EP_GEMM_FUSE_ALL_GATHER && is_copier && warp < kCopyWarps) {
        // ------------------------------------------------------------------ all-gather fused into this kernel
        // Copier CTAs pull the remote shards of A, one 128-row tile at a time, from the owners' symmetric buffers
        // (TMA bulk loads over NVLink, no multicast) into the local copy and publish one flag per tile.
        const RankCtx& ctx = g.ctx;
        const int copier = static_cast<int>(blockIdx.x) - gemm_ctas;
        const int row_bytes = g.K * (kFp8 ? 1 : 2);
        uint8_t* stage = smem + static_cast<size_t>(warp) * 2 * 16384;
        uint64_t* bars = sm->copy_bar[warp];
        if (lane == 0) {
            ptx::mbar_init(&bars[0], 1);
            ptx::mbar_init(&bars[1], 1);
            ptx::mbar_fence_init();
        }
        __syncwarp();
        bool alive = !is_aborted(ws);
        // every rank's shard must be in place: the first copier runs the cross-GPU barrier, the others wait for it
        uint64_t* entry_word = &ws->tile_flags[EP_MAX_TILE_FLAGS - 1];
        if (copier == 0 && warp == 0) {
            if (lane < ctx.num_ranks) {
                Workspace* pws = reinterpret_cast<Workspace*>(ctx.peer_base[lane]);
                ptx::red_add_release_sys(&pws->xbar[EP_CH_GEMM][ctx.rank], 1ull);
                const uint64_t* mine = &ws->xbar[EP_CH_GEMM][lane];
                alive = bounded_wait(
                    ctx, ws, EP_PH_XGPU_BARRIER, lane, 2 * epoch - 1, [&] { return ptx::ld_acquire_sys(mine) >= 2 * epoch - 1; },
                    [&] { return ptx::ld_relaxed_sys(mine); });
            }
            alive = __all_sync(0xffffffffu, alive);
            if (lane == 0 && alive) ptx::st_release_sys(entry_word, epoch);
        }
        if (alive)
            alive = bounded_wait(
                ctx, ws, EP_PH_TILE_FLAG, -1, epoch, [&] { return ptx::ld_acquire_sys(entry_word) >= epoch; },
                [&] { return ptx::ld_relaxed_sys(entry_word); });
        alive = __all_sync(0xffffffffu, alive);
        if (!alive) sm->failed = 7;
        asm volatile("bar.sync 1, %0;" ::"r"(kCopyWarps * 32) : "memory");
        if (*reinterpret_cast<volatile int*>(&sm->failed)) alive = false;
        // work item = one 128-row tile of a remote shard, visited in the order in which the tensor-core CTAs need
        // them (nearest rank first); each copy warp keeps two row loads in flight
        uint32_t n_loaded = 0;
        const int num_items = (ctx.num_ranks - 1) * tiles_per_shard;
        for (int item = copier; item < num_items && alive; item += g.num_copy_ctas) {
            const int src = (ctx.rank + 1 + item / tiles_per_shard) % ctx.num_ranks;
            const int m_blk = src * tiles_per_shard + item % tiles_per_shard;
            // this warp's rows of the tile, each moved in pieces of at most one 16 KB staging buffer
            constexpr int kPiece = 16384;
            const int pieces = (row_bytes + kPiece - 1) / kPiece;
            const int my_rows = (kBlockM - warp + kCopyWarps - 1) / kCopyWarps * pieces;   // (row, piece) pairs
            auto row_offset = [&](int i) {
                return g.off_full + (static_cast<int64_t>(m_blk) * kBlockM + warp + (i / pieces) * kCopyWarps) * row_bytes + static_cast<int64_t>(i % pieces) * kPiece;
            };
            auto piece_bytes = [&](int i) { return min(kPiece, row_bytes - (i % pieces) * kPiece); };
            auto issue_load = [&](int i) {
                const uint32_t l = n_loaded + i;
                if (lane == 0) {
                    ptx::mbar_arrive_expect_tx(&bars[l & 1], piece_bytes(i));
                    ptx::bulk_load(stage + (l & 1) * kPiece, ctx.peer_base[src] + row_offset(i), piece_bytes(i), &bars[l & 1]);
                }
            };
            ptx::bulk_wait_read<0>();
            __syncwarp();
            issue_load(0);
            for (int i = 0; i < my_rows && alive; ++i) {
                if (i + 1 < my_rows) {
                    ptx::bulk_wait_read<0>();   // the other stage was the source of the previous piece's store
                    __syncwarp();
                    issue_load(i + 1);
                }
                const uint32_t l = n_loaded + i;
                alive = mbar_wait_bounded(ctx, ws, &bars[l & 1], (l >> 1) & 1, EP_PH_COMBINE_LOAD);
                if (!alive) {
                    sm->failed = 7;
                    break;
                }
                if (lane == 0) ptx::bulk_store(ctx.peer_base[ctx.rank] + row_offset(i), stage + (l & 1) * kPiece, piece_bytes(i));
                ptx::bulk_commit();
            }
            n_loaded += my_rows;
            ptx::bulk_wait<0>();
            __threadfence();
            // all copy warps of this CTA have finished their rows of the tile -> publish it
            asm volatile("bar.sync 1, %0;" ::"r"(kCopyWarps * 32) : "memory");
            if (*reinterpret_cast<volatile int*>(&sm->failed)) alive = false;   // same decision in every copy warp
            if (warp == 0 && lane == 0 && alive) ptx::st_release_sys(&ws->tile_flags[m_blk], epoch);
        }
    }
    if (!kFp8 && g.fuse == EP_GEMM_FUSE_REDUCE_SCATTER) {
        ptx::bulk_commit();
        ptx::bulk_wait<0>();
        __threadfence_system();
    }
    umma::fence_before_thread_sync();
    __syncthreads();
    if (warp == 1) umma::tmem_dealloc(tmem_base, kTmemColumns);

    if (!kFp8 && g.fuse != EP_GEMM_FUSE_NONE) {
        // All partial rows have left this rank (RS) / all pulls from the peers are done (AG): cross-GPU barrier.
        const RankCtx& ctx = g.ctx;
        bool alive = grid_sync(ctx, ws, EP_CH_GEMM, EP_PH_GRID_SYNC);
        if (blockIdx.x == 0) {
            // arrival number 2 * epoch of this channel (the AG entry barrier used 2 * epoch - 1)
            int ok = alive ? 1 : 0;
            if (alive && threadIdx.x < ctx.num_ranks) {
                Workspace* pws = reinterpret_cast<Workspace*>(ctx.peer_base[threadIdx.x]);
                if (g.fuse == EP_GEMM_FUSE_REDUCE_SCATTER) ptx::red_add_release_sys(&pws->xbar[EP_CH_GEMM][ctx.rank], 1ull);   // stands in for the entry arrival
                ptx::red_add_release_sys(&pws->xbar[EP_CH_GEMM][ctx.rank], 1ull);
                const uint64_t* mine = &ws->xbar[EP_CH_GEMM][threadIdx.x];
                ok = bounded_wait(
                    ctx, ws, EP_PH_XGPU_BARRIER, threadIdx.x, 2 * epoch, [&] { return ptx::ld_acquire_sys(mine) >= 2 * epoch; },
                    [&] { return ptx::ld_relaxed_sys(mine); });
            }
            alive = __syncthreads_and(ok) != 0;
        }
        alive = grid_sync(ctx, ws, EP_CH_GEMM, EP_PH_GRID_SYNC) && alive;
        if (g.fuse == EP_GEMM_FUSE_REDUCE_SCATTER && alive) {
            // every rank's partial rows for this rank have arrived: sum the R slots in rank order in fp32
            const int rows_per_rank = g.M / ctx.num_ranks;
            const int64_t vecs = static_cast<int64_t>(rows_per_rank) * g.N / 8;
            const uint8_t* slots = ctx.peer_base[ctx.rank] + g.off_slots + (epoch & 1) * g.slot_set_bytes;
            const int64_t slot_bytes = static_cast<int64_t>(rows_per_rank) * g.N * 2;
            for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < vecs; v += static_cast<int64_t>(gridDim.x) * blockDim.x) {
                float acc[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                for (int r = 0; r < ctx.num_ranks; ++r) {
                    const int4 raw = __ldcg(reinterpret_cast<const int4*>(slots + r * slot_bytes + v * 16));
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __bfloat1622float2(h[j]);
                        acc[2 * j] += f.x;
                        acc[2 * j + 1] += f.y;
                    }
                }
                int4 out;
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
                *reinterpret_cast<int4*>(reinterpret_cast<uint8_t*>(g.rs_out) + v * 16) = out;
            }
        }
        if (blockIdx.x == 0 && threadIdx.x == 0) ws->epoch[EP_CH_GEMM] = epoch;
    }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// K-major [rows, K] operand, box = box_rows (128 or 256) rows x 128 bytes, 128B swizzle, out-of-range elements read as zero
bool make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int64_t ld_elems, bool fp8, int box_rows) {
    EncodeTiledFn encode = get_encode_fn();
    if (encode == nullptr) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_elems * (fp8 ? 1 : 2))};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(fp8 ? 128 : 64), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem_strides[2] = {1, 1};
    return encode(map, fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                  elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

cudaError_t launch_gemm(const GemmArgs& g, int num_sms, cudaStream_t stream) {
    if (g.M <= 0 || g.N <= 0 || g.K <= 0) return cudaSuccess;
    const int elem = g.is_fp8 ? 1 : 2;
    if ((g.lda * elem) % 16 != 0 || (g.ldb * elem) % 16 != 0 || g.ldc % 8 != 0 || g.N % 8 != 0) return cudaErrorInvalidValue;
    if (reinterpret_cast<uintptr_t>(g.a) % 16 != 0 || reinterpret_cast<uintptr_t>(g.b) % 16 != 0 || reinterpret_cast<uintptr_t>(g.c) % 16 != 0)
        return cudaErrorInvalidValue;
    // 128 x 256 output tiles (fewer A re-reads, longer MMAs); the reduce-scatter epilogue (which stages 128-column rows)
    // and narrow outputs use 128 x 128 tiles.  The bf16 kernel also has 128 x 224 tiles and takes them when they need less
    // tensor-core time: fewer idle CTAs in the last wave (8192 x 7168: 1792 tiles of 256 columns are 12.1 waves of 148
    // CTAs, paid as 13; 2048 tiles of 224 columns are 13.8 waves of 7/8 the length), or no half-empty last column tile
    // (N = 896 = 4 x 224).
    int block_n = (g.fuse != EP_GEMM_FUSE_REDUCE_SCATTER && g.N >= 256) ? 256 : 128;
    if (block_n == 256 && !g.is_fp8) {
        const int64_t num_m_tiles = (g.M + kBlockM - 1) / kBlockM, groups = g.k_group_off != nullptr ? g.num_groups : 1;
        const int64_t workers = std::max(1, (num_sms < 1 ? 1 : num_sms) - (g.fuse == EP_GEMM_FUSE_ALL_GATHER ? g.num_copy_ctas : 0));
        auto cost = [&](int bn) {
            const int64_t tiles = num_m_tiles * ((g.N + bn - 1) / bn) * groups;
            return (tiles + workers - 1) / workers * (bn + 16);     // waves x (columns + per-tile overhead)
        };
        if (cost(224) < cost(256)) block_n = 224;
    }
    CUtensorMap map_a, map_b;
    if (!make_operand_map(&map_a, g.a, g.M, g.K, g.lda, g.is_fp8, 128) ||
        !make_operand_map(&map_b, g.b, static_cast<int64_t>(g.k_group_off != nullptr ? 1 : g.num_groups) * g.N, g.K, g.ldb, g.is_fp8, block_n))
        return cudaErrorInvalidValue;
    const void* fn = g.is_fp8 ? (block_n == 256 ? (const void*)gemm_kernel<true, 256> : (const void*)gemm_kernel<true, 128>)
                              : (block_n == 256   ? (const void*)gemm_kernel<false, 256>
                                 : block_n == 224 ? (const void*)gemm_kernel<false, 224>
                                                  : (const void*)gemm_kernel<false, 128>);
    const int kGemmSmemBytes = gemm_smem_bytes(block_n, g.is_fp8 != 0);
    cudaError_t err = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes);
    if (err != cudaSuccess) return err;
    if (g.k_group_off != nullptr && (g.is_fp8 || g.fuse != EP_GEMM_FUSE_NONE || g.tile_group != nullptr || g.num_groups < 1)) return cudaErrorInvalidValue;
    const int num_tiles = ((g.M + kBlockM - 1) / kBlockM) * ((g.N + block_n - 1) / block_n) * (g.k_group_off != nullptr ? g.num_groups : 1);
    int ctas = num_sms < 1 ? 1 : num_sms;
    void* params[] = {&map_a, &map_b, const_cast<GemmArgs*>(&g)};
    if (g.fuse != EP_GEMM_FUSE_NONE) {
        // the CTAs of a fused launch wait on one another (grid barrier, copier -> producer flags): cooperative launch
        const int R = g.ctx.num_ranks;
        if (g.is_fp8 || g.M % (kBlockM * R) != 0 || g.N % 128 != 0 || g.tile_group != nullptr) return cudaErrorInvalidValue;
        if (g.fuse == EP_GEMM_FUSE_ALL_GATHER && (g.num_copy_ctas < 1 || g.num_copy_ctas >= ctas)) return cudaErrorInvalidValue;
        if (g.fuse == EP_GEMM_FUSE_REDUCE_SCATTER && g.num_copy_ctas != 0) return cudaErrorInvalidValue;
        if (g.M / kBlockM >= EP_MAX_TILE_FLAGS - 1) return cudaErrorInvalidValue;
        return cudaLaunchCooperativeKernel(fn, dim3(ctas, 1, 1), dim3(kGemmThreads, 1, 1), params, kGemmSmemBytes, stream);
    }
    if (ctas > num_tiles) ctas = num_tiles;
    return cudaLaunchKernel(fn, dim3(ctas, 1, 1), dim3(gemm_threads(g.is_fp8 != 0, block_n), 1, 1), params, kGemmSmemBytes, stream);
}

}  // namespace ep
