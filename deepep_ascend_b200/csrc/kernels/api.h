// Host-visible contract of the CUDA kernels: limits, status words, per-rank context and the argument structs
// of every launcher.  Plain C++ (no torch, no CUDA headers beyond the runtime API) so that host-only unit
// tests can include it.
#pragma once
#include <cuda_runtime_api.h>
#include <stdint.h>

#define EP_MAX_RANKS 8
#define EP_MAX_EXPERTS 1024
#define EP_MAX_TOPK 16
#define EP_MAX_CTAS 160
#define EP_MAX_TILE_FLAGS 16384
#define EP_WORKSPACE_BYTES (4u << 20)
#define EP_BUFFER_ALIGNMENT (2u << 20)
// The last 4 KB of the workspace hold flag words that the HOST addresses directly (stream memory operations written into
// the peers' buffers and waited for in the local one): uint64 [EP_NUM_CHANNELS][EP_MAX_RANKS], [channel][source rank].
#define EP_WS_HOST_FLAGS_BYTES 4096u
#define EP_WS_HOST_FLAGS_OFFSET (EP_WORKSPACE_BYTES - EP_WS_HOST_FLAGS_BYTES)

// One independent sequence of collective calls per channel (own epoch, own barrier counters), so that e.g.
// a low-latency step on one stream never aliases an all-gather session on another.
enum EpChannel {
    EP_CH_DISPATCH = 0,
    EP_CH_COMBINE = 1,
    EP_CH_BARRIER = 2,
    EP_CH_LL_DISPATCH = 3,
    EP_CH_LL_COMBINE = 4,
    EP_CH_AGRS = 5,
    EP_CH_PP = 6,
    EP_CH_ENGRAM = 7,
    EP_CH_GEMM = 8,
    EP_CH_FUSED = 9,
    EP_NUM_CHANNELS = 12
};

// Status block (uint64 words in pinned, device-mapped host memory).
enum EpStatusWord {
    EP_STATUS_CODE = 0,
    EP_STATUS_PHASE = 1,
    EP_STATUS_PEER = 2,
    EP_STATUS_EXPECTED = 3,
    EP_STATUS_OBSERVED = 4,
    EP_STATUS_RANK = 5,
    EP_STATUS_NUM_RECV = 8,        // epoch-tagged: rows received by the last dispatch
    EP_STATUS_NUM_EXPANDED = 9,    // epoch-tagged: rows of the expand layout
    EP_STATUS_EXPERT_BASE = 16,    // epoch-tagged per-local-expert counts follow
    EP_STATUS_WORDS = 16 + EP_MAX_EXPERTS
};

enum EpError { EP_OK = 0, EP_ERR_TIMEOUT = 1, EP_ERR_BOUNDS = 2, EP_ERR_PROTOCOL = 3 };

// Where a wait gave up (EP_STATUS_PHASE).
enum EpPhase {
    EP_PH_GRID_SYNC = 1,
    EP_PH_XGPU_BARRIER = 2,
    EP_PH_COUNT_EXCHANGE = 3,
    EP_PH_DISPATCH_LOAD = 4,
    EP_PH_DISPATCH_DONE = 5,
    EP_PH_COMBINE_ENTRY = 6,
    EP_PH_COMBINE_LOAD = 7,
    EP_PH_COMBINE_EXIT = 8,
    EP_PH_LL_RECV_COUNT = 9,
    EP_PH_LL_COMBINE_FLAG = 10,
    EP_PH_TEST_FLAG = 11,
    EP_PH_PP = 12,
    EP_PH_TILE_FLAG = 13,
    EP_PH_GEMM_PIPE = 14,
    EP_PH_DISPATCH_ASSIGN = 15,
    EP_PH_CTA_COUNTS = 16
};

struct RankCtx {
    int rank;
    int num_ranks;
    uint8_t* peer_base[EP_MAX_RANKS];   // every rank's symmetric buffer as mapped here; [rank] is local
    uint64_t* status;                   // device pointer of this rank's status block
    uint64_t timeout_ns;
};

struct DispatchArgs {
    RankCtx ctx;
    // inputs
    const void* x;                 // [T, H] bf16, or e4m3 when x_is_fp8
    const float* sf;               // [T, H/128] fp32 scales of pre-quantized input, else null
    const void* topk_idx;          // [T, K] int64 or int32
    const float* topk_weights;     // [T, K] or null
    int num_tokens, hidden, num_topk, num_experts;
    int idx_is_64;
    int x_is_fp8;                  // input already e4m3
    int quantize;                  // bf16 in, e4m3 + 1x128 scales out (fused cast)
    int do_expand;
    int expert_alignment;
    int cached;                    // reuse lane_src / plan of an earlier call
    int num_max_tokens;            // per rank; src_token_global_idx = rank * num_max_tokens + t
    // handle tensors (local)
    int32_t* lane_src;             // [T, K]
    int32_t* plan;                 // [T, K]
    int32_t* psum_rank;            // [R]
    int32_t* psum_expert;          // [E_local]
    int32_t* recv_per_expert;      // [E_local]
    int32_t* stats;                // [E_local] cumulative, or null
    // receive regions: byte offsets inside every rank's symmetric buffer
    uint64_t off_recv_x, off_recv_sf, off_recv_idx, off_recv_w, off_recv_meta;
    int64_t sf_stride_row, sf_stride_col;   // element strides of the receiver's scale tensor
    int recv_capacity_rows;
    uint64_t* prof;                // optional [8] phase timestamps (ns), or null: start, counted, exchanged, assigned, CTA 0 done
                                   //     sending | by the last CTA of the rank to finish: all stores drained, peers done, end
    // Bulk side stores (non-expand layout, row-major scales whose row is a multiple of 16 bytes): besides the payload row
    // every destination row gets ONE bulk store of its scales (into recv_sf) and ONE of a tail record
    // {expert ids relative to the receiver | weights | source token, source rank * K + sending lane} built by the sender,
    // so nothing is left for the receiver to rewrite.  Otherwise the small pieces go out as plain peer stores.
    int side_packed;
    int tail_bytes, tail_off_w, tail_off_meta;   // tail record: ids at 0, weights, metadata; multiple of 16 bytes
    int tail_pitch;                              // distance of two rows' tail records at the receiver (>= tail_bytes, multiple of 16)
    uint64_t off_recv_tail;
    int do_zero_padding;           // expand layout: zero the rows (and scales) between an expert's last row and its aligned end
    int tune_warps, tune_stages;   // 0 = automatic; warps per CTA and staging buffers per warp of the fused-cast path
};

struct CombineArgs {
    RankCtx ctx;
    uint64_t off_x;                // combine input rows [rows, H] bf16 inside every rank's symmetric buffer
    uint64_t off_w;                // optional weights to carry back (fp32), 0 when unused
    int w_cols;                    // K (non-expand) or 1 (expand)
    const int32_t* plan;           // [T, K]
    const int32_t* lane_src;       // [T, K]
    const float* mul_weights;      // [T, K] multiply rows by these (weighted reduce), or null
    const void* bias0;             // [T, H] bf16 or null
    const void* bias1;
    void* out;                     // [T, H] bf16
    float* out_w;                  // [T, K] or null
    int num_tokens, hidden, num_topk;
    uint64_t* prof;                // optional [8] phase timestamps (ns) written by CTA 0, or null
};

struct LayoutArgs {
    const void* topk_idx;
    int idx_is_64;
    int num_tokens, num_topk, num_experts, num_ranks;
    int32_t* num_tokens_per_rank;     // [R]
    int32_t* num_tokens_per_expert;   // [E]
    uint8_t* is_token_in_rank;        // [T, R] bool
};

struct QuantArgs {
    const void* x;        // [T, H] bf16
    void* q;              // [T, H] e4m3
    float* sf;            // [T, H/128] fp32 (or packed UE8M0 int32 [T, ceil(H/512)])
    int num_tokens, hidden;
    int round_scale, use_ue8m0;
    int64_t sf_stride_row, sf_stride_col;
};

namespace ep {

struct LaunchShape {
    int num_ctas;
    int num_warps;
    int smem_bytes;
    int num_stages;
};

// Every launcher takes `n` argument structs: n == 1 is the production path (this process drives one GPU);
// n > 1 runs n virtual ranks that all live on the current device as ONE cooperative launch (gridDim.y = n),
// which is how the multi-rank protocol is exercised on a single GPU.
cudaError_t launch_dispatch(const DispatchArgs* args, int n, int num_sms, cudaStream_t stream);
cudaError_t launch_combine(const CombineArgs* args, int n, int num_sms, cudaStream_t stream);
cudaError_t launch_barrier(const RankCtx* ctxs, int n, int channel, cudaStream_t stream);
cudaError_t launch_wait_flag_test(const RankCtx* ctxs, int n, uint64_t expected, cudaStream_t stream);
cudaError_t launch_layout(const LayoutArgs& args, cudaStream_t stream);
cudaError_t launch_quant(const QuantArgs& args, cudaStream_t stream);

LaunchShape dispatch_launch_shape(const DispatchArgs& a, int num_sms);
LaunchShape combine_launch_shape(const CombineArgs& a, int num_sms);

}  // namespace ep

// ------------------------------------------------------------------------------------------------ low latency
enum { EP_LL_SEND = 1, EP_LL_RECV = 2 };

struct LLDispatchArgs {
    RankCtx ctx;
    const void* x;               // [T, H] bf16
    const void* topk_idx;        // [T, K]
    int idx_is_64;
    int num_tokens, hidden, num_topk, num_experts, num_max_tokens;
    int use_fp8, round_scale, use_ue8m0;
    int phases;                  // EP_LL_SEND | EP_LL_RECV
    uint64_t off_slab[2];        // per buffer set: [E_local][R][M] messages inside every rank's symmetric buffer
    int msg_bytes;               // 16-byte header + payload (+ scales), multiple of 16
    void* packed_x;              // [E_local, R*M, H] e4m3 or bf16
    void* packed_sf;             // fp32 [E_local, G, R*M] (column-major per expert) or int32 [E_local, G/4, R*M]
    int32_t* packed_src_info;    // [E_local, R*M]: (lane << 20) | source token
    int64_t* layout_range;       // [E_local, R]: (begin << 32) | count
    int32_t* packed_count;       // [E_local]
    int32_t* stats;              // [E_local] cumulative or null
    int64_t* wait_stats;         // [R] accumulated wait ns per source rank, or null
    int32_t* mask;               // [R] ranks to ignore (shrink mode) or null
    int shrink;                  // a source that never arrives is masked instead of poisoning the buffer
    uint64_t* prof;              // [8] phase timestamps (ns) or null: start, sends issued, sends complete, counts published
                                 //     (by the last CTA), first counts received, packed, end
};

struct LLCombineArgs {
    RankCtx ctx;
    const void* x;               // [E_local, R*M, H] bf16
    const void* topk_idx;        // [T, K]
    int idx_is_64;
    const float* topk_weights;   // [T, K]
    const int32_t* src_info;     // [E_local, R*M]
    const int64_t* layout_range; // [E_local, R]
    int num_tokens, hidden, num_topk, num_experts, num_max_tokens;
    int phases;
    uint64_t off_slab[2];        // per buffer set: [M * K][H] bf16 rows inside every rank's symmetric buffer
    void* out;                   // [T, H] bf16
    int64_t* wait_stats;
    int32_t* mask;
    int shrink;
    int use_logfmt;              // rows cross the wire as 10-bit logarithmic codes with one range per 128 channels (logfmt.cuh)
    uint64_t* prof;              // [8] phase timestamps (ns) or null: start, stores issued, stores complete, flags published
                                 //     (by the last CTA), flags received, reduced
};

namespace ep {
cudaError_t launch_ll_dispatch(const LLDispatchArgs* args, int n, int num_sms, cudaStream_t stream);
cudaError_t launch_ll_combine(const LLCombineArgs* args, int n, int num_sms, cudaStream_t stream);
}  // namespace ep

// ------------------------------------------------------------------------------------------------ Engram fetch
struct EngramFetchArgs {
    RankCtx ctx;
    const int32_t* indices;      // [num_fetches] global entry ids; owner rank = id / entries_per_rank
    int num_fetches;
    int entries_per_rank;
    int entry_bytes;             // multiple of 16
    const uint8_t* storage[EP_MAX_RANKS];   // every rank's table as seen from this GPU: a region of the peer's symmetric
                                 //     buffer, or the peer's CPU segment (pinned host memory mapped into this GPU)
    void* out;                   // [num_fetches, entry_bytes]
    // scale factors of quantised tables: a table replicated on every rank, gathered locally with the fetch
    const int32_t* sf_table;     // [num_ranks * entries_per_rank, sf_packs] 4-byte packs (fp32 or four UE8M0), or null
    int32_t* fetched_sf;         // pack p of fetch i (token i / per_token, entry i % per_token) goes to
    int sf_packs;                //     fetched_sf[token * sf_token_stride + (entry * sf_packs + p) * sf_pack_stride]
    int entries_per_token;
    int64_t sf_token_stride, sf_pack_stride;
};

// ------------------------------------------------------------------------------------------------ local reduce
struct ReduceSlotsArgs {
    const void* slots;           // [num_slots, n] bf16 / fp32
    void* out;                   // [n]
    int64_t n;
    int num_slots;
    int is_bf16;
};

namespace ep {
cudaError_t launch_engram_fetch(const EngramFetchArgs* args, int n, int num_sms, cudaStream_t stream);
cudaError_t launch_reduce_slots(const ReduceSlotsArgs& args, cudaStream_t stream);
}  // namespace ep

// ------------------------------------------------------------------------------------------------ tcgen05 GEMM
// C[M, N] (bf16) = A[M, K] * B[g][N, K]^T, both operands K-major.  bf16 inputs, or e4m3 inputs with fp32 block
// scales (A: one per row and 128 channels; B: one per 128 x 128 block).  With `tile_group` the M dimension is
// a concatenation of 128-row tiles, each using the weights of one group (expert); -1 skips a tile.
struct GemmArgs {
    const void* a;
    const void* b;
    void* c;
    int M, N, K;
    int num_groups;
    int is_fp8;
    int64_t lda, ldb, ldc;            // row strides in elements
    const float* sfa;                 // fp8: scale of (row, k block) at sfa[row * sfa_stride_row + kb * sfa_stride_kb]
    int64_t sfa_stride_row, sfa_stride_kb;
    const float* sfb;                 // fp8: [num_groups, ceil(N/128), ceil(K/128)] contiguous
    const int32_t* tile_group;        // [ceil(M/128)] or null (single group 0)
    int* error;                       // device int set to non-zero if a pipeline wait ran out
    uint64_t* status;                 // status block of a communication buffer that should hear about such a failure, or null
    int status_rank;
    uint64_t timeout_ns;              // limit of every pipeline wait; 0 = 4 s
    // fused collectives (null / 0 when unused)
    const uint64_t* a_ready_flags;    // all-gather fused into the loads: rows of M tile t may be read once
    uint64_t a_ready_value;           //   a_ready_flags[a_flag_of_tile[t]] >= a_ready_value
    const int32_t* a_flag_of_tile;
    // one-kernel fusion with a collective over peer memory (EP_GEMM_FUSE_*); needs a cooperative launch
    int fuse;
    RankCtx ctx;
    int num_copy_ctas;                // AG: CTAs (at the end of the grid) that pull the remote shards over NVLink
    uint64_t off_full;                // AG: gathered A [M, K] inside every rank's symmetric buffer; rank r owns rows
                                      //     [r * M / R, (r + 1) * M / R) and writes its shard there before the call
    uint64_t off_slots;               // RS: two sets of [R][M / R][N] bf16 partial results inside every rank's buffer
    uint64_t slot_set_bytes;
    void* rs_out;                     // RS: [M / R, N] bf16
    int m_tile_offset;                // M tiles are visited starting from this one (local shard first)
    // K-grouped product (weight gradients of a grouped layer): C[e][M, N] = A[:, k0:k1] * B[:, k0:k1]^T with
    // k0 = k_group_off[e], k1 = k_group_off[e + 1] (device array of num_groups + 1 multiples of 64); C is
    // [num_groups * M, N]; an empty range gives zeros.  bf16 only; null when unused.
    const int32_t* k_group_off;
};
enum { EP_GEMM_FUSE_NONE = 0, EP_GEMM_FUSE_ALL_GATHER = 1, EP_GEMM_FUSE_REDUCE_SCATTER = 2 };

namespace ep {
cudaError_t launch_gemm(const GemmArgs& args, int num_sms, cudaStream_t stream);
}  // namespace ep

// ------------------------------------------------------------------------------------------------ MoE helpers
// h [rows, 2 * I] bf16 (gate | up) -> act = silu(gate) * up, cast to e4m3 with one fp32 scale per (row, 128 channels)
struct SwigluQuantArgs {
    const void* h;          // [rows, 2 * inter] bf16, row stride ldh elements
    int64_t ldh;
    void* q;                // [rows, inter] e4m3
    float* sf;              // scale of (row, block) at sf[row * sf_stride_row + blk * sf_stride_col]
    int64_t sf_stride_row, sf_stride_col;
    void* act_bf16;         // optional [rows, inter] bf16 copy of the activation (kept for the backward pass), or null
    int rows, inter;
};

// Element-wise kernels of the MoE backward pass.  Each also writes the TRANSPOSE of its result ([channels, rows]),
// which is the K-major operand layout the weight-gradient GEMM needs (K = rows), so no separate transpose pass runs.
// `valid` (one byte per row, 0 = alignment padding row) zeroes the results of padding rows.  rows % 64 == 0.
enum { EP_MOE_BWD_PREP = 0, EP_MOE_BWD_SWIGLU = 1, EP_MOE_BWD_DEQUANT_T = 2 };
struct MoeBwdArgs {
    int op;
    int rows, cols;               // PREP / DEQUANT_T: cols = hidden; SWIGLU: cols = intermediate size I
    const uint8_t* valid;         // [rows]
    // PREP: g [rows, H] bf16 (gradient of the combined output at every expert row), y [rows, H] bf16 (the expert
    //       outputs), w [rows] fp32 -> out = g * w [rows, H], out_t = out^T [H, rows], row_dot[b * rows + row] = sum(g * y) over
//       the columns of column block b (moe_bwd_prep_col_blocks of them; the caller adds them up)
    //       (y, out and row_dot may each be null: that piece is then skipped)
    // SWIGLU: g = d_act [rows, I], y = h [rows, 2I] (gate | up) -> out = d_h [rows, 2I], out_t = d_h^T [2I, rows],
    //       out2_t = (silu(gate) * up)^T [I, rows]; optional w [rows]: d_act is multiplied by w[row] first, and
    //       optional row_dot[b * rows + row] = sum over the 64 columns of block b of d_act * activation (before w)
    // DEQUANT_T: y = q [rows, H] e4m3, w = scales (row, 128-block) at w[row * sf_stride_row + blk * sf_stride_col]
    //       -> out_t = (q * scale)^T [H, rows] bf16
    const void* g;
    const void* y;
    const float* w;
    int64_t sf_stride_row, sf_stride_col;
    void* out;
    void* out_t;
    void* out2_t;
    float* row_dot;
};

// Bookkeeping of the expand layout for a grouped GEMM (see expert_segments_kernel).  The start of a segment is a tile
// boundary (alignment % 128 == 0), so a tile belongs to one segment and holds a token iff its first row does.
struct ExpertSegmentsArgs {
    const int32_t* psum_ends;     // [num_groups] inclusive ends of the segments' token rows
    int num_groups, num_rows, alignment;
    int32_t* tile_group;          // [ceil(num_rows / 128)] or null
    uint8_t* valid_row;           // [num_rows] or null
    int32_t* seg_off;             // [num_groups + 1] or null
};

// Local expansion of a (token, rank) layout into the (token, expert) layout of a grouped GEMM, and its inverse.  A
// non-expand dispatch delivers every token once per rank together with the ids of the local experts it selected
// (recv_idx [rows, K], -1 elsewhere).  PLAN numbers the (row, k) pairs of every local expert in row order inside that
// expert's 128-aligned segment; COPY writes each received row to its expert rows; REDUCE adds the expert rows of a received
// row (optionally weighted) back into one row.  What crosses NVLink is then one row per (token, rank) instead of one per
// (token, expert).
struct LocalExpandPlanArgs {
    const void* recv_idx;             // [rows, K] int64 / int32, row pitch idx_pitch elements
    int idx_is_64;
    int64_t idx_pitch;
    int num_rows, num_topk, num_local_experts;
    const int32_t* seg_end_aligned;   // [El] inclusive prefix sums of the 128-aligned expert counts (segment e starts at [e - 1])
    int32_t* pos;                     // [rows, K] expert row of (row, k); the caller fills it with -1 first
    int32_t* seg_end;                 // [El] out: end of the token rows of every segment (start + count)
    int num_ctas;                     // CTAs of the two launches (8 warps each)
    int32_t* warp_counts;             // scratch [num_ctas * 8, El]
    int32_t* cta_counts;              // scratch [num_ctas, El]
};
struct LocalExpandCopyArgs {
    const int32_t* pos;               // [rows, K]
    int num_rows, num_topk;
    const void* src;                  // [rows] rows of row_bytes (multiple of 16), pitch src_pitch bytes
    int64_t src_pitch;
    int row_bytes;
    void* dst;                        // [expert rows, row_bytes] contiguous
    const float* sf_src;              // optional scales [rows, sf_cols], element strides sf_stride_row / sf_stride_col
    int64_t sf_stride_row, sf_stride_col;
    int sf_cols;
    float* sf_dst;                    // [expert rows, sf_cols] contiguous
    const float* w_src;               // optional weights [rows, K], row pitch w_pitch elements
    int64_t w_pitch;
    float* w_dst;                     // [expert rows]
};
struct LocalReduceArgs {
    const int32_t* pos;               // [rows, K]
    int num_rows, num_topk;
    const void* src;                  // [expert rows, cols] bf16 contiguous
    int cols;                         // multiple of 8
    const float* w;                   // optional weight of every expert row [expert rows]; null: plain sum
    void* dst;                        // [rows, cols] bf16 contiguous; rows without an expert row get zeros
};

namespace ep {
cudaError_t launch_local_expand_plan(const LocalExpandPlanArgs& args, cudaStream_t stream);
cudaError_t launch_local_expand_copy(const LocalExpandCopyArgs& args, cudaStream_t stream);
cudaError_t launch_local_reduce(const LocalReduceArgs& args, cudaStream_t stream);
cudaError_t launch_expert_segments(const ExpertSegmentsArgs& args, cudaStream_t stream);
cudaError_t launch_swiglu_quant(const SwigluQuantArgs& args, cudaStream_t stream);
cudaError_t launch_moe_bwd(const MoeBwdArgs& args, cudaStream_t stream);
int moe_bwd_prep_col_blocks(int cols);   // PREP writes row_dot as [col_blocks, rows] partial sums
}  // namespace ep
