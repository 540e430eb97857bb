// Allocation-free entry point (no counterpart in the reference implementation).
//
// Some hosts of this library may not allocate device memory at the moment they need a dispatch: code that runs
// inside a memory pool it does not own, inside a region where the CUDA allocator is locked or being captured, or
// a runtime that has handed all device memory to its own arena up front.  Every other path of the library keeps
// its scratch (barrier counters, per-CTA partial counts, status words) in the symmetric buffer that
// `ElasticBuffer` allocates with cudaMalloc / cudaHostAlloc.  This entry point runs the single-GPU (one rank)
// dispatch with that scratch in a fixed array that is part of the library image instead, and touches no
// allocator at all: not cudaMalloc / cudaFree, not the stream-ordered allocator, not torch's.
//
// Limits (fixed by the size of the built-in array, about 1.2 MB held on every GPU that loads the library until
// the process exits): at most EP_MAX_EXPERTS (1024) experts, EP_MAX_TOPK (16) selections per token,
// EP_MAX_CTAS (160) CTAs and 2^24 - 1 tokens; larger requests are rejected with an error message.
//
// Behaviour to know about:
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress) with that
//     device current; make that first call outside any stream capture;
//   * all calls on a device share the one array; it keeps the previous call's counters, which the protocol
//     tolerates (they are epoch-tagged) and the failure flags are cleared at the start of every call with a
//     stream-ordered memset; two calls that overlap on the GPU (different streams, no ordering) race on it;
//   * the caller owns every input and output buffer; outputs must hold `num_tokens` rows.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// One-rank dispatch: every token with at least one valid expert id is written to the next output row, in token
// order (the same result as ElasticBuffer.dispatch on a group of one rank, non-expand layout).
//   x                [T, H] bf16
//   topk_idx         [T, K] int64, -1 = no selection
//   topk_weights     [T, K] fp32
//   quantize         != 0: rows are cast to e4m3 with one fp32 scale per 128 channels (recv_sf [T, ceil(H/128)])
//   recv_x           [T, H] bf16, or e4m3 when quantize
//   recv_topk_idx    [T, K] int64     recv_topk_weights [T, K] fp32     recv_src_meta [T, 2] int32
//   lane_src, plan   [T, K] int32     psum_rank [1]     psum_expert, recv_per_expert [num_experts] int32
//   stream           cudaStream_t (0 for the default stream)
// Returns 0 on success.  On failure returns non-zero and, if `err` is not null, writes a message of at most
// `err_len` bytes.  The launch is asynchronous: synchronise the stream before reading the outputs.
int ep_dispatch_one_rank_noalloc(const void* x, const void* topk_idx, const float* topk_weights, int num_tokens, int hidden,
                                 int num_topk, int num_experts, int quantize, void* recv_x, float* recv_sf, void* recv_topk_idx,
                                 float* recv_topk_weights, int32_t* recv_src_meta, int32_t* lane_src, int32_t* plan,
                                 int32_t* psum_rank, int32_t* psum_expert, int32_t* recv_per_expert, int num_sms, void* stream,
                                 char* err, int err_len);

#ifdef __cplusplus
}
#endif
