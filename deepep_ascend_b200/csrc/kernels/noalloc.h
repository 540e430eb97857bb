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
//     tolerates (they are epoch-tagged); the failure flags and every counter that a call which gave up half way
//     could have left non-zero are cleared at the start of every call with stream-ordered memsets; two calls that
//     overlap on the GPU (different streams, no ordering) race on it;
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
//   topk_weights     [T, K] fp32, or null (recv_topk_weights is then left untouched)
//   quantize         != 0: rows are cast to e4m3 with one fp32 scale per 128 channels (recv_sf [T, ceil(H/128)])
//   recv_x           [T, H] bf16, or e4m3 when quantize
//   recv_topk_idx    [T, K] int64     recv_topk_weights [T, K] fp32     recv_src_meta [T, 2] int32
//   lane_src, plan   [T, K] int32     psum_rank [1]     psum_expert, recv_per_expert [num_experts] int32
//   stream           cudaStream_t (0 for the default stream)
// Pointers must be aligned: x and recv_x to 16 bytes, topk_idx / recv_topk_idx / recv_src_meta to 8, all others to 4;
// anything else is rejected here (on the GPU it would fault).
// Returns 0 once the kernel has been LAUNCHED: the work is asynchronous, so synchronise the stream before reading the
// outputs, and ask ep_noalloc_last_status() whether the kernel itself reported a failure.  On a host-side failure
// returns non-zero and, if `err` is not null, writes a message of at most `err_len` bytes.
int ep_dispatch_one_rank_noalloc(const void* x, const void* topk_idx, const float* topk_weights, int num_tokens, int hidden,
                                 int num_topk, int num_experts, int quantize, void* recv_x, float* recv_sf, void* recv_topk_idx,
                                 float* recv_topk_weights, int32_t* recv_src_meta, int32_t* lane_src, int32_t* plan,
                                 int32_t* psum_rank, int32_t* psum_expert, int32_t* recv_per_expert, int num_sms, void* stream,
                                 char* err, int err_len);

// What the last ep_dispatch_one_rank_noalloc kernel on the current device reported, copied out of the built-in array
// (no allocation; waits for `stream`): out = {code, phase, peer, expected, observed, rank}; code 0 = no failure,
// 1 = a bounded wait ran out, 2 = a bounds check failed (see EpError / EpPhase in api.h).  Call it after the dispatch
// on the same stream.  Returns 0 on success, non-zero with a message in `err` otherwise.
int ep_noalloc_last_status(unsigned long long out[6], void* stream, char* err, int err_len);

#ifdef __cplusplus
}
#endif
