// Overflow-checked placement of every region inside a symmetric buffer.  All ranks compute the same offsets
// from the same arguments, which is what lets a sender address a peer's tensors directly.
//
//   [ workspace | recv slot 0 | recv slot 1 | ... | combine input 0 | combine input 1 | extra (AG/RS, PP, Engram, LL) ]
//
// A recv slot holds the final output tensors of one dispatch: x rows, scales, localised expert ids, weights
// and per-row source metadata.  There are two combine input regions, used alternately: peers may still be pulling
// from the one of call n while the rows of call n + 1 are written, and the entry barrier of call n + 1 (which no
// rank passes before all ranks have finished call n) is what frees the region of call n, so combine needs no exit
// barrier.  Plain C++17, host-testable.
// Parity: the sizing rules of csrc/elastic/buffer.hpp:588-688 and the checked layout of the reference's NPU
// backend (csrc/backends/ascend/elastic/layout.hpp:218-299).
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>

#include "../kernels/api.h"

namespace ep_host {

inline int64_t checked_mul(int64_t a, int64_t b) {
    if (a < 0 || b < 0) throw std::overflow_error("negative size");
    if (a != 0 && b > INT64_MAX / a) throw std::overflow_error("buffer size overflows int64");
    return a * b;
}
inline int64_t checked_add(int64_t a, int64_t b) {
    if (a < 0 || b < 0 || a > INT64_MAX - b) throw std::overflow_error("buffer size overflows int64");
    return a + b;
}
inline int64_t align_up(int64_t x, int64_t a) { return checked_add(x, a - 1) / a * a; }

struct MoeShape {
    int num_ranks = 1;
    int num_max_tokens_per_rank = 0;
    int hidden = 0;
    int num_topk = 0;
    int num_experts_hint = 0;     // only needed to bound the expand layout
    int expert_alignment = 1;
    bool use_fp8_dispatch = false;
    bool enable_expand = false;
    int num_recv_slots = 2;
};

struct RecvSlot {
    int64_t x = 0, sf = 0, idx = 0, w = 0, meta = 0;
    int64_t tail = 0;   // per-row tail records {local expert ids | weights | source metadata} of the bulk side stores
};

struct RegionLayout {
    int64_t capacity_rows = 0;     // rows a rank can receive in one dispatch
    int64_t x_row_bytes = 0;       // widest row dispatch may write (bf16 unless fp8-only)
    int64_t sf_cols = 0;
    int64_t tail_bytes = 0;        // bytes reserved per tail record (multiple of 128)
    int64_t sf_row_bytes = 0;      // bytes reserved per scale row (multiple of 128)
    int num_recv_slots = 0;
    RecvSlot slots[4];
    int64_t combine_x[2] = {0, 0}, combine_w[2] = {0, 0};
    int64_t extra = 0;             // first byte after the MoE regions
    int64_t moe_bytes = 0;         // workspace + MoE regions, aligned to EP_BUFFER_ALIGNMENT
};

inline int64_t recv_capacity_rows(const MoeShape& s) {
    int64_t rows = checked_mul(s.num_ranks, s.num_max_tokens_per_rank);
    if (s.enable_expand) {
        const int per_rank = s.num_experts_hint > 0 ? s.num_experts_hint / s.num_ranks : s.num_topk;
        const int hits = s.num_topk < per_rank ? s.num_topk : per_rank;
        rows = checked_add(checked_mul(rows, hits > 0 ? hits : 1),
                           checked_mul(per_rank > 0 ? per_rank : 1, s.expert_alignment > 1 ? s.expert_alignment : 0));
    }
    if (rows >= (1 << 24)) throw std::overflow_error("more than 2^24 receive rows per rank");
    return align_up(rows > 0 ? rows : 1, 4);
}

inline RegionLayout plan_regions(const MoeShape& s) {
    if (s.num_ranks < 1 || s.num_ranks > EP_MAX_RANKS) throw std::invalid_argument("unsupported number of ranks");
    if (s.num_recv_slots < 1 || s.num_recv_slots > 4) throw std::invalid_argument("num_recv_slots must be 1..4");
    if (s.num_topk > EP_MAX_TOPK) throw std::invalid_argument("num_topk too large");
    RegionLayout r;
    r.capacity_rows = recv_capacity_rows(s);
    r.x_row_bytes = s.use_fp8_dispatch ? s.hidden : checked_mul(s.hidden, 2);
    r.sf_cols = (s.hidden + 127) / 128;
    // room for the line-aligned variant of the side stores: scale rows and tail records padded to 128-byte multiples
    r.tail_bytes = align_up(static_cast<int64_t>(s.num_topk) * 12 + 8, 128);
    r.sf_row_bytes = align_up(r.sf_cols * 4, 128);
    r.num_recv_slots = s.num_recv_slots;
    const int64_t A = 1024;
    int64_t off = EP_WORKSPACE_BYTES;
    for (int i = 0; i < s.num_recv_slots; ++i) {
        r.slots[i].x = off;    off = align_up(checked_add(off, checked_mul(r.capacity_rows, r.x_row_bytes)), A);
        r.slots[i].sf = off;   off = align_up(checked_add(off, checked_mul(r.capacity_rows, r.sf_row_bytes)), A);
        r.slots[i].idx = off;  off = align_up(checked_add(off, checked_mul(r.capacity_rows, s.num_topk * 8)), A);
        r.slots[i].w = off;    off = align_up(checked_add(off, checked_mul(r.capacity_rows, s.num_topk * 4)), A);
        r.slots[i].meta = off; off = align_up(checked_add(off, checked_mul(r.capacity_rows, 8)), A);
        r.slots[i].tail = off; off = align_up(checked_add(off, checked_mul(r.capacity_rows, r.tail_bytes)), A);
    }
    for (int i = 0; i < 2; ++i) {
        r.combine_x[i] = off; off = align_up(checked_add(off, checked_mul(r.capacity_rows, checked_mul(s.hidden, 2))), A);
        r.combine_w[i] = off; off = align_up(checked_add(off, checked_mul(r.capacity_rows, s.num_topk * 4)), A);
    }
    r.extra = off;
    r.moe_bytes = align_up(off, EP_BUFFER_ALIGNMENT);
    return r;
}

}  // namespace ep_host
