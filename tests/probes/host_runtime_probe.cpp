// Host-only checks of the buffer life-cycle state machine and of the region layout arithmetic.
// Compiled and run by tests/test_host_runtime.py; exits non-zero on the first failed check.
#include <cstdio>
#include <cstdlib>
#include <string>

#include "runtime/coordinator.hpp"
#include "runtime/layout.hpp"

using namespace ep_host;

static int failures = 0;
#define CHECK(cond)                                                          \
    do {                                                                     \
        if (!(cond)) {                                                       \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);    \
            ++failures;                                                      \
        }                                                                    \
    } while (0)

template <typename F>
static bool throws(F f) {
    try {
        f();
    } catch (const std::exception&) {
        return true;
    }
    return false;
}

static void test_coordinator() {
    OperationCoordinator c;
    CHECK(c.usable() && c.generation() == 0);
    const uint64_t g1 = c.begin("dispatch");
    CHECK(g1 == 1 && c.state() == BufferState::Active);
    CHECK(throws([&] { c.begin("combine"); }));          // one operation at a time
    c.complete(g1, true);
    CHECK(c.usable());
    const uint64_t g2 = c.begin("combine");
    CHECK(g2 == 2);                                       // generations strictly increase
    c.complete(g2, false, "device wait timed out");
    CHECK(c.state() == BufferState::Poisoned && c.reason() == "device wait timed out");
    CHECK(throws([&] { c.begin("dispatch"); }));          // a poisoned buffer refuses work
    c.poison("second failure");                           // first reason is kept
    CHECK(c.reason() == "device wait timed out");
    CHECK(c.begin_destroy());                             // ... but can still be destroyed
    c.end_destroy(false);                                 // a failed release leaves it retryable
    CHECK(c.state() == BufferState::Poisoned);
    CHECK(c.begin_destroy());
    c.end_destroy(true);
    CHECK(c.state() == BufferState::Destroyed);
    CHECK(!c.begin_destroy());                            // idempotent
    CHECK(throws([&] { c.begin("barrier"); }));

    // an operation that unwinds without commit() poisons the buffer
    OperationCoordinator d;
    try {
        OperationScope scope(d, "dispatch");
        throw std::runtime_error("validation failed after admission");
    } catch (const std::exception&) {
    }
    CHECK(d.state() == BufferState::Poisoned);
    // a committed scope leaves it idle; a stale completion poisons
    OperationCoordinator e;
    {
        OperationScope scope(e, "dispatch");
        scope.commit();
    }
    CHECK(e.usable());
    e.complete(12345, true);
    CHECK(e.state() == BufferState::Poisoned);
}

static void test_layout() {
    MoeShape s;
    s.num_ranks = 8;
    s.num_max_tokens_per_rank = 8192;
    s.hidden = 7168;
    s.num_topk = 8;
    s.use_fp8_dispatch = true;
    s.num_recv_slots = 2;
    const RegionLayout r = plan_regions(s);
    CHECK(r.capacity_rows == 8 * 8192);
    CHECK(r.x_row_bytes == 7168 && r.sf_cols == 56);
    CHECK(r.tail_bytes % 128 == 0 && r.tail_bytes >= 8 * 12 + 8 && r.sf_row_bytes % 128 == 0 && r.sf_row_bytes >= 56 * 4);
    // regions are ordered, aligned, disjoint and inside the buffer
    int64_t prev_end = EP_WORKSPACE_BYTES;
    for (int i = 0; i < 2; ++i) {
        const int64_t offs[] = {r.slots[i].x, r.slots[i].sf, r.slots[i].idx, r.slots[i].w, r.slots[i].meta, r.slots[i].tail};
        const int64_t sizes[] = {r.capacity_rows * r.x_row_bytes, r.capacity_rows * r.sf_row_bytes, r.capacity_rows * 64, r.capacity_rows * 32,
                                 r.capacity_rows * 8, r.capacity_rows * r.tail_bytes};
        for (int k = 0; k < 6; ++k) {
            CHECK(offs[k] % 1024 == 0 && offs[k] >= prev_end);
            prev_end = offs[k] + sizes[k];
        }
    }
    // two combine input regions (alternate calls), each followed by its weight rows
    CHECK(r.combine_x[0] >= prev_end && r.combine_w[0] >= r.combine_x[0] + r.capacity_rows * 7168 * 2);
    CHECK(r.combine_x[1] >= r.combine_w[0] + r.capacity_rows * 8 * 4 && r.combine_w[1] >= r.combine_x[1] + r.capacity_rows * 7168 * 2);
    CHECK(r.extra >= r.combine_w[1] + r.capacity_rows * 8 * 4 && r.moe_bytes >= r.extra && r.moe_bytes % EP_BUFFER_ALIGNMENT == 0);
    // bf16 buffers are wider, expand buffers hold more rows
    MoeShape b = s;
    b.use_fp8_dispatch = false;
    CHECK(plan_regions(b).x_row_bytes == 2 * 7168 && plan_regions(b).moe_bytes > r.moe_bytes);
    MoeShape x = s;
    x.enable_expand = true;
    x.num_experts_hint = 256;
    x.expert_alignment = 128;
    CHECK(plan_regions(x).capacity_rows >= 8 * 8192 * 8);
    // rejected shapes
    MoeShape bad = s;
    bad.num_ranks = EP_MAX_RANKS + 1;
    CHECK(throws([&] { plan_regions(bad); }));
    bad = s;
    bad.num_topk = EP_MAX_TOPK + 1;
    CHECK(throws([&] { plan_regions(bad); }));
    bad = s;
    bad.num_max_tokens_per_rank = 1 << 22;                 // 8 * 2^22 rows do not fit the 24-bit row field
    CHECK(throws([&] { plan_regions(bad); }));
    CHECK(throws([] { checked_mul(INT64_MAX / 2, 3); }));
    CHECK(throws([] { checked_add(INT64_MAX, 1); }));
    CHECK(align_up(1, 16) == 16 && align_up(32, 16) == 32);
}

int main() {
    test_coordinator();
    test_layout();
    if (failures == 0) std::printf("host runtime probe: all checks passed\n");
    return failures == 0 ? 0 : 1;
}
