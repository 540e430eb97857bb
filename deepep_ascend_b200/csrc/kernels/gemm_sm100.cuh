// tcgen05 / TMEM / TMA building blocks for the sm_100a GEMM kernels of this library (inline PTX, no CUTLASS
// templates; the descriptor bit layouts follow the PTX ISA "tcgen05" chapter).
//   * shared-memory matrix descriptors for K-major operands written by TMA with the 128-byte swizzle,
//   * the 32-bit instruction descriptor of tcgen05.mma (kind::f16 and kind::f8f6f4, fp32 accumulate),
//   * TMEM allocation, tcgen05.mma / commit / ld / fences,
//   * 2-D tiled TMA loads (never multicast).
#pragma once
#include <cuda.h>
#include <stdint.h>

#include "ptx.cuh"

namespace ep {
namespace umma {

// 64-bit shared-memory matrix descriptor, K-major tile of rows x 128 bytes, 128B swizzle:
//   bits [0,14)  start address >> 4          bits [16,30) leading byte offset >> 4 (unused for swizzled K-major: 1)
//   bits [32,46) stride byte offset >> 4 = 1024 >> 4 (eight rows of 128 bytes form one swizzle atom)
//   bits [46,48) descriptor version = 1 on sm_100   bits [61,64) layout type: 2 = SWIZZLE_128B
__device__ __forceinline__ uint64_t make_smem_desc_sw128(const void* smem_tile) {
    const uint64_t addr = ptx::smem_u32(smem_tile);
    uint64_t desc = 0;
    desc |= (addr & 0x3ffffull) >> 4;
    desc |= 1ull << 16;
    desc |= (1024ull >> 4) << 32;
    desc |= 1ull << 46;
    desc |= 2ull << 61;
    return desc;
}
// advance a K-major SW128 descriptor by `bytes` along K inside the 128-byte swizzle row (bytes < 128)
__device__ __forceinline__ uint64_t advance_desc_k(uint64_t desc, uint32_t bytes) { return desc + (bytes >> 4); }

// 32-bit instruction descriptor: D fp32, A/B K-major, dense.
//   bits [4,6) D format: 1 = F32     bits [7,10) A format     bits [10,13) B format   (kind::f16: 0 F16, 1 BF16;
//   kind::f8f6f4: 0 E4M3, 1 E5M2)    bits [17,23) N >> 3      bits [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_instr_desc(int m, int n, int ab_format) {
    return (1u << 4) | (static_cast<uint32_t>(ab_format) << 7) | (static_cast<uint32_t>(ab_format) << 10) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
constexpr int kFormatBF16 = 1;   // kind::f16
constexpr int kFormatE4M3 = 0;   // kind::f8f6f4

// ------------------------------------------------------------------------------------------------ TMEM
// Allocate `columns` (power of two >= 32) TMEM columns; executed by one whole warp; base address lands in smem.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_u32(smem_result)), "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t tmem_base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(columns) : "memory");
}
__device__ __forceinline__ void fence_before_thread_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_thread_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.  accumulate == 0 overwrites D.
template <bool kFp8>
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    if (kFp8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n" ::"r"(tmem_d), "l"(desc_a),
            "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n" ::"r"(tmem_d), "l"(desc_a),
            "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
            : "memory");
    }
}
// arrive on `bar` (count 1) once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ptx::smem_u32(bar)) : "memory");
}

// 32 lanes x 32 columns of 32-bit TMEM -> 32 registers per thread (thread i of the warp reads lane base+i)
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------------------------------------------ packed fp32 math
// Two fp32 lanes per instruction (fma.rn.f32x2, sm_100): acc.{lo,hi} += x.{lo,hi} * s.{lo,hi}.  The promotion of block-scaled
// accumulators is bound by instruction issue, so halving the FMA count matters.
__device__ __forceinline__ uint64_t pack_f32x2(uint32_t lo, uint32_t hi) {
    uint64_t v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(lo), "r"(hi));
    return v;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
    uint32_t a, b;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(v));
    lo = __uint_as_float(a);
    hi = __uint_as_float(b);
}
__device__ __forceinline__ void fma_f32x2(uint64_t& acc, uint64_t x, uint64_t s) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(x), "l"(s));
}

// ------------------------------------------------------------------------------------------------ TMA
// 2-D tile load, global -> this CTA's shared memory (no multicast).  c0 = innermost coordinate (elements).
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            ptx::smem_u32(smem_dst)),
        "l"(map), "r"(ptx::smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

}  // namespace umma
}  // namespace ep
