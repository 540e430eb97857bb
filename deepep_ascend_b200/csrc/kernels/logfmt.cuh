// LogFMT-10: a 10-bit logarithmic code (1 sign bit + 9 magnitude bits) for bf16 rows, used by the low-latency combine to
// put 36 % fewer bytes on the wire.  Every group of 128 channels carries its own range: the largest and the smallest
// non-zero magnitude of the group (two bf16 values); magnitudes are coded as equal steps of log2 between the two.
//
//   code 0            : zero
//   code m in 1..511  : 2 ^ (lo + (m - 1) * step),  lo = max(log2(amin), log2(amax) - 32),  step = (log2(amax) - lo) / 510
//
// Row layout: [ groups x 160 B of codes | groups x 4 B {amax, amin} ], i.e. hidden * 10 / 8 + hidden / 32 bytes.
// A lane handles 16 consecutive channels (20 bytes of codes, five 32-bit words); eight lanes share a group.
// Parity: the role of logfmt_encode / decode_and_accumulate in csrc/kernels/legacy/internode_ll.cu:556-712 of the
// reference (same bit budget; this layout is fixed-size and codes every group).
#pragma once
#include "ptx.cuh"

namespace ep {
namespace logfmt {

constexpr int kGroup = 128;            // channels per range
constexpr int kLaneChannels = 16;      // channels per lane and step
constexpr int kStepChannels = 512;     // channels per warp step
constexpr int kCodeBytesPerGroup = 160;
constexpr float kMaxOctaves = 32.f;

__host__ __device__ inline int row_bytes(int hidden) { return hidden / kGroup * (kCodeBytesPerGroup + 4); }
// bytes one coded row puts on the wire: rounded up to the 16-byte granularity of bulk copies
__host__ __device__ inline int wire_bytes(int hidden) { return (row_bytes(hidden) + 15) / 16 * 16; }
__host__ __device__ inline int code_bytes(int hidden) { return hidden / kGroup * kCodeBytesPerGroup; }

struct Range {
    float lo, step, inv_step;
};

// the coding range of a group from its two bf16 header values (the same arithmetic on both sides of the wire)
__device__ __forceinline__ Range make_range(float amax, float amin) {
    Range r;
    const float hi = __log2f(amax);
    r.lo = fmaxf(__log2f(amin), hi - kMaxOctaves);
    r.step = (hi - r.lo) * (1.f / 510.f);
    r.inv_step = r.step > 0.f ? 1.f / r.step : 0.f;
    return r;
}

__device__ __forceinline__ uint32_t encode_one(float v, const Range& r) {
    const float mag = fabsf(v);
    if (mag == 0.f) return 0u;
    const float pos = (__log2f(mag) - r.lo) * r.inv_step;
    uint32_t m = static_cast<uint32_t>(__float2int_rn(fminf(fmaxf(pos, 0.f), 510.f))) + 1u;
    return m | (v < 0.f ? 512u : 0u);
}

__device__ __forceinline__ float decode_one(uint32_t code, const Range& r) {
    const uint32_t m = code & 511u;
    if (m == 0u) return 0.f;
    const float mag = exp2f(fmaf(static_cast<float>(m - 1u), r.step, r.lo));
    return (code & 512u) ? -mag : mag;
}

// 16 codes of 10 bits -> five 32-bit words (code i occupies bits [10 i, 10 i + 10))
__device__ __forceinline__ void pack16(const uint32_t (&c)[16], uint32_t (&w)[5]) {
    uint64_t acc = 0;
    int bits = 0, wi = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        acc |= static_cast<uint64_t>(c[i]) << bits;
        bits += 10;
        if (bits >= 32) {
            w[wi++] = static_cast<uint32_t>(acc);
            acc >>= 32;
            bits -= 32;
        }
    }
}

__device__ __forceinline__ void unpack16(const uint32_t (&w)[5], uint32_t (&c)[16]) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int bit = 10 * i, word = bit >> 5, shift = bit & 31;
        uint32_t v = w[word] >> shift;
        if (shift > 22) v |= w[word + 1] << (32 - shift);
        c[i] = v & 1023u;
    }
}

// Encode one bf16 row of `hidden` channels (a multiple of 128) IN PLACE in shared memory: on return the first
// row_bytes(hidden) bytes of `row` hold the coded row.  `hdr` is a per-warp scratch of hidden / 128 words.  Called by
// all lanes of one warp.  Codes are written from the front, behind the channels already read, so nothing unread is lost.
__device__ __forceinline__ void encode_row_in_place(uint8_t* row, uint32_t* hdr, int hidden) {
    const int lane = ptx::lane_id();
    const int groups = hidden / kGroup;
    for (int base = 0; base < hidden; base += kStepChannels) {
        const int ch = base + lane * kLaneChannels;
        const bool in_row = ch < hidden;
        float v[16];
        if (in_row) {
            const int4 a = *reinterpret_cast<const int4*>(row + ch * 2), b = *reinterpret_cast<const int4*>(row + ch * 2 + 16);
            const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
            const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 fa = __bfloat1622float2(ha[j]), fb = __bfloat1622float2(hb[j]);
                v[2 * j] = fa.x, v[2 * j + 1] = fa.y, v[8 + 2 * j] = fb.x, v[8 + 2 * j + 1] = fb.y;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
        float amax = 0.f, amin = __int_as_float(0x7f800000);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float m = fabsf(v[j]);
            amax = fmaxf(amax, m);
            if (m > 0.f) amin = fminf(amin, m);
        }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {   // the eight lanes of a group
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            amin = fminf(amin, __shfl_xor_sync(0xffffffffu, amin, o));
        }
        if (amax == 0.f) amin = 0.f;
        __syncwarp();   // every lane has read its channels of this step
        if (in_row) {
            const Range r = make_range(amax, amin);
            uint32_t c[16], w[5];
#pragma unroll
            for (int j = 0; j < 16; ++j) c[j] = amax == 0.f ? 0u : encode_one(v[j], r);
            pack16(c, w);
            uint32_t* out = reinterpret_cast<uint32_t*>(row + (ch / kLaneChannels) * 20);
#pragma unroll
            for (int j = 0; j < 5; ++j) out[j] = w[j];
            if ((lane & 7) == 0) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(amax, amin);   // exact: both are bf16 values already
                hdr[ch / kGroup] = *reinterpret_cast<const uint32_t*>(&h);
            }
        }
        __syncwarp();
    }
    for (int g = lane; g < groups; g += 32) reinterpret_cast<uint32_t*>(row + groups * kCodeBytesPerGroup)[g] = hdr[g];
    __syncwarp();
}

}  // namespace logfmt
}  // namespace ep
