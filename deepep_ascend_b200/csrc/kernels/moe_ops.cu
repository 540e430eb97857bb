// Element-wise pieces of the MoE expert FFN that sit between the two grouped GEMMs: SwiGLU fused with the
// e4m3 (1x128 scales) cast of the second GEMM's input, so the activation is written once in FP8 instead of being
// written in bf16 and re-read by a separate quantisation kernel.
#include "common.cuh"

namespace ep {

namespace {

// one warp per row; each step covers 256 channels (two 128-channel scale groups)
__global__ void swiglu_quant_kernel(const SwigluQuantArgs a) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= a.rows) return;
    const int I = a.inter;
    const uint8_t* gate = reinterpret_cast<const uint8_t*>(a.h) + static_cast<int64_t>(row) * a.ldh * 2;
    const uint8_t* up = gate + static_cast<int64_t>(I) * 2;
    uint8_t* q = reinterpret_cast<uint8_t*>(a.q) + static_cast<int64_t>(row) * I;
    const int iters = (I + 255) / 256;
    for (int i = 0; i < iters; ++i) {
        const int elem = (i * 32 + lane) * 8;
        const bool in_range = elem < I;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.f;
        if (in_range) {
            const int4 graw = ptx::ld_nc_v4(gate + elem * 2), uraw = ptx::ld_nc_v4(up + elem * 2);
            const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&graw);
            const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uraw);
            int4 act_raw;
            __nv_bfloat162* ah = reinterpret_cast<__nv_bfloat162*>(&act_raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 gf = __bfloat1622float2(gh[j]), uf = __bfloat1622float2(uh[j]);
                const float a0 = gf.x / (1.f + __expf(-gf.x)) * uf.x, a1 = gf.y / (1.f + __expf(-gf.y)) * uf.y;
                // the activation is rounded to bf16 first so that the FP8 cast sees the same values as a bf16 pipeline
                ah[j] = __floats2bfloat162_rn(a0, a1);
                const float2 r = __bfloat1622float2(ah[j]);
                v[2 * j] = r.x;
                v[2 * j + 1] = r.y;
            }
            if (a.act_bf16 != nullptr)
                *reinterpret_cast<int4*>(reinterpret_cast<uint8_t*>(a.act_bf16) + (static_cast<int64_t>(row) * I + elem) * 2) = act_raw;
        }
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
        amax = fmaxf(ptx::warp_max_16(amax), 1e-4f);
        const float scale = __fmul_rn(448.f, __frcp_rn(amax));
        if (in_range) {
            uint32_t packed[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j] * scale, v[4 * j + 1] * scale), __NV_SATFINITE, __NV_E4M3);
                const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j + 2] * scale, v[4 * j + 3] * scale), __NV_SATFINITE, __NV_E4M3);
                packed[j] = lo | (hi << 16);
            }
            *reinterpret_cast<uint2*>(q + elem) = make_uint2(packed[0], packed[1]);
            if ((lane & 15) == 0) a.sf[static_cast<int64_t>(row) * a.sf_stride_row + (elem / 128) * a.sf_stride_col] = __fdiv_rn(amax, 448.f);
        }
    }
}

}  // namespace

cudaError_t launch_swiglu_quant(const SwigluQuantArgs& a, cudaStream_t stream) {
    if (a.rows == 0) return cudaSuccess;
    const int warps = 8;
    swiglu_quant_kernel<<<(a.rows + warps - 1) / warps, warps * 32, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace ep
