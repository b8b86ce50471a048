// Device pieces of the 1x128 FP8 quantisation shared by the plain quantiser and the fused quantise-and-dispatch
// kernel of the expert-parallel exchange. Rounding sequence of the reference's torch oracle
// (aiter/ops/quant.py:64-94): amax -> scale = amax / 448 (IEEE division; 0 -> 1) -> code = RNE_e4m3(x / scale).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace b200 {

// eight 16-bit floats (bf16 or fp16) of one 16-byte load -> fp32
template <bool F16>
__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
    if (F16) {
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    } else {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
}

// 16 consecutive lanes of a warp (an aligned half-warp) hold one 128-element group, 8 elements each. Returns the
// group's scale (on all 16 lanes) and this lane's 8 codes. Must be called by the whole warp (shuffles).
template <bool F16>
__device__ __forceinline__ float quant_group16(const uint4& raw, uint2& codes) {
    float v[8];
    unpack8<F16>(raw, v);
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int d = 8; d >= 1; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    float scale = __fdiv_rn(amax, 448.0f);
    if (scale == 0.f) scale = 1.f;
    uint32_t w[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        float2 lo = make_float2(__fdiv_rn(v[4 * i], scale), __fdiv_rn(v[4 * i + 1], scale));
        float2 hi = make_float2(__fdiv_rn(v[4 * i + 2], scale), __fdiv_rn(v[4 * i + 3], scale));
        uint32_t a = __nv_cvt_float2_to_fp8x2(lo, __NV_SATFINITE, __NV_E4M3);
        uint32_t b = __nv_cvt_float2_to_fp8x2(hi, __NV_SATFINITE, __NV_E4M3);
        w[i] = a | (b << 16);
    }
    codes = make_uint2(w[0], w[1]);
    return scale;
}

}  // namespace b200
