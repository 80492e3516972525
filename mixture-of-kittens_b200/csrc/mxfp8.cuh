// MXFP8 block helpers shared by the standalone quantiser, the quantising dispatch and the
// block-scaled GEMM epilogues.  One block = 32 consecutive elements along the contraction axis,
// E4M3 data, one E8M0 scale.  Arithmetic follows csrc/mxfp8.cuh:45-90 of Mixture-of-Kittens:
//   scale = max(amax * 0.002232142857f, 1e-12f);  e = cvt.rp.satfinite.ue8m0(scale)
//   q = cvt.rn.satfinite.e4m3(x * 2^(127 - e));   dequantised value = q * 2^(e - 127)
#pragma once

#include <cuda_fp8.h>

#include "common.cuh"

namespace mok {

// Conversions use the hardware converters (cvt.rp.satfinite.ue8m0x2, cvt.rn.satfinite.e4m3x2, fp8x2 ->
// f16x2): two values per instruction.  An all-integer formulation of the same roundings was measured
// and was slower in every kernel here (the kernels are issue-bound, not converter-bound).
__device__ __forceinline__ uint32_t mx_scale_byte(float amax) {
    const float scale = fmaxf(amax * 0.002232142857f, 0.000000000001f);
    uint16_t sc2;
    asm("cvt.rp.satfinite.ue8m0x2.f32 %0, %1, %2;" : "=h"(sc2) : "f"(scale), "f"(scale));
    return sc2 & 0xFFu;
}
__device__ __forceinline__ float mx_inv_scale(uint32_t scale_byte) {
    return __uint_as_float((254u - scale_byte) << 23);
}
// two floats -> two E4M3 bytes, `lo` in the low byte
__device__ __forceinline__ uint32_t mx_pack2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ uint32_t mx_pack4(float a, float b, float c, float d) {
    return mx_pack2(a, b) | (mx_pack2(c, d) << 16);
}
__device__ __forceinline__ float2 mx_unpack2(uint16_t two_bytes, float scale) {
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(two_bytes), __NV_E4M3);
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
    return make_float2(f.x * scale, f.y * scale);
}
__device__ __forceinline__ float mx_scale_value(uint32_t scale_byte) {
    return __uint_as_float(scale_byte << 23);
}

// 32 bf16 values (16 packed words) -> 32 fp8 bytes (8 words) + the E8M0 scale byte
__device__ __forceinline__ void mx_quantize_block(const uint32_t (&in)[16], uint32_t (&out)[8], uint32_t& scale_byte) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float2 v = unpack_bf16(in[i]);
        amax = fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y)));
    }
    scale_byte = mx_scale_byte(amax);
    const float inv = mx_inv_scale(scale_byte);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float2 a = unpack_bf16(in[2 * i]);
        const float2 b = unpack_bf16(in[2 * i + 1]);
        out[i] = mx_pack4(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
    }
}

// byte offset of the scale of (row r, 32-wide k-block kb) inside the [rows/128, kcols/128, 32, 16]
// scale tensor (tcgen05 block-scale layout; csrc/mxfp8.cuh:184)
__device__ __forceinline__ size_t mx_scale_offset(int r, int kb, int k_tiles) {
    return (static_cast<size_t>(r >> 7) * k_tiles + (kb >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (kb & 3);
}

}  // namespace mok
