// Per-head RMSNorm + RoPE of one 128-value row held by a warp (lane l owns dimensions 4l..4l+3), with the
// reference's arithmetic: five bf16 roundings per element (17.cu:15496-15546), rsqrtf, and its sum-of-squares
// reduction order - a shuffle-down tree inside each 32-thread warp, then (w0 + w2) + (w1 + w3) over the four warp
// sums (17.cu:15107-15196).  Here the 32 values of reference "warp" j sit in lanes 8j..8j+7, and the same pairs
// are added in the same order with xor shuffles (float addition commutes, so a + b from either side is equal).
#pragma once

#include "qm_common.cuh"

__device__ __forceinline__ float reference_order_sum_of_squares(float s0, float s1, float s2, float s3) {
    // Tree inside the 8-lane group holding one reference warp's 32 values.
    s0 += __shfl_xor_sync(0xffffffffu, s0, 4);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 4);
    s2 += __shfl_xor_sync(0xffffffffu, s2, 4);
    s3 += __shfl_xor_sync(0xffffffffu, s3, 4);
    s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    s2 += __shfl_xor_sync(0xffffffffu, s2, 2);
    s3 += __shfl_xor_sync(0xffffffffu, s3, 2);
    s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
    s2 += __shfl_xor_sync(0xffffffffu, s2, 1);
    s3 += __shfl_xor_sync(0xffffffffu, s3, 1);
    s0 = __fadd_rn(s0, s2);
    s1 = __fadd_rn(s1, s3);
    const float warp_sum = __fadd_rn(s0, s1);      // exact in lanes 0, 8, 16, 24
    const float w0 = __shfl_sync(0xffffffffu, warp_sum, 0);
    const float w1 = __shfl_sync(0xffffffffu, warp_sum, 8);
    const float w2 = __shfl_sync(0xffffffffu, warp_sum, 16);
    const float w3 = __shfl_sync(0xffffffffu, warp_sum, 24);
    return __fadd_rn(__fadd_rn(w0, w2), __fadd_rn(w1, w3));
}

// kHardwareRounding: round with cvt.rn.bf16 (one instruction; identical to the reference's integer rounding for
// every finite value and infinity, different NaN payload).  The caller picks the integer path when a row holds a
// non-finite input, so NaN bits also match the reference.
template <bool kHardwareRounding>
__device__ __forceinline__ float rope_round(float v) {
    if (kHardwareRounding) return __bfloat162float(__float2bfloat16_rn(v));
    return round_bf16(v);
}

template <bool kHardwareRounding>
__device__ __forceinline__ uint2 norm_rope_row_impl(const float (&x)[4], const float (&w)[4], const float (&c)[4],
                                                    const float (&s)[4], int lane, float epsilon) {
    const float sum = reference_order_sum_of_squares(__fmul_rn(x[0], x[0]), __fmul_rn(x[1], x[1]),
                                                     __fmul_rn(x[2], x[2]), __fmul_rn(x[3], x[3]));
    // sum / 128 is exact as a multiplication by 2^-7
    const float inverse_rms = rsqrtf(__fadd_rn(__fmul_rn(sum, 1.0f / (float)kHeadDim), epsilon));
    // RMSNorm: normalise in fp32 -> bf16 -> multiply by the bf16 weight -> bf16.
    float n[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
        n[i] = rope_round<kHardwareRounding>(__fmul_rn(rope_round<kHardwareRounding>(__fmul_rn(x[i], inverse_rms)), w[i]));
    // rotate_half: dimension d pairs with d +- 64, which lane l ^ 16 holds.
    float y[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float partner = __shfl_xor_sync(0xffffffffu, n[i], 16);
        if (lane < 16) partner = -partner;
        const float first = rope_round<kHardwareRounding>(__fmul_rn(n[i], c[i]));
        const float second = rope_round<kHardwareRounding>(__fmul_rn(partner, s[i]));
        y[i] = __fadd_rn(first, second);
    }
    if (kHardwareRounding) return make_uint2(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]));
    return make_uint2(f32_to_bf16_bits(y[0]) | (f32_to_bf16_bits(y[1]) << 16),
                      f32_to_bf16_bits(y[2]) | (f32_to_bf16_bits(y[3]) << 16));
}

// One row: raw = 4 packed bf16 of this lane; returns the normed + roped row, packed.
__device__ __forceinline__ uint2 norm_rope_row(uint2 raw, uint2 wraw, const float (&c)[4], const float (&s)[4], int lane,
                                               float epsilon) {
    const float x[4] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y)};
    const float w[4] = {bf16_lo(wraw.x), bf16_hi(wraw.x), bf16_lo(wraw.y), bf16_hi(wraw.y)};
    // exponent all ones <=> inf or NaN, for any of the four inputs of any lane
    const bool odd = ((raw.x & 0x7f80u) == 0x7f80u) || ((raw.x & 0x7f800000u) == 0x7f800000u) ||
                     ((raw.y & 0x7f80u) == 0x7f80u) || ((raw.y & 0x7f800000u) == 0x7f800000u);
    if (__any_sync(0xffffffffu, odd)) return norm_rope_row_impl<false>(x, w, c, s, lane, epsilon);
    return norm_rope_row_impl<true>(x, w, c, s, lane, epsilon);
}
