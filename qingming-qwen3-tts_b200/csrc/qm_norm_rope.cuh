// Per-head RMSNorm + RoPE of one 128-value row held by a warp (lane l owns dimensions 4l..4l+3), with the
// reference's arithmetic: five bf16 roundings per element (17.cu:15496-15546), rsqrtf, and its sum-of-squares
// reduction order - a shuffle-down tree inside each 32-thread warp, then (w0 + w2) + (w1 + w3) over the four warp
// sums (17.cu:15107-15196).  Here the 32 values of reference "warp" j sit in lanes 8j..8j+7, and the same pairs
// are added in the same order with xor shuffles (float addition commutes, so a + b from either side is equal).
#pragma once

#include <math_constants.h>

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
    // Every lane of 8-lane group j now holds w_j, the sum of reference warp j: the butterflies above add the same
    // pairs in every lane, only with the operands of some additions swapped.  (w0 + w2) + (w1 + w3) likewise:
    // xor 16 pairs group j with j ^ 2, xor 8 then pairs the two partial sums.
    const float warp_sum = __fadd_rn(s0, s1);
    const float pair_sum = __fadd_rn(warp_sum, __shfl_xor_sync(0xffffffffu, warp_sum, 16));
    return __fadd_rn(pair_sum, __shfl_xor_sync(0xffffffffu, pair_sum, 8));
}

// The rest of a row once its sum of squares is known, integer rounding throughout (any input): the reference's
// arithmetic spelled out value by value.
__device__ __forceinline__ uint2 norm_rope_row_exact(const float (&x)[4], const float (&w)[4], const float (&c)[4],
                                                     const float (&s)[4], int lane, float inverse_rms) {
    float n[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) n[i] = round_bf16(__fmul_rn(round_bf16(__fmul_rn(x[i], inverse_rms)), w[i]));
    float y[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // rotate_half: dimension d pairs with d +- 64, which lane l ^ 16 holds.
        float partner = __shfl_xor_sync(0xffffffffu, n[i], 16);
        if (lane < 16) partner = -partner;
        const float first = round_bf16(__fmul_rn(n[i], c[i]));
        const float second = round_bf16(__fmul_rn(partner, s[i]));
        y[i] = __fadd_rn(first, second);
    }
    return make_uint2(f32_to_bf16_bits(y[0]) | (f32_to_bf16_bits(y[1]) << 16),
                      f32_to_bf16_bits(y[2]) | (f32_to_bf16_bits(y[3]) << 16));
}

// The same for rows whose values are all finite, two values per instruction: cvt.rn.bf16x2 rounds a pair (equal
// to the integer rounding for every finite value), the partner values travel as two packed words instead of four
// floats, and the sign of rotate_half is folded into the sine ((-a) * b and a * (-b) are the same bits).
__device__ __forceinline__ uint2 norm_rope_row_packed(const float (&x)[4], const float (&w)[4], const float (&c)[4],
                                                      const float (&s)[4], int lane, float inverse_rms) {
    const uint32_t a01 = pack_bf16x2(__fmul_rn(x[0], inverse_rms), __fmul_rn(x[1], inverse_rms));
    const uint32_t a23 = pack_bf16x2(__fmul_rn(x[2], inverse_rms), __fmul_rn(x[3], inverse_rms));
    const uint32_t n01 = pack_bf16x2(__fmul_rn(bf16_lo(a01), w[0]), __fmul_rn(bf16_hi(a01), w[1]));
    const uint32_t n23 = pack_bf16x2(__fmul_rn(bf16_lo(a23), w[2]), __fmul_rn(bf16_hi(a23), w[3]));
    const uint32_t p01 = __shfl_xor_sync(0xffffffffu, n01, 16);
    const uint32_t p23 = __shfl_xor_sync(0xffffffffu, n23, 16);
    const bool low_half = lane < 16;
    const float s0 = low_half ? -s[0] : s[0], s1 = low_half ? -s[1] : s[1];
    const float s2 = low_half ? -s[2] : s[2], s3 = low_half ? -s[3] : s[3];
    const uint32_t f01 = pack_bf16x2(__fmul_rn(bf16_lo(n01), c[0]), __fmul_rn(bf16_hi(n01), c[1]));
    const uint32_t f23 = pack_bf16x2(__fmul_rn(bf16_lo(n23), c[2]), __fmul_rn(bf16_hi(n23), c[3]));
    const uint32_t g01 = pack_bf16x2(__fmul_rn(bf16_lo(p01), s0), __fmul_rn(bf16_hi(p01), s1));
    const uint32_t g23 = pack_bf16x2(__fmul_rn(bf16_lo(p23), s2), __fmul_rn(bf16_hi(p23), s3));
    return make_uint2(pack_bf16x2(__fadd_rn(bf16_lo(f01), bf16_lo(g01)), __fadd_rn(bf16_hi(f01), bf16_hi(g01))),
                      pack_bf16x2(__fadd_rn(bf16_lo(f23), bf16_lo(g23)), __fadd_rn(bf16_hi(f23), bf16_hi(g23))));
}

// One row: raw = 4 packed bf16 of this lane; returns the normed + roped row, packed.
__device__ __forceinline__ uint2 norm_rope_row(uint2 raw, uint2 wraw, const float (&c)[4], const float (&s)[4], int lane,
                                               float epsilon) {
    const float x[4] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y)};
    const float w[4] = {bf16_lo(wraw.x), bf16_hi(wraw.x), bf16_lo(wraw.y), bf16_hi(wraw.y)};
    const float sum = reference_order_sum_of_squares(__fmul_rn(x[0], x[0]), __fmul_rn(x[1], x[1]),
                                                     __fmul_rn(x[2], x[2]), __fmul_rn(x[3], x[3]));
    // sum / 128 is exact as a multiplication by 2^-7
    const float inverse_rms = rsqrtf(__fadd_rn(__fmul_rn(sum, 1.0f / (float)kHeadDim), epsilon));
    // An infinite or NaN input makes the sum (the same value in every lane) infinite or NaN; so does a finite
    // input whose square overflows.  Those rows take the integer-rounding path, whose NaN bits are the reference's.
    if (!(sum < CUDART_INF_F)) return norm_rope_row_exact(x, w, c, s, lane, inverse_rms);
    return norm_rope_row_packed(x, w, c, s, lane, inverse_rms);
}
