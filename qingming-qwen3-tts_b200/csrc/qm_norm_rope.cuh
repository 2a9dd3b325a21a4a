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

// Two bf16 values per instruction.  mul.rn.bf16x2 / add.rn.bf16x2 round the exact product / sum once to bf16.
// The reference multiplies (adds) two bf16 values in fp32 and rounds the result to bf16: the fp32 product of two
// 8-bit significands is exact, and an fp32 sum of two bf16 values rounded again to bf16 equals the once-rounded
// sum (24 >= 2 * 8 + 2 bits), so for finite results both give the same bits.
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t add_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// The same for rows whose values are all finite, on packed pairs: cvt.rn.bf16x2 rounds the fp32 products with
// the inverse RMS (equal to the integer rounding for every finite value); every later step has two bf16
// operands and runs as one packed instruction per pair; the partner values travel as two packed words; and the
// sign of rotate_half is folded into the sine ((-a) * b and a * (-b) are the same bits).
__device__ __forceinline__ uint2 norm_rope_row_packed(const float (&x)[4], uint2 w, uint2 c, uint2 s, int lane, float inverse_rms) {
    const uint32_t a01 = pack_bf16x2(__fmul_rn(x[0], inverse_rms), __fmul_rn(x[1], inverse_rms));
    const uint32_t a23 = pack_bf16x2(__fmul_rn(x[2], inverse_rms), __fmul_rn(x[3], inverse_rms));
    const uint32_t n01 = mul_bf16x2(a01, w.x);
    const uint32_t n23 = mul_bf16x2(a23, w.y);
    const uint32_t p01 = __shfl_xor_sync(0xffffffffu, n01, 16);
    const uint32_t p23 = __shfl_xor_sync(0xffffffffu, n23, 16);
    const uint32_t flip = lane < 16 ? 0x80008000u : 0u;
    const uint32_t f01 = mul_bf16x2(n01, c.x);
    const uint32_t f23 = mul_bf16x2(n23, c.y);
    const uint32_t g01 = mul_bf16x2(p01, s.x ^ flip);
    const uint32_t g23 = mul_bf16x2(p23, s.y ^ flip);
    return make_uint2(add_bf16x2(f01, g01), add_bf16x2(f23, g23));
}

// The rest of one row once its inverse RMS is known (the same value in every lane).  raw, wraw, craw, sraw: this
// lane's four values of the row, of the norm weight and of the RoPE row, packed bf16.  `exact` (the same in every
// lane) selects the integer-rounding path, whose NaN bits are the reference's: it is for rows whose sum of squares
// is not finite (an infinite or NaN input, or a finite one whose square overflows).
__device__ __forceinline__ uint2 norm_rope_row_with_inverse(uint2 raw, uint2 wraw, uint2 craw, uint2 sraw, int lane,
                                                            float inverse_rms, bool exact) {
    const float x[4] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y)};
    if (exact) {
        const float w[4] = {bf16_lo(wraw.x), bf16_hi(wraw.x), bf16_lo(wraw.y), bf16_hi(wraw.y)};
        const float c[4] = {bf16_lo(craw.x), bf16_hi(craw.x), bf16_lo(craw.y), bf16_hi(craw.y)};
        const float s[4] = {bf16_lo(sraw.x), bf16_hi(sraw.x), bf16_lo(sraw.y), bf16_hi(sraw.y)};
        return norm_rope_row_exact(x, w, c, s, lane, inverse_rms);
    }
    return norm_rope_row_packed(x, wraw, craw, sraw, lane, inverse_rms);
}

// sum / 128 is exact as a multiplication by 2^-7
__device__ __forceinline__ float inverse_rms_of(float sum, float epsilon) {
    return rsqrtf(__fadd_rn(__fmul_rn(sum, 1.0f / (float)kHeadDim), epsilon));
}

// The rest of one row once its sum of squares (the same value in every lane) is known.
__device__ __forceinline__ uint2 norm_rope_row_with_sum(uint2 raw, uint2 wraw, uint2 craw, uint2 sraw, int lane, float epsilon,
                                                        float sum) {
    return norm_rope_row_with_inverse(raw, wraw, craw, sraw, lane, inverse_rms_of(sum, epsilon), !(sum < CUDART_INF_F));
}

// One row: returns the normed + roped row, packed.
__device__ __forceinline__ uint2 norm_rope_row(uint2 raw, uint2 wraw, uint2 craw, uint2 sraw, int lane, float epsilon) {
    const float x[4] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y)};
    const float sum = reference_order_sum_of_squares(__fmul_rn(x[0], x[0]), __fmul_rn(x[1], x[1]),
                                                     __fmul_rn(x[2], x[2]), __fmul_rn(x[3], x[3]));
    return norm_rope_row_with_sum(raw, wraw, craw, sraw, lane, epsilon, sum);
}

// Sums of squares of EIGHT rows held by one warp, in the same order of additions as above, with 30 shuffles
// instead of 112.  After an xor butterfly step both partners hold the same sum, so half of its results are
// redundant: here, at the step over lane bit b, a lane with the bit clear keeps the rows whose index has the
// matching bit clear and hands its values of the other rows to its partner, and the other way round.  Every kept
// value is own + partner's, the same two operands as in the full butterfly (in one order or the other, which gives
// the same bits).  Three steps (lane xor 4, 2, 1: the reference's offsets 16, 8, 4 within its warp) leave lane l
// with the four partial sums of row (l & 7); the last two tree levels and the fold over the four reference warps
// follow as above.  Returns the sum of row (lane & 7).
__device__ __forceinline__ float reference_order_sum_of_squares_rows8(const uint2 (&raw)[8], int lane) {
    const bool up4 = (lane & 4) != 0, up2 = (lane & 2) != 0, up1 = (lane & 1) != 0;     // row bits 2, 1, 0
    float v[4];                       // v[i]: partial sum over this lane's value i
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // value i of the eight rows, one after the other, so that few squares are alive at a time
        float q[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const uint32_t word = i < 2 ? raw[r].x : raw[r].y;
            const float x = (i & 1) ? bf16_hi(word) : bf16_lo(word);
            q[r] = __fmul_rn(x, x);
        }
        float h[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {          // rows r and r + 4 meet over lane bit 2
            const float keep = up4 ? q[r + 4] : q[r];
            const float give = up4 ? q[r] : q[r + 4];
            h[r] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, give, 4));
        }
        float p[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {          // rows r and r + 2 over lane bit 1
            const float keep = up2 ? h[r + 2] : h[r];
            const float give = up2 ? h[r] : h[r + 2];
            p[r] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, give, 2));
        }
        const float keep = up1 ? p[1] : p[0];  // rows r and r + 1 over lane bit 0
        const float give = up1 ? p[0] : p[1];
        v[i] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, give, 1));
    }
    const float s0 = __fadd_rn(v[0], v[2]);
    const float s1 = __fadd_rn(v[1], v[3]);
    const float warp_sum = __fadd_rn(s0, s1);
    const float pair_sum = __fadd_rn(warp_sum, __shfl_xor_sync(0xffffffffu, warp_sum, 16));
    return __fadd_rn(pair_sum, __shfl_xor_sync(0xffffffffu, pair_sum, 8));
}
