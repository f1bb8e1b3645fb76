// Per-row softmax arithmetic of the attention kernel: a thread owns one query row of a
// 128-key tile in registers (fp32 scores as loaded from tensor memory).
//
//   row_max64       maximum of 64 scores folded into 8 independent chains
//   exp_chunk16     P = 2^(c*s + neg_mc) for 16 scores -> 8 packed bf16 pairs, and the sum of
//                   the unrounded values (four partial sums)
//
// 2^x comes from two places: the special-function unit (ex2.approx, 4 lanes per clock per
// scheduler; the two softmax groups of a CTA share it) and a cubic polynomial on the FMA pipe for
// `kPolyOf8` of every 8 key pairs. Both agree to better than 1e-4 relative, far inside the bf16
// rounding P goes through next. Measured on the 4608-token shape, the polynomial share does not
// pay: 1 of 8 pairs came out between 1.3 % faster and 7 % slower than none depending on how the
// rest of the kernel happened to be scheduled, 2 of 8 and more always slower (the polynomial
// costs issue slots the row needs elsewhere). It ships switched off (F2K_OPT_POLY_OF8 = 0).
#pragma once

#include "ptx.cuh"

namespace f2k {

// Running maxima of 64 scores folded into kMaxChains independent chains (3-input max, two new
// scores per step and chain); `first` starts the chains.
#ifndef F2K_OPT_MAX_CHAINS
#define F2K_OPT_MAX_CHAINS 8
#endif
constexpr int kMaxChains = F2K_OPT_MAX_CHAINS;   // 8 or 4
template <bool kFirst>
__device__ __forceinline__ void row_max64(const uint32_t* s, float (&m)[kMaxChains]) {
    using namespace f2k::ptx;
#pragma unroll
    for (int i = 0; i < 64; i += 2 * kMaxChains)
#pragma unroll
        for (int k = 0; k < kMaxChains; ++k) {
            const float a = __uint_as_float(s[i + 2 * k]), b = __uint_as_float(s[i + 2 * k + 1]);
            m[k] = (kFirst && i == 0) ? fmaxf(a, b) : fmax3(m[k], a, b);
        }
}
__device__ __forceinline__ float row_max_finish(const float (&m)[kMaxChains]) {
    using namespace f2k::ptx;
    if constexpr (kMaxChains == 8)
        return fmaxf(fmax3(m[0], m[1], m[2]), fmax3(fmax3(m[3], m[4], m[5]), m[6], m[7]));
    else
        return fmaxf(fmax3(m[0], m[1], m[2]), m[3]);
}

// 2^x on the FMA pipe: x = n + f by the 1.5*2^23 rounding trick, cubic fit of 2^f on [-0.5, 0.5]
// (relative error < 1e-4, far inside bf16 resolution), exponent patched in with an integer
// shift-add: six FMA-pipe operations, one clamp and one shift-add. x is clamped at -126 so that
// the exponent arithmetic cannot wrap (the result is then ~2^-126, i.e. nothing). Scalar on
// purpose: the packed f32x2 form measured slower inside the kernel.
__device__ __forceinline__ float exp2_fma_scalar(float x) {
    constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23
    x = fmaxf(x, -126.0f);
    const float t = __fadd_rn(x, kMagic);
    const float f = __fsub_rn(x, __fsub_rn(t, kMagic));
    float p = __fmaf_rn(f, 0.0550886838f, 0.242604051f);
    p = __fmaf_rn(p, f, 0.693276242f);
    p = __fmaf_rn(p, f, 0.99992894f);
    return __uint_as_float((__float_as_uint(t) << 23) + __float_as_uint(p));
}
// 16 scores -> 8 packed bf16 pairs. `pair0` is the index of the first pair inside its group of 8
// pairs (0 or 8 key pairs into a 32-key chunk), which decides who takes the polynomial.
template <int kPolyOf8>
__device__ __forceinline__ void exp_chunk16(const uint32_t* s, uint32_t* pk, float c, float neg_mc,
                                            float (&sum)[4]) {
    using namespace f2k::ptx;
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
        float x0, x1, x2, x3;
        fma2(x0, x1, __uint_as_float(s[i + 0]), __uint_as_float(s[i + 1]), c, c, neg_mc, neg_mc);
        fma2(x2, x3, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]), c, c, neg_mc, neg_mc);
        // pair index within a group of 8 pairs (16 keys); the polynomial pairs are spread out
        // so that both pipes stay busy all the way through the chunk
        const int pa = (i >> 1) & 7, pb = pa + 1;
        const bool poly_a = ((pa + 1) * kPolyOf8 / 8) != (pa * kPolyOf8 / 8);
        const bool poly_b = ((pb + 1) * kPolyOf8 / 8) != (pb * kPolyOf8 / 8);
        float p0, p1, p2, p3;
        if (poly_a) { p0 = exp2_fma_scalar(x0); p1 = exp2_fma_scalar(x1); }
        else { p0 = ex2_approx(x0); p1 = ex2_approx(x1); }
        if (poly_b) { p2 = exp2_fma_scalar(x2); p3 = exp2_fma_scalar(x3); }
        else { p2 = ex2_approx(x2); p3 = ex2_approx(x3); }
        add2(sum[0], sum[1], sum[0], sum[1], p0, p1);
        add2(sum[2], sum[3], sum[2], sum[3], p2, p3);
        pk[i / 2 + 0] = pack_bf16x2(p0, p1);
        pk[i / 2 + 1] = pack_bf16x2(p2, p3);
    }
}

}  // namespace f2k
