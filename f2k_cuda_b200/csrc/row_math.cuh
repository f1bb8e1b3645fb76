// Per-row arithmetic of the QK prologue (per-head RMSNorm + interleaved-pair rotation) shared by
// the stand-alone prologue kernels (qk_prologue.cu) and the head exchange that the attention
// kernel's spare warps run (attn_fwd_sm100.cu): a half-warp owns one 128-element head row, lane i
// holds elements [8i, 8i+8) = rotation pairs 4i .. 4i+3.
#pragma once

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace f2k {

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i]     = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&b);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 v;
    v.x = pack2(f[0], f[1]);
    v.y = pack2(f[2], f[3]);
    v.z = pack2(f[4], f[5]);
    v.w = pack2(f[6], f[7]);
    return v;
}
// One rotation, with the roundings spelled out: x0 c - x1 s as fma(x0, c, -(x1 s)) and
// x0 s + x1 c as fma(x1, c, x0 s). This is what nvcc makes of the reference kernel's expressions
// (src/backend/cuda/kernels/rope_4axis.cu:35-36), so the stand-alone kernels reproduce its bits.
__device__ __forceinline__ void rotate_pair(float& y0, float& y1, float x0, float x1, float c, float s) {
    y0 = __fmaf_rn(x0, c, -__fmul_rn(x1, s));
    y1 = __fmaf_rn(x1, c, __fmul_rn(x0, s));
}

// Sum over the 16 lanes of a half-warp (xor offsets below 16 never leave the half).
// The two halves of a warp may leave the row loop at different times, so each half
// synchronises only with itself.
__device__ __forceinline__ float half_warp_sum(float v) {
    const uint32_t mask = 0xFFFFu << (threadIdx.x & 16);
    v += __shfl_xor_sync(mask, v, 8);
    v += __shfl_xor_sync(mask, v, 4);
    v += __shfl_xor_sync(mask, v, 2);
    v += __shfl_xor_sync(mask, v, 1);
    return v;
}

// y = RoPE(RMSNorm(x) * g) for the 8 elements of a row this lane holds; cs/sn are the lane's four
// (cos, sin) pairs of the token. fp32 arithmetic, one bf16 rounding.
__device__ __forceinline__ uint4 norm_rope_row(const uint4& raw, const float (&g)[8], const float (&cs)[4],
                                               const float (&sn)[4], float eps) {
    float v[8];
    unpack8(raw, v);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
    ss = half_warp_sum(ss);
    const float rrms = rsqrtf(ss * (1.0f / 128.0f) + eps);
    float y[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float a = v[2 * k] * rrms * g[2 * k];
        const float b = v[2 * k + 1] * rrms * g[2 * k + 1];
        rotate_pair(y[2 * k], y[2 * k + 1], a, b, cs[k], sn[k]);
    }
    return pack8(y);
}

}  // namespace f2k
