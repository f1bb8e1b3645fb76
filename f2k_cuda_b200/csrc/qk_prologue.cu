// Memory-bound kernels in front of the attention: per-head RMSNorm and 4-axis RoPE.
//
//  * qk_prologue_kernel     both steps fused, for the Q and K of up to two streams in
//                           ONE launch: reads each raw element once, writes the
//                           normalised + rotated bf16 once (one rounding instead of the
//                           reference's two). Replaces, per block, the reference's
//                           2-4 rmsnorm_bf16 launches, 2-4 rope_4axis_inplace_bf16
//                           launches and the fill_pos_ids_expanded launches
//                           (F2K_CUDA src/backend/cuda/double_stream_block.cu:290-372,
//                           single_stream_block.cu:254-264).
//  * rmsnorm_rows_kernel*   stand-alone RMSNorm with the reference's contract
//                           (src/backend/cuda/kernels/rmsnorm.cu:42-88).
//  * rope4_rows_kernel*     stand-alone interleaved-pair rotation with the reference's
//                           contract (src/backend/cuda/kernels/rope_4axis.cu:13-54).
//
// All of them are HBM-bound: 16-byte loads/stores, a half-warp (dim 128) or a warp per
// 128-element head row, grid sized as a multiple of the SM count, grid-stride loop.

#include "attn_launch.h"
#include "row_math.cuh"

#include <cuda_bf16.h>

namespace f2k {

namespace {

constexpr int kBlock = 256;

__device__ __forceinline__ float warp_sum(float v) {
    v += __shfl_xor_sync(0xFFFFFFFFu, v, 16);
    v += __shfl_xor_sync(0xFFFFFFFFu, v, 8);
    v += __shfl_xor_sync(0xFFFFFFFFu, v, 4);
    v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
    v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
    return v;
}

// ---------------------------------------------------------------------------------
// Fused RMSNorm + RoPE, head_dim 128. A half-warp owns one head row: lane i holds
// elements [8i, 8i+8) = rotation pairs 4i .. 4i+3, so both the reduction and the
// rotation stay inside the half-warp and inside a lane respectively.
// ---------------------------------------------------------------------------------
// A half-warp takes kGroup consecutive head rows of ONE token per iteration (kGroup divides the
// head count): their loads are issued back to back (kGroup x 16 bytes in flight per lane), and the
// token's table row and the gains are fetched once for the group.
template <int kGroup>
__global__ void __launch_bounds__(kBlock, 4)
qk_prologue_kernel(const __grid_constant__ QkPrologueParams p) {
    const int hl = threadIdx.x & 15;  // lane inside the half-warp
    const long long total = p.row_start[p.n_jobs] / kGroup;          // in groups
    const long long n_hw  = (long long)gridDim.x * (kBlock / 16);
    for (long long grp = (long long)blockIdx.x * (kBlock / 16) + (threadIdx.x >> 4); grp < total; grp += n_hw) {
        const long long row = grp * kGroup;
        int j = 0;
#pragma unroll
        for (int i = 1; i < kMaxPrologueJobs; ++i)
            if (i < p.n_jobs && row >= p.row_start[i]) j = i;
        const QkPrologueJob& job = p.job[j];
        const long long lr = row - p.row_start[j];
        const long long trow = lr / p.n_heads;                 // token row over batch * seq
        const int tok = (int)(trow % job.seq);
        const int hd0 = (int)(lr - trow * p.n_heads);           // first head of the group
        // plain loads of x: y may alias x, so x is not read-only for the kernel's lifetime. A token
        // row of x may be a slice of a wider row (x_tok_stride); y is always dense.
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(job.x) +
                                                          trow * job.x_tok_stride + (long long)hd0 * kHeadDim);
        uint4 raw[kGroup];
#pragma unroll
        for (int u = 0; u < kGroup; ++u) raw[u] = src[u * 16 + hl];
        const uint4  graw = __ldg(reinterpret_cast<const uint4*>(job.gamma) + hl);
        const float4 c4 = __ldg(reinterpret_cast<const float4*>(job.cos_tab + (long long)tok * 64) + hl);
        const float4 s4 = __ldg(reinterpret_cast<const float4*>(job.sin_tab + (long long)tok * 64) + hl);
        float g[8];
        unpack8(graw, g);
        const float cs[4] = {c4.x, c4.y, c4.z, c4.w};
        const float sn[4] = {s4.x, s4.y, s4.z, s4.w};
        uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(job.y) + lr * kHeadDim);
#pragma unroll
        for (int u = 0; u < kGroup; ++u) {
            float v[8];
            unpack8(raw[u], v);
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
            ss = half_warp_sum(ss);
            const float rrms = rsqrtf(ss * (1.0f / kHeadDim) + p.eps);
            float y[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float a = v[2 * k] * rrms * g[2 * k];
                const float b = v[2 * k + 1] * rrms * g[2 * k + 1];
                rotate_pair(y[2 * k], y[2 * k + 1], a, b, cs[k], sn[k]);
            }
            dst[u * 16 + hl] = pack8(y);
        }
    }
}

// ---------------------------------------------------------------------------------
// Head exchange: the same row arithmetic, every row stored into the memory of the rank that owns
// its head (peer stores over NVLink, 256 contiguous bytes per half-warp and row). Work item =
// kGroup consecutive heads (all of one destination) of one token of one of the three tensors.
// ---------------------------------------------------------------------------------
template <int kGroup>
__global__ void __launch_bounds__(kBlock, 4)
qkv_scatter_kernel(const __grid_constant__ QkvScatterParams p) {
    const int hl = threadIdx.x & 15;
    const long long per_tensor = (long long)p.s_loc * p.n_heads / kGroup;
    const long long total = 3 * per_tensor;
    const long long n_hw  = (long long)gridDim.x * (kBlock / 16);
    for (long long grp = (long long)blockIdx.x * (kBlock / 16) + (threadIdx.x >> 4); grp < total; grp += n_hw) {
        const int which = (int)(grp / per_tensor);                       // 0 q, 1 k, 2 v
        const long long lr = (grp - which * per_tensor) * kGroup;        // row inside the tensor
        const int tok = (int)(lr / p.n_heads);
        const int hd0 = (int)(lr - (long long)tok * p.n_heads);
        const int dst_rank = hd0 / p.heads_per_rank;
        const int hh = hd0 - dst_rank * p.heads_per_rank;
        const void* xin = which == 0 ? p.q : (which == 1 ? p.k : p.v);
        unsigned char* base = which == 0 ? p.dst_q[dst_rank] : (which == 1 ? p.dst_k[dst_rank] : p.dst_v[dst_rank]);
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(xin) + lr * kHeadDim);
        uint4* dst = reinterpret_cast<uint4*>(
            base + (((long long)p.rank * p.s_loc + tok) * p.heads_per_rank + hh) * (long long)(kHeadDim * 2));
        uint4 raw[kGroup];
#pragma unroll
        for (int u = 0; u < kGroup; ++u) raw[u] = src[u * 16 + hl];
        if (which == 2) {
#pragma unroll
            for (int u = 0; u < kGroup; ++u) dst[u * 16 + hl] = raw[u];
            continue;
        }
        const uint4  graw = __ldg(reinterpret_cast<const uint4*>(which == 0 ? p.gamma_q : p.gamma_k) + hl);
        const float4 c4 = __ldg(reinterpret_cast<const float4*>(p.cos_tab + (long long)tok * 64) + hl);
        const float4 s4 = __ldg(reinterpret_cast<const float4*>(p.sin_tab + (long long)tok * 64) + hl);
        float g[8];
        unpack8(graw, g);
        const float cs[4] = {c4.x, c4.y, c4.z, c4.w};
        const float sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int u = 0; u < kGroup; ++u) {
            float v[8];
            unpack8(raw[u], v);
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
            ss = half_warp_sum(ss);
            const float rrms = rsqrtf(ss * (1.0f / kHeadDim) + p.eps);
            float y[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float a = v[2 * k] * rrms * g[2 * k];
                const float b = v[2 * k + 1] * rrms * g[2 * k + 1];
                rotate_pair(y[2 * k], y[2 * k + 1], a, b, cs[k], sn[k]);
            }
            dst[u * 16 + hl] = pack8(y);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // the same publication as f2k::ptx::grid_done_publish, spelled out here to keep this file
        // free of the PTX header
        __threadfence_system();
        const unsigned int seen = atomicAdd(p.counter, 1u);
        if (seen == gridDim.x - 1u) {
            atomicExch(p.counter, 0u);
            __threadfence_system();
            for (int i = 0; i < p.world; ++i)
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flag[i]), "r"(p.value) : "memory");
        }
    }
}

// ---------------------------------------------------------------------------------
// Stand-alone RMSNorm. dim == 128: half-warp per row, one pass. Other dims (multiple
// of 8): one warp per row, two passes over the row (the second hits L1/L2).
// y = bf16( x * rsqrt(mean(x^2) + eps) * gamma ), fp32 arithmetic.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(kBlock)
rmsnorm_rows128_kernel(const __nv_bfloat16* x, const __nv_bfloat16* __restrict__ gamma,
                       __nv_bfloat16* y, long long rows, float eps) {  // y may alias x
    const int hl = threadIdx.x & 15;
    const long long n_hw = (long long)gridDim.x * (kBlock / 16);
    const uint4 graw = __ldg(reinterpret_cast<const uint4*>(gamma) + hl);
    float g[8];
    unpack8(graw, g);
    for (long long row = (long long)blockIdx.x * (kBlock / 16) + (threadIdx.x >> 4); row < rows;
         row += n_hw) {
        const uint4 raw = reinterpret_cast<const uint4*>(x + row * 128)[hl];
        float v[8];
        unpack8(raw, v);
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
        ss = half_warp_sum(ss);
        const float rrms = rsqrtf(ss * (1.0f / 128.0f) + eps);
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = v[i] * rrms * g[i];
        reinterpret_cast<uint4*>(y + row * 128)[hl] = pack8(o);
    }
}

__global__ void __launch_bounds__(kBlock)
rmsnorm_rows_generic_kernel(const __nv_bfloat16* x, const __nv_bfloat16* __restrict__ gamma,
                            __nv_bfloat16* y, long long rows, int dim, float inv_dim,
                            float eps) {  // y may alias x
    const int lane = threadIdx.x & 31;
    const long long n_w = (long long)gridDim.x * (kBlock / 32);
    const int chunks = dim >> 3;  // 16-byte chunks per row
    for (long long row = (long long)blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5); row < rows;
         row += n_w) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + row * dim);
        float ss = 0.f;
        for (int ch = lane; ch < chunks; ch += 32) {
            float v[8];
            unpack8(xr[ch], v);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
        }
        ss = warp_sum(ss);
        const float rrms = rsqrtf(ss * inv_dim + eps);
        uint4* yr = reinterpret_cast<uint4*>(y + row * dim);
        for (int ch = lane; ch < chunks; ch += 32) {
            float v[8], g[8], o[8];
            unpack8(xr[ch], v);
            unpack8(__ldg(reinterpret_cast<const uint4*>(gamma) + ch), g);
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = v[i] * rrms * g[i];
            yr[ch] = pack8(o);
        }
    }
}

// ---------------------------------------------------------------------------------
// Stand-alone rotation, in place. pos = clamp(pos_ids[row], 0, seq_max - 1);
// x'[2k] = x[2k] c - x[2k+1] s ; x'[2k+1] = x[2k] s + x[2k+1] c with c, s = table[pos][k].
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(kBlock)
rope4_rows128_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cos_tab,
                     const float* __restrict__ sin_tab, const int32_t* __restrict__ pos_ids,
                     long long rows, int seq_max) {
    const int hl = threadIdx.x & 15;
    const long long n_hw = (long long)gridDim.x * (kBlock / 16);
    for (long long row = (long long)blockIdx.x * (kBlock / 16) + (threadIdx.x >> 4); row < rows;
         row += n_hw) {
        int pos = __ldg(pos_ids + row);
        pos = pos >= seq_max ? seq_max - 1 : (pos < 0 ? 0 : pos);
        uint4* xp = reinterpret_cast<uint4*>(x + row * 128) + hl;
        const float4 c4 = __ldg(reinterpret_cast<const float4*>(cos_tab + (long long)pos * 64) + hl);
        const float4 s4 = __ldg(reinterpret_cast<const float4*>(sin_tab + (long long)pos * 64) + hl);
        float v[8], o[8];
        unpack8(*xp, v);
        const float cs[4] = {c4.x, c4.y, c4.z, c4.w};
        const float sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) rotate_pair(o[2 * k], o[2 * k + 1], v[2 * k], v[2 * k + 1], cs[k], sn[k]);
        *xp = pack8(o);
    }
}

__global__ void __launch_bounds__(kBlock)
rope4_rows_generic_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cos_tab,
                          const float* __restrict__ sin_tab, const int32_t* __restrict__ pos_ids,
                          long long rows, int head_dim, int seq_max) {
    const int lane = threadIdx.x & 31;
    const long long n_w = (long long)gridDim.x * (kBlock / 32);
    const int half = head_dim >> 1;
    for (long long row = (long long)blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5); row < rows;
         row += n_w) {
        int pos = __ldg(pos_ids + row);
        pos = pos >= seq_max ? seq_max - 1 : (pos < 0 ? 0 : pos);
        uint32_t* xr = reinterpret_cast<uint32_t*>(x + row * head_dim);
        const float* cr = cos_tab + (long long)pos * half;
        const float* sr = sin_tab + (long long)pos * half;
        for (int k = lane; k < half; k += 32) {
            const uint32_t w = xr[k];
            const float x0 = __uint_as_float(w << 16);
            const float x1 = __uint_as_float(w & 0xFFFF0000u);
            const float c = __ldg(cr + k), s = __ldg(sr + k);
            float y0, y1;
            rotate_pair(y0, y1, x0, x1, c, s);
            xr[k] = pack2(y0, y1);
        }
    }
}

int grid_for(long long units, int units_per_block) {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    const long long need = (units + units_per_block - 1) / units_per_block;
    const long long cap  = (long long)sms * 8;  // 8 x 256 threads = a full SM of resident threads
    return (int)(need < cap ? (need > 0 ? need : 1) : cap);
}

}  // namespace

cudaError_t qk_prologue_prepare() {
    cudaFuncAttributes attr;
    cudaError_t e = cudaFuncGetAttributes(&attr, qk_prologue_kernel<4>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&attr, qk_prologue_kernel<1>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&attr, qkv_scatter_kernel<4>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&attr, qkv_scatter_kernel<1>);
    return e;
}

cudaError_t qk_prologue_launch(const QkPrologueParams& params, cudaStream_t stream) {
    QkPrologueParams p = params;
    for (int i = 0; i < p.n_jobs; ++i)
        if (p.job[i].x_tok_stride == 0) p.job[i].x_tok_stride = (long long)p.n_heads * kHeadDim;
    const long long total = p.row_start[p.n_jobs];
    if (total <= 0) return cudaSuccess;
    if (p.n_heads % 4 == 0)
        qk_prologue_kernel<4><<<grid_for(total / 4, kBlock / 16), kBlock, 0, stream>>>(p);
    else
        qk_prologue_kernel<1><<<grid_for(total, kBlock / 16), kBlock, 0, stream>>>(p);
    return cudaPeekAtLastError();
}

cudaError_t qkv_scatter_launch(const QkvScatterParams& p, cudaStream_t stream) {
    const long long rows = 3ll * p.s_loc * p.n_heads;
    if (rows <= 0) return cudaErrorInvalidValue;
    if (p.heads_per_rank % 4 == 0)
        qkv_scatter_kernel<4><<<grid_for(rows / 4, kBlock / 16), kBlock, 0, stream>>>(p);
    else
        qkv_scatter_kernel<1><<<grid_for(rows, kBlock / 16), kBlock, 0, stream>>>(p);
    return cudaPeekAtLastError();
}

cudaError_t rmsnorm_rows_launch(const void* x, const void* gamma, void* y, int rows, int dim,
                                float eps, cudaStream_t stream) {
    auto xb = static_cast<const __nv_bfloat16*>(x);
    auto gb = static_cast<const __nv_bfloat16*>(gamma);
    auto yb = static_cast<__nv_bfloat16*>(y);
    if (dim == 128) {
        rmsnorm_rows128_kernel<<<grid_for(rows, kBlock / 16), kBlock, 0, stream>>>(xb, gb, yb, rows, eps);
    } else {
        rmsnorm_rows_generic_kernel<<<grid_for(rows, kBlock / 32), kBlock, 0, stream>>>(
            xb, gb, yb, rows, dim, 1.0f / (float)dim, eps);
    }
    return cudaPeekAtLastError();
}

cudaError_t rope4_rows_launch(void* x, const float* cos_tab, const float* sin_tab,
                              const int32_t* pos_ids, int rows, int head_dim, int seq_max,
                              cudaStream_t stream) {
    auto xb = static_cast<__nv_bfloat16*>(x);
    if (head_dim == 128) {
        rope4_rows128_kernel<<<grid_for(rows, kBlock / 16), kBlock, 0, stream>>>(xb, cos_tab, sin_tab,
                                                                                pos_ids, rows, seq_max);
    } else {
        rope4_rows_generic_kernel<<<grid_for(rows, kBlock / 32), kBlock, 0, stream>>>(
            xb, cos_tab, sin_tab, pos_ids, rows, head_dim, seq_max);
    }
    return cudaPeekAtLastError();
}

}  // namespace f2k
