// Host-callable launchers of the CUDA kernels behind the C ABI (include/f2k_attn.h).
#pragma once

#include "attn_params.h"

#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

namespace f2k {

// tcgen05 flash-attention forward (attn_fwd_sm100.cu).
size_t      attn_fwd_smem_bytes();
cudaError_t attn_fwd_prepare();   // load + configure the kernel on the current device (idempotent)
cudaError_t attn_fwd_launch(const AttnParams& p, cudaStream_t stream);

// Fused per-head RMSNorm + 4-axis RoPE for the Q and K of up to two streams in one
// launch (qk_prologue.cu). One job per tensor; all jobs share head count and eps.
struct QkPrologueJob {
    const void*  x;        // [batch, seq, heads, 128] bf16, raw projection output
    long long    x_tok_stride;  // elements between two token rows of x (0 = dense, heads * 128)
    void*        y;        // same shape; may equal x
    const void*  gamma;    // [128] bf16
    const float* cos_tab;  // [seq, 64] fp32
    const float* sin_tab;  // [seq, 64] fp32
    int          seq;      // tokens per batch element
    long long    rows;     // batch * seq * heads head-rows
};
constexpr int kMaxPrologueJobs = 4;
struct QkPrologueParams {
    QkPrologueJob job[kMaxPrologueJobs];
    long long     row_start[kMaxPrologueJobs + 1];  // prefix sum of rows
    int           n_jobs;
    int           n_heads;
    float         eps;
};
cudaError_t qk_prologue_launch(const QkPrologueParams& p, cudaStream_t stream);
cudaError_t qk_prologue_prepare();   // load the prologue kernels on the current device

// Head exchange (qk_prologue.cu): the prologue of a rank that holds `s_loc` tokens of all heads,
// writing every head row straight into the memory of the rank that attends that head. Q and K
// are normalised and rotated on the way, V is copied. Destination layout on rank r:
// [world * s_loc tokens, heads_per_rank, 128], this rank's tokens at token offset rank * s_loc.
// The last CTA then stores `value` to flag[0 .. world) (one word per destination rank).
struct QkvScatterParams {
    const void*  q; const void* k; const void* v;          // [s_loc, n_heads, 128] bf16, dense
    const void*  gamma_q; const void* gamma_k;             // [128] bf16
    const float* cos_tab; const float* sin_tab;            // [s_loc, 64] fp32 (this rank's rows)
    unsigned char* dst_q[8]; unsigned char* dst_k[8]; unsigned char* dst_v[8];
    unsigned int*  flag[8];
    unsigned int*  counter;                                // zero before the launch, zero after
    unsigned int   value;
    int   s_loc, n_heads, heads_per_rank, world, rank;
    float eps;
};
cudaError_t qkv_scatter_launch(const QkvScatterParams& p, cudaStream_t stream);

// Stand-alone kernels with the reference's call shapes (qk_prologue.cu).
cudaError_t rmsnorm_rows_launch(const void* x, const void* gamma, void* y, int rows, int dim,
                                float eps, cudaStream_t stream);
cudaError_t rope4_rows_launch(void* x, const float* cos_tab, const float* sin_tab,
                              const int32_t* pos_ids, int rows, int head_dim, int seq_max,
                              cudaStream_t stream);

}  // namespace f2k
