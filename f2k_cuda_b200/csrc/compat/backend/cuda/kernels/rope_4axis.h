// Source-compatible stand-in for F2K_CUDA src/backend/cuda/kernels/rope_4axis.h:31-50.
// Interleaved-pair rotary embedding whose per-token cos/sin rows already combine the
// four position axes (t, h, w, l):
//   pos = clamp(pos_ids[row], 0, seq_max - 1);  c, s = table[pos][k]
//   x[2k], x[2k+1]  <-  x[2k] c - x[2k+1] s,  x[2k] s + x[2k+1] c
#pragma once

#include <cstdint>
#include <vector>

struct CUstream_st;
using cudaStream_t = CUstream_st*;

namespace f2k::cuda {

// In place on bf16 rows of head_dim elements; tables are device fp32
// [seq_max, head_dim / 2]. Returns false for rows <= 0, odd or > 512 head_dim,
// and when the launch fails.
bool rope_4axis_inplace_bf16(void* x_bf16, const float* cos_table, const float* sin_table,
                             const int32_t* pos_ids, int batch_rows, int head_dim, int seq_max,
                             cudaStream_t stream = nullptr);

// Host-side table construction: token_positions is [seq][axes]; axis a owns
// axes_dim[a] / 2 consecutive pair slots with frequency theta^(-2k / axes_dim[a]).
void build_rope_4axis_tables(const std::vector<int>& axes_dim,
                             const std::vector<std::vector<int>>& token_positions,
                             float theta, std::vector<float>& cos_out,
                             std::vector<float>& sin_out);

}  // namespace f2k::cuda
