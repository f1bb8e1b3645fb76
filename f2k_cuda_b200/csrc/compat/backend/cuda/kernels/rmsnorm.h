// Source-compatible stand-in for F2K_CUDA src/backend/cuda/kernels/rmsnorm.h:23-29.
// y[r, :] = bf16( x[r, :] * rsqrt(mean(x[r, :]^2) + eps) * gamma ), fp32 arithmetic,
// bf16 in and out, y may be x. Returns false for rows <= 0, dim <= 0 or dim % 8 != 0,
// and when the launch fails.
#pragma once

#include <cstddef>

struct CUstream_st;
using cudaStream_t = CUstream_st*;

namespace f2k::cuda {

bool rmsnorm_bf16(const void* x_bf16, const void* gamma_bf16, void* y_bf16,
                  int batch_rows, int dim, float eps, cudaStream_t stream = nullptr);

}  // namespace f2k::cuda
