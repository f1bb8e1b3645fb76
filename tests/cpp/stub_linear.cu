// A stand-in for the reference's f2k::cuda::Linear (declared in its
// src/backend/cuda/linear.h; the real one is a CUTLASS NVFP4 / MXFP8 GEMM that needs CUTLASS to
// build) for the block-level integration test: same class, same members, weights ignored.
//
//   y[r][n] = bf16( sum_{j<4} x[r][(5 n + 131 j + 7) mod K] * c(n, j) ),   c in (-0.5, 0.5)
//
// a fixed sparse "projection" that mixes four inputs per output, so that every buffer the blocks
// pass around carries values of projection-like size that depend on the row and the column. It is
// the same function in both builds of the test (this repository's attention behind the
// reference's blocks, and the reference's own), so the two can be compared output for output.
#include "backend/cuda/linear.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <string>

namespace {
__device__ __forceinline__ float coeff(unsigned n, unsigned j) {
    unsigned h = n * 2654435761u + j * 40503u + 12345u;
    h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
    return (float)(h & 0xFFFFu) / 65536.0f - 0.5f;
}
__global__ void stub_linear_kernel(const __nv_bfloat16* x, __nv_bfloat16* y, int rows, int K, int N) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * N) return;
    const int r = (int)(i / N), n = (int)(i % N);
    float acc = 0.f;
    for (unsigned j = 0; j < 4; ++j)
        acc += __bfloat162float(x[(long long)r * K + (5u * n + 131u * j + 7u) % (unsigned)K]) * coeff(n, j);
    y[i] = __float2bfloat16(acc);
}
}  // namespace

namespace f2k::cuda {

struct Linear::Impl {
    int rows = 0, K = 0, N = 0;
    bool valid = false;
    std::string err;
};

Linear::Linear(const Config& cfg) : impl_(std::make_unique<Impl>()) {
    impl_->rows = cfg.batch_rows; impl_->K = cfg.in_features; impl_->N = cfg.out_features;
    if (cfg.batch_rows <= 0 || cfg.in_features <= 0 || cfg.out_features <= 0) { impl_->err = "Linear: zero/negative dim"; return; }
    impl_->valid = true;
}
Linear::~Linear() = default;
Linear::Linear(Linear&&) noexcept = default;
Linear& Linear::operator=(Linear&&) noexcept = default;
bool        Linear::ok() const { return impl_ && impl_->valid; }
const char* Linear::last_error() const { return impl_ ? impl_->err.c_str() : "no impl"; }
size_t      Linear::workspace_size_bytes() const { return 256; }
bool Linear::forward(const void* x, void* y, void*, size_t, cudaStream_t stream) {
    if (!ok()) return false;
    const long long n = (long long)impl_->rows * impl_->N;
    stub_linear_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), impl_->rows, impl_->K, impl_->N);
    return cudaPeekAtLastError() == cudaSuccess;
}

}  // namespace f2k::cuda
