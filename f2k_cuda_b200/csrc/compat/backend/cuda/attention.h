// Source-compatible stand-in for the reference header of the same path
// (F2K_CUDA src/backend/cuda/attention.h:29-54). Code that includes
// "backend/cuda/attention.h" and links against libf2k_attn instead of the
// reference's attention.cu keeps compiling unchanged; the work is done by the
// sm_100a engine behind the C ABI in include/f2k_attn.h.
//
// Contract kept from the reference: Q, K, V, O are device pointers to bf16
// [batch, seq, n_heads, head_dim]; scale <= 0 means 1/sqrt(head_dim); the
// constructor never throws and reports problems through ok()/last_error();
// forward() is asynchronous on `stream` and returns false on failure.
// Deviation: only head_dim == 128 is implemented (the MMDiT shape). Any other
// head_dim constructs an object whose ok() is false and whose last_error() says so.
#pragma once

#include <cstddef>

struct CUstream_st;
using cudaStream_t = CUstream_st*;
struct f2k_attn;

namespace f2k::cuda {

class Attention {
public:
    struct Config {
        int   batch    = 0;
        int   seq      = 0;
        int   n_heads  = 0;
        int   head_dim = 0;
        float scale    = 0.0f;
    };

    explicit Attention(const Config& cfg);
    ~Attention();
    Attention(const Attention&)            = delete;
    Attention& operator=(const Attention&) = delete;

    bool        ok() const;
    const char* last_error() const;

    bool forward(const void* Q, const void* K, const void* V, void* O,
                 cudaStream_t stream = nullptr);

private:
    ::f2k_attn* handle_ = nullptr;
    bool        valid_  = false;
};

}  // namespace f2k::cuda
