// Source-compatible stand-in for the reference header of the same path
// (F2K_CUDA src/backend/cuda/joint_attention.h:21-54): attention over the text
// tokens followed by the image tokens of an MMDiT block, with separate inputs and
// outputs per modality.
//
// Unlike the reference, nothing is concatenated: the engine reads both modalities
// where they lie, so workspace_size_bytes() is 0 and forward() ignores the
// workspace arguments (a caller that still passes the reference-sized buffer is
// fine). Error behaviour is the reference's: no exceptions, ok()/last_error(),
// forward() returns false.
#pragma once

#include <cstddef>

struct CUstream_st;
using cudaStream_t = CUstream_st*;
struct f2k_attn;

namespace f2k::cuda {

class JointAttention {
public:
    struct Config {
        int   batch    = 0;
        int   seq_txt  = 0;
        int   seq_img  = 0;
        int   n_heads  = 0;
        int   head_dim = 0;
        float scale    = 0.0f;
    };

    explicit JointAttention(const Config& cfg);
    ~JointAttention();
    JointAttention(const JointAttention&)            = delete;
    JointAttention& operator=(const JointAttention&) = delete;

    bool        ok() const;
    const char* last_error() const;
    size_t      workspace_size_bytes() const;

    // Every tensor: device bf16 [batch, seq_txt or seq_img, n_heads, head_dim].
    bool forward(const void* Q_txt, const void* K_txt, const void* V_txt,
                 const void* Q_img, const void* K_img, const void* V_img,
                 void* O_txt, void* O_img,
                 void* workspace, size_t workspace_size,
                 cudaStream_t stream = nullptr);

private:
    ::f2k_attn* handle_ = nullptr;
    bool        valid_  = false;
};

}  // namespace f2k::cuda
