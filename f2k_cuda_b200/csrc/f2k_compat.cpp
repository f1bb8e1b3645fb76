// C++ call surface of the reference (f2k::cuda::Attention, JointAttention,
// rmsnorm_bf16, rope_4axis_inplace_bf16, build_rope_4axis_tables) implemented on
// top of the C ABI. Host-only code: it holds a handle and forwards.

#include "backend/cuda/attention.h"
#include "backend/cuda/joint_attention.h"
#include "backend/cuda/kernels/rmsnorm.h"
#include "backend/cuda/kernels/rope_4axis.h"

#include "f2k_attn.h"

namespace f2k::cuda {

// ---- Attention (reference: src/backend/cuda/attention.cu:763-781, 887-927) ----
Attention::Attention(const Config& cfg) {
    f2k_attn_config c{};
    c.batch    = cfg.batch;
    c.seq_txt  = 0;
    c.seq_img  = cfg.seq;
    c.n_heads  = cfg.n_heads;
    c.head_dim = cfg.head_dim;
    c.scale    = cfg.scale;
    valid_ = f2k_attn_create(&c, &handle_) == F2K_OK;
}
Attention::~Attention() { f2k_attn_destroy(handle_); }
bool        Attention::ok() const { return valid_; }
const char* Attention::last_error() const { return f2k_attn_last_error(handle_); }
bool Attention::forward(const void* Q, const void* K, const void* V, void* O, cudaStream_t stream) {
    if (!valid_) return false;
    return f2k_attn_forward(handle_, nullptr, nullptr, nullptr, Q, K, V, nullptr, O, nullptr, 0,
                            stream) == F2K_OK;
}

// ---- JointAttention (reference: src/backend/cuda/joint_attention.cu:78-167) ----
JointAttention::JointAttention(const Config& cfg) {
    f2k_attn_config c{};
    c.batch    = cfg.batch;
    // The reference refuses an empty text stream; the C ABI would read 0 as "plain
    // attention", so the refusal is made here by handing over an invalid length.
    c.seq_txt  = cfg.seq_txt > 0 ? cfg.seq_txt : -1;
    c.seq_img  = cfg.seq_img;
    c.n_heads  = cfg.n_heads;
    c.head_dim = cfg.head_dim;
    c.scale    = cfg.scale;
    valid_ = f2k_attn_create(&c, &handle_) == F2K_OK;
}
JointAttention::~JointAttention() { f2k_attn_destroy(handle_); }
bool        JointAttention::ok() const { return valid_; }
const char* JointAttention::last_error() const { return f2k_attn_last_error(handle_); }
size_t      JointAttention::workspace_size_bytes() const {
    return valid_ ? f2k_attn_workspace_bytes(handle_) : 0;
}
bool JointAttention::forward(const void* Q_txt, const void* K_txt, const void* V_txt,
                             const void* Q_img, const void* K_img, const void* V_img, void* O_txt,
                             void* O_img, void* workspace, size_t workspace_size,
                             cudaStream_t stream) {
    if (!valid_) return false;
    return f2k_attn_forward(handle_, Q_txt, K_txt, V_txt, Q_img, K_img, V_img, O_txt, O_img,
                            workspace, workspace_size, stream) == F2K_OK;
}

// ---- kernels ----
bool rmsnorm_bf16(const void* x, const void* gamma, void* y, int batch_rows, int dim, float eps,
                  cudaStream_t stream) {
    return f2k_rmsnorm_bf16(x, gamma, y, batch_rows, dim, eps, stream) == F2K_OK;
}

bool rope_4axis_inplace_bf16(void* x, const float* cos_table, const float* sin_table,
                             const int32_t* pos_ids, int batch_rows, int head_dim, int seq_max,
                             cudaStream_t stream) {
    return f2k_rope_4axis_inplace_bf16(x, cos_table, sin_table, pos_ids, batch_rows, head_dim,
                                       seq_max, stream) == F2K_OK;
}

void build_rope_4axis_tables(const std::vector<int>& axes_dim,
                             const std::vector<std::vector<int>>& token_positions, float theta,
                             std::vector<float>& cos_out, std::vector<float>& sin_out) {
    const int n_axes = (int)axes_dim.size();
    const int seq    = (int)token_positions.size();
    int head_dim = 0;
    for (int d : axes_dim) head_dim += d;
    const size_t n = (size_t)seq * (head_dim / 2);
    cos_out.assign(n, 0.0f);
    sin_out.assign(n, 0.0f);
    if (n == 0 || n_axes == 0) return;
    std::vector<int> flat((size_t)seq * n_axes, 0);
    for (int s = 0; s < seq; ++s)
        for (int a = 0; a < n_axes && a < (int)token_positions[s].size(); ++a)
            flat[(size_t)s * n_axes + a] = token_positions[s][a];
    f2k_build_rope_4axis_tables(axes_dim.data(), n_axes, flat.data(), seq, theta, cos_out.data(),
                                sin_out.data());
}

}  // namespace f2k::cuda
