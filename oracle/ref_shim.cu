// extern "C" doorway into the UNMODIFIED reference sources, for tests and the
// benchmark's reference arm only (test infrastructure, like the rest of oracle/).
//
// oracle/Makefile compiles this file together with the reference's own
//   src/backend/cuda/attention.cu, joint_attention.cu, kernels/rmsnorm.cu,
//   kernels/rope_4axis.cu
// (read where they lie in the reference checkout, never copied) into
// oracle/_ref/libf2k_ref.so for sm_100a. Everything here only forwards to the
// reference's public C++ API (f2k::cuda::Attention, JointAttention, rmsnorm_bf16,
// rope_4axis_inplace_bf16, build_rope_4axis_tables).

#include "backend/cuda/attention.h"
#include "backend/cuda/joint_attention.h"
#include "backend/cuda/kernels/rmsnorm.h"
#include "backend/cuda/kernels/rope_4axis.h"

#include <cstring>
#include <vector>

using f2k::cuda::Attention;
using f2k::cuda::JointAttention;

extern "C" {

void* f2k_ref_joint_create(int batch, int seq_txt, int seq_img, int n_heads, int head_dim, float scale) {
    JointAttention::Config c{};
    c.batch = batch; c.seq_txt = seq_txt; c.seq_img = seq_img;
    c.n_heads = n_heads; c.head_dim = head_dim; c.scale = scale;
    return new JointAttention(c);
}
int f2k_ref_joint_ok(void* h) { return static_cast<JointAttention*>(h)->ok() ? 1 : 0; }
const char* f2k_ref_joint_last_error(void* h) { return static_cast<JointAttention*>(h)->last_error(); }
size_t f2k_ref_joint_workspace_bytes(void* h) { return static_cast<JointAttention*>(h)->workspace_size_bytes(); }
int f2k_ref_joint_forward(void* h, const void* q_txt, const void* k_txt, const void* v_txt,
                          const void* q_img, const void* k_img, const void* v_img, void* o_txt,
                          void* o_img, void* ws, size_t ws_bytes, void* stream) {
    return static_cast<JointAttention*>(h)->forward(q_txt, k_txt, v_txt, q_img, k_img, v_img, o_txt,
                                                    o_img, ws, ws_bytes,
                                                    static_cast<cudaStream_t>(stream)) ? 1 : 0;
}
void f2k_ref_joint_destroy(void* h) { delete static_cast<JointAttention*>(h); }

void* f2k_ref_attn_create(int batch, int seq, int n_heads, int head_dim, float scale) {
    Attention::Config c{};
    c.batch = batch; c.seq = seq; c.n_heads = n_heads; c.head_dim = head_dim; c.scale = scale;
    return new Attention(c);
}
int f2k_ref_attn_ok(void* h) { return static_cast<Attention*>(h)->ok() ? 1 : 0; }
const char* f2k_ref_attn_last_error(void* h) { return static_cast<Attention*>(h)->last_error(); }
int f2k_ref_attn_forward(void* h, const void* q, const void* k, const void* v, void* o, void* stream) {
    return static_cast<Attention*>(h)->forward(q, k, v, o, static_cast<cudaStream_t>(stream)) ? 1 : 0;
}
void f2k_ref_attn_destroy(void* h) { delete static_cast<Attention*>(h); }

int f2k_ref_rmsnorm_bf16(const void* x, const void* gamma, void* y, int rows, int dim, float eps, void* stream) {
    return f2k::cuda::rmsnorm_bf16(x, gamma, y, rows, dim, eps, static_cast<cudaStream_t>(stream)) ? 1 : 0;
}
int f2k_ref_rope_4axis_inplace_bf16(void* x, const float* cos_table, const float* sin_table,
                                    const int32_t* pos_ids, int rows, int head_dim, int seq_max,
                                    void* stream) {
    return f2k::cuda::rope_4axis_inplace_bf16(x, cos_table, sin_table, pos_ids, rows, head_dim, seq_max,
                                              static_cast<cudaStream_t>(stream)) ? 1 : 0;
}
void f2k_ref_build_rope_4axis_tables(const int* axes_dim, int n_axes, const int* positions, int seq,
                                     float theta, float* cos_out, float* sin_out) {
    std::vector<int> axes(axes_dim, axes_dim + n_axes);
    std::vector<std::vector<int>> pos(seq, std::vector<int>(n_axes));
    for (int s = 0; s < seq; ++s)
        for (int a = 0; a < n_axes; ++a) pos[s][a] = positions[(size_t)s * n_axes + a];
    std::vector<float> c, sn;
    f2k::cuda::build_rope_4axis_tables(axes, pos, theta, c, sn);
    std::memcpy(cos_out, c.data(), c.size() * sizeof(float));
    std::memcpy(sin_out, sn.data(), sn.size() * sizeof(float));
}

}  // extern "C"
