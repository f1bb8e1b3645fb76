/* f2k_oracle.h - interface of the CPU oracle (test infrastructure, see f2k_oracle.c). */
#ifndef F2K_ORACLE_H
#define F2K_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { F2K_ORACLE_IDEAL = 0, F2K_ORACLE_REF_ROUND = 1 };

/* One joint-attention problem. Tensors are bf16 bit patterns, [batch, seq, heads, D].
 * seq_txt may be 0 (plain attention over the image stream). With apply_prologue == 0 the
 * gamma / table pointers are ignored and q, k are used as given. */
typedef struct f2k_oracle_problem {
    int mode;            /* F2K_ORACLE_IDEAL or F2K_ORACLE_REF_ROUND */
    int apply_prologue;  /* 1: per-head RMSNorm + RoPE of q and k first */
    int batch, seq_txt, seq_img, n_heads, head_dim;
    int head_begin, head_end; /* compute heads [begin, end); end <= 0 means all */
    float scale;         /* <= 0: 1/sqrt(head_dim) */
    float eps;
    const uint16_t *q_txt, *k_txt, *v_txt, *q_img, *k_img, *v_img;
    const uint16_t *gamma_q_txt, *gamma_k_txt, *gamma_q_img, *gamma_k_img;
    const float *cos_txt, *sin_txt, *cos_img, *sin_img; /* [seq, D/2], position = token index */
} f2k_oracle_problem;

/* Writes fp32 outputs [batch, seq_txt|seq_img, heads, D] (only the selected heads).
 * Returns 0 on success. */
int f2k_oracle_joint_path(const f2k_oracle_problem* pr, float* o_txt, float* o_img);

/* Selected query rows (indices into the joint text||image sequence) of one (batch, head):
 * out is fp32 [n_rows][D]. Same arithmetic as f2k_oracle_joint_path; threads split the rows. */
int f2k_oracle_joint_rows(const f2k_oracle_problem* pr, int b, int h, const int* rows, int n_rows, float* out);

int f2k_oracle_attention_f32(const uint16_t* Q, const uint16_t* K, const uint16_t* V, float* O,
                             int B, int S, int H, int D, float scale, int head_begin, int head_end);

void f2k_oracle_rmsnorm_ideal(const uint16_t* x, const uint16_t* gamma, float* y, long rows, int dim, float eps);
void f2k_oracle_rmsnorm_bf16(const uint16_t* x, const uint16_t* gamma, uint16_t* y, long rows, int dim, float eps);
void f2k_oracle_build_rope_tables(const int* axes_dim, int n_axes, const int* positions, int seq,
                                  float theta, float* cos_out, float* sin_out);
void f2k_oracle_rope_bf16(uint16_t* x, const float* cos_tab, const float* sin_tab,
                          const int32_t* pos_ids, long rows, int head_dim, int seq_max);

float    f2k_oracle_bf16_to_f32(uint16_t b);
uint16_t f2k_oracle_f32_to_bf16(float f);
int      f2k_oracle_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif
