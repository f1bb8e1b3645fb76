/* f2k_attn.h - C ABI of the B200 (sm_100a) joint-attention engine.
 *
 * This library replaces ONE path of chrisjhebert1973/F2K_CUDA: the MMDiT joint
 * attention of FLUX.2-klein (per-head QK-RMSNorm, 4-axis RoPE, non-causal attention
 * over text||image tokens, 32 heads x head_dim 128, bf16). Each entry point below
 * names the reference interface it stands in for (paths inside the reference tree).
 *
 * Conventions
 *  - Every tensor pointer is a DEVICE pointer to contiguous bf16 laid out
 *    [batch, seq, n_heads, head_dim] unless the function says "host".
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *  - Calls return 0 on success and a positive F2K_ERR_* code otherwise; nothing throws.
 *    f2k_attn_last_error() gives a message that stays valid until the next call on
 *    the same handle.
 *  - forward calls are asynchronous on `stream`, never synchronise and never allocate
 *    (the *_host variant allocates its staging buffers on its first call only).
 *  - The kernels use 16-byte loads and stores: every tensor, gain and RoPE-table pointer must be
 *    16-byte aligned, and a call with one that is not is refused with F2K_ERR_INVALID before
 *    anything is launched. (The reference's stand-alone kernels use 2-byte accesses and take any
 *    bf16-aligned pointer; its callers only ever pass cudaMalloc'd bases and whole-row offsets,
 *    which are 16-byte aligned.)
 *  - A handle holds mutable state (error text, cached TMA descriptors): use it from
 *    one host thread at a time. Distinct handles on distinct streams are independent.
 *  - There is no CPU fallback and no other GPU path: on a device that is not
 *    compute capability 10.x, or for head_dim != 128, creation fails with a message.
 *  - Three environment variables override choices the library otherwise makes itself; they
 *    exist for measurements and tests: F2K_HOST_PIPELINE = "rows" | "heads" and
 *    F2K_HOST_GROUPS = n (how f2k_attn_forward_fused_host splits its work),
 *    F2K_SEQPAR_GROUPS = n (head groups a shard is pulled in by f2k_seqpar_forward).
 */
#ifndef F2K_ATTN_H
#define F2K_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct f2k_attn f2k_attn; /* opaque */

enum {
    F2K_OK              = 0,
    F2K_ERR_INVALID     = 1, /* zero/negative dimension, null pointer */
    F2K_ERR_UNSUPPORTED = 2, /* head_dim != 128, wrong GPU architecture */
    F2K_ERR_WORKSPACE   = 3, /* workspace smaller than the *_workspace_bytes() value */
    F2K_ERR_CUDA        = 4, /* a CUDA runtime/driver call failed; message has the detail */
    F2K_ERR_DEVICE      = 5  /* a kernel reported a problem through the status word */
};

/* Shape of one attention module, fixed at creation like the reference's
 * Attention::Config (src/backend/cuda/attention.h:31-37) and JointAttention::Config
 * (src/backend/cuda/joint_attention.h:23-30).  seq_txt == 0 describes the plain
 * self-attention module over seq_img tokens. */
typedef struct f2k_attn_config {
    int   batch;
    int   seq_txt;
    int   seq_img;
    int   n_heads;
    int   head_dim; /* 128 */
    float scale;    /* <= 0 selects 1/sqrt(head_dim), as the reference does */
} f2k_attn_config;

/* Replaces Attention::Attention (src/backend/cuda/attention.cu:763-776) and
 * JointAttention::JointAttention (src/backend/cuda/joint_attention.cu:78-112).
 * *out is set to a handle whenever memory for it could be obtained, also on failure,
 * so that the message can be read; a failed handle refuses every forward call. */
int f2k_attn_create(const f2k_attn_config* cfg, f2k_attn** out);

/* Replaces the destructors of both reference classes. NULL is allowed. */
void f2k_attn_destroy(f2k_attn* h);

/* Replaces Attention::last_error / JointAttention::last_error
 * (src/backend/cuda/attention.cu:781, joint_attention.cu:117-119). */
const char* f2k_attn_last_error(const f2k_attn* h);

/* Replaces JointAttention::workspace_size_bytes (joint_attention.cu:120-122).
 * The reference needs four concatenation buffers; this engine reads both streams in
 * place, so the answer is 0 and f2k_attn_forward accepts workspace == NULL. */
size_t f2k_attn_workspace_bytes(const f2k_attn* h);

/* Workspace of f2k_attn_forward_fused: normalised+rotated copies of Q and K. */
size_t f2k_attn_fused_workspace_bytes(const f2k_attn* h);

/* Replaces JointAttention::forward (joint_attention.cu:124-167) and, with
 * seq_txt == 0 and the *_txt pointers NULL, Attention::forward
 * (attention.cu:887-927). Inputs are already normalised and rotated by the caller.
 * O_txt/O_img receive softmax(scale * Q K^T) V over the text||image sequence. */
int f2k_attn_forward(f2k_attn* h,
                     const void* q_txt, const void* k_txt, const void* v_txt,
                     const void* q_img, const void* k_img, const void* v_img,
                     void* o_txt, void* o_img,
                     void* workspace, size_t workspace_bytes, void* stream);

/* The whole per-block sequence of the reference callers in one call
 * (DoubleStreamBlock::forward, src/backend/cuda/double_stream_block.cu:290-379;
 * SingleStreamBlock::forward, single_stream_block.cu:254-267): per-head RMSNorm of Q
 * and K with the stream's gains, 4-axis RoPE with the stream's tables at position =
 * token index, then joint attention. q and k are the raw projection outputs and are
 * left untouched; V gets neither step. gamma_*: [128] bf16. cos/sin: fp32
 * [seq, 64] as built by f2k_build_rope_4axis_tables. */
int f2k_attn_forward_fused(f2k_attn* h,
                           const void* q_txt, const void* k_txt, const void* v_txt,
                           const void* q_img, const void* k_img, const void* v_img,
                           const void* gamma_q_txt, const void* gamma_k_txt,
                           const void* gamma_q_img, const void* gamma_k_img,
                           const float* cos_txt, const float* sin_txt,
                           const float* cos_img, const float* sin_img,
                           float eps,
                           void* o_txt, void* o_img,
                           void* workspace, size_t workspace_bytes, void* stream);

/* Token strides, in elements, for a fused call whose tensor rows are not dense. A token row of
 * Q, K or V may be a slice of a wider row - the fused QKV(+MLP) projection output of the
 * reference's single-stream block, 36864 elements per token, which the reference first splits
 * with split_qkv_mlp_kernel (src/backend/cuda/kernels/qkv_mlp_split.cu:12-42) - and a row of O
 * a slice of the [attn | mlp] buffer it otherwise fills with concat_attn_mlp_kernel (same file,
 * :44-57; 16384 elements per token). 0 = dense (n_heads * 128). Rows of all batch elements are
 * consecutive: token (b, s) starts at (b * seq + s) * stride. Every stride must be a multiple
 * of 8 and at least n_heads * 128; every base pointer 16-byte aligned. */
typedef struct f2k_attn_strides {
    long long q_txt, k_txt, v_txt, o_txt;
    long long q_img, k_img, v_img, o_img;
} f2k_attn_strides;

/* f2k_attn_forward_fused on strided rows (strides NULL = all dense): reads Q, K, V where the
 * projection left them and writes O where the next layer wants it, so that the reference's
 * split and concat copies around the attention (single_stream_block.cu:247-250, 272-274)
 * are not needed. The normalised Q/K copies in the workspace stay dense. */
int f2k_attn_forward_fused_strided(f2k_attn* h,
                                   const void* q_txt, const void* k_txt, const void* v_txt,
                                   const void* q_img, const void* k_img, const void* v_img,
                                   const void* gamma_q_txt, const void* gamma_k_txt,
                                   const void* gamma_q_img, const void* gamma_k_img,
                                   const float* cos_txt, const float* sin_txt,
                                   const float* cos_img, const float* sin_img,
                                   float eps,
                                   void* o_txt, void* o_img,
                                   const f2k_attn_strides* strides,
                                   void* workspace, size_t workspace_bytes, void* stream);

/* Same computation as f2k_attn_forward_fused with q, k, v, o in HOST memory (pinned
 * memory makes the copies asynchronous); gains and tables stay device pointers, like
 * the construction-time uploads of the reference. Never synchronises: the call starts
 * after earlier work on `stream`, and later work on `stream` starts after the outputs
 * are in host memory. Inside, larger problems run as a pipeline over groups of heads on
 * two transfer streams the handle owns, so that the copies in, the kernels and the
 * copies out of different groups overlap. Device staging, streams and per-group state
 * are allocated on the first call.
 * No counterpart in the reference, whose callers always hold device buffers; it exists
 * so that end-to-end time including host<->device traffic can be measured. */
int f2k_attn_forward_fused_host(f2k_attn* h,
                                const void* hq_txt, const void* hk_txt, const void* hv_txt,
                                const void* hq_img, const void* hk_img, const void* hv_img,
                                const void* gamma_q_txt, const void* gamma_k_txt,
                                const void* gamma_q_img, const void* gamma_k_img,
                                const float* cos_txt, const float* sin_txt,
                                const float* cos_img, const float* sin_img,
                                float eps,
                                void* ho_txt, void* ho_img, void* stream);

/* The computation of f2k_attn_forward_fused for callers that cannot allocate device memory:
 * a real-time loop that may not take the allocator's locks, a plug-in whose host application
 * forbids device allocations after start-up, a process whose device memory was all handed out
 * at start-up. It
 * needs no handle (f2k_attn_create allocates a status word) and no workspace: both live in a
 * 32 MiB array inside the library's device image. Shapes whose
 * normalised Q and K copies do not fit (256 + 2*B*(seq_txt+seq_img)*n_heads*128*2 bytes, each
 * tensor rounded up to 256) are refused with F2K_ERR_WORKSPACE and a message.
 * The array's 32 MiB are reserved on a GPU when the CUDA runtime loads the module that holds it
 * into that GPU's context: with the runtime's default lazy loading that is the FIRST call of
 * this function or of f2k_attn_noalloc_device_status on the device (with
 * CUDA_MODULE_LOADING=EAGER, context creation). That first call also looks the array's device
 * address up and loads the kernels. It is the one call that can fail for lack of device memory:
 * make it at start-up, before device memory is handed out and before any stream capture
 * (f2k_attn_noalloc_device_status(NULL, NULL, 0) is enough). After it nothing in these two
 * calls allocates, frees or loads. The memory stays reserved until the process exits.
 * All calls on a device share the array: calls whose GPU work may overlap race on it, so keep
 * them on one stream. errbuf (may be NULL) receives a message when the result is not F2K_OK.
 * No counterpart in the reference, whose callers always allocate their own workspace. */
int f2k_attn_forward_fused_noalloc(const f2k_attn_config* cfg,
                                   const void* q_txt, const void* k_txt, const void* v_txt,
                                   const void* q_img, const void* k_img, const void* v_img,
                                   const void* gamma_q_txt, const void* gamma_k_txt,
                                   const void* gamma_q_img, const void* gamma_k_img,
                                   const float* cos_txt, const float* sin_txt,
                                   const float* cos_img, const float* sin_img,
                                   float eps, void* o_txt, void* o_img, void* stream,
                                   char* errbuf, size_t errbuf_len);

/* The status word of f2k_attn_forward_fused_noalloc on the current device (it lives in the same
 * built-in array; there is no handle to ask). Synchronises the device, stores the word to
 * *status_out (may be NULL) and, when it is not zero, clears it and returns F2K_ERR_DEVICE: a
 * bounded wait inside a kernel expired and the outputs of the allocation-free calls since the
 * last read must not be used. The word is not cleared by the forward calls, so a failure stays
 * visible until it is read here. Allocates nothing (first call on a device: see above).
 * No counterpart in the reference, which never checks for asynchronous kernel failure. */
int f2k_attn_noalloc_device_status(int* status_out, char* errbuf, size_t errbuf_len);

/* Limits of the bounded waits inside the kernels this handle launches, in SM clock cycles
 * (about 1.9e9 per second); 0 keeps the default. in_cta_clk bounds waits between the roles of one
 * thread block (default 2e9); peer_clk bounds waits on words that a copy engine or another GPU
 * writes (default 4e10; only the sequence-parallel layers have such waits). When a wait runs
 * out the kernel returns normally and f2k_attn_device_status reports F2K_ERR_DEVICE.
 * No counterpart in the reference, whose kernels never wait on anything. */
int f2k_attn_set_wait_limits(f2k_attn* h, long long in_cta_clk, long long peer_clk);

/* Reads and clears the device status word the kernels of this handle write
 * (0 = clean). Synchronises the device. A non-zero word means a bounded wait inside
 * a kernel expired and the last outputs must not be used; the call then returns
 * F2K_ERR_DEVICE. No counterpart in the reference, which never checks for
 * asynchronous kernel failure. */
int f2k_attn_device_status(f2k_attn* h, int* status_out);

/* Replaces rmsnorm_bf16 (src/backend/cuda/kernels/rmsnorm.cu:74-88):
 * y = bf16(x * rsqrt(mean(x^2) + eps) * gamma) per row; y may alias x;
 * dim must be a positive multiple of 8. */
int f2k_rmsnorm_bf16(const void* x, const void* gamma, void* y,
                     int rows, int dim, float eps, void* stream);

/* Replaces rope_4axis_inplace_bf16 (src/backend/cuda/kernels/rope_4axis.cu:44-54):
 * interleaved-pair rotation in place, position clamped to [0, seq_max-1];
 * head_dim must be even and <= 512. */
int f2k_rope_4axis_inplace_bf16(void* x, const float* cos_table, const float* sin_table,
                                const int32_t* pos_ids, int rows, int head_dim, int seq_max,
                                void* stream);

/* Replaces build_rope_4axis_tables (src/backend/cuda/kernels/rope_4axis.cu:56-97).
 * Host function. positions is [seq][n_axes] row-major; cos_out/sin_out receive
 * [seq][sum(axes_dim)/2] fp32. */
int f2k_build_rope_4axis_tables(const int* axes_dim, int n_axes,
                                const int* positions, int seq, float theta,
                                float* cos_out, float* sin_out);

/* ---- sequence-parallel attention over the GPUs of one box --------------------------------
 * None of this has a counterpart in the reference, which runs on a single GPU. Tokens are
 * sharded by rank (one process per GPU); every rank attends its seq_local queries to the keys
 * and values of all ranks. Remote K/V shards are pulled into local memory by the copy engines
 * over NVLink while the attention kernel already works on the shards that have arrived.
 * Call order per step: write this rank's normalised K and its V (on the compute stream) to the
 * pointers given by f2k_seqpar_local_kv, then f2k_seqpar_forward. No collective is needed: the
 * ranks announce "written" to each other through words in their shard buffers.
 * Meant for one process per GPU. Several ranks on ONE GPU (an emulation for tests) work only if
 * every rank's K/V is in place before the first rank calls forward (a rank's kernel fills the
 * GPU and must never wait for another rank's kernels) and the process has at least two hardware
 * queues per rank (CUDA_DEVICE_MAX_CONNECTIONS), so that no two streams share one. */
typedef struct f2k_seqpar f2k_seqpar; /* opaque */

typedef struct f2k_seqpar_config {
    int   batch;
    int   seq_local; /* tokens held by every rank */
    int   n_heads;
    int   head_dim;  /* 128 */
    int   world;     /* 1..8 ranks */
    int   rank;
    float scale;     /* <= 0 selects 1/sqrt(head_dim) */
} f2k_seqpar_config;

/* Allocates this rank's shard buffer (4 * world * B * seq_local * n_heads * 128 * 2 bytes). */
int         f2k_seqpar_create(const f2k_seqpar_config* cfg, f2k_seqpar** out);
void        f2k_seqpar_destroy(f2k_seqpar* h);
const char* f2k_seqpar_last_error(const f2k_seqpar* h);
/* Base and size of this rank's shard buffer (to be exported to the peers). */
int f2k_seqpar_buffer(f2k_seqpar* h, void** base, size_t* bytes);
/* peer_bases[r] = rank r's shard buffer as addressable from this process (entry `rank` is
 * ignored): an f2k_ipc_open mapping, or the pointer itself when ranks share a process. */
int f2k_seqpar_attach(f2k_seqpar* h, void* const* peer_bases);
/* Where this rank's K (normalised, rotated) and V for the next forward call have to be written. */
int f2k_seqpar_local_kv(f2k_seqpar* h, void** k, void** v);
/* q_local, o_local: [batch, seq_local, n_heads, 128] bf16. overlap != 0: the kernel starts at
 * once and waits per shard for its arrival; overlap == 0: it starts after all pulls.
 * copy_stream NULL selects a stream the handle owns (it must differ from compute_stream). */
int f2k_seqpar_forward(f2k_seqpar* h, const void* q_local, void* o_local, int overlap,
                       void* compute_stream, void* copy_stream);
int f2k_seqpar_device_status(f2k_seqpar* h, int* status_out);
/* As f2k_attn_set_wait_limits, for the kernels of this handle. peer_clk bounds the wait for a
 * remote K/V shard's arrival; it has to cover the skew between the rank processes. */
int f2k_seqpar_set_wait_limits(f2k_seqpar* h, long long in_cta_clk, long long peer_clk);
/* The way out when a peer is gone: forward() parks the copy stream on waits for the peers'
 * "written" words, and with a dead peer neither that stream nor anything that synchronises with
 * it (f2k_seqpar_device_status, f2k_seqpar_destroy) would ever return. abort writes the awaited
 * words of the current step itself (on a stream of its own; it does not touch the caller's
 * streams), so the step drains: the pulls copy whatever the peers' slots hold, the kernel's
 * bounded waits are satisfied or have expired, and f2k_seqpar_device_status then returns
 * F2K_ERR_DEVICE once. The output of the aborted step is invalid. */
int f2k_seqpar_abort(f2k_seqpar* h);

/* ---- sequence-parallel attention by head exchange ----------------------------------------
 * Same sharding outside (rank r holds Q, K, V of its seq_local tokens, all heads, and gets the
 * output of its tokens), but inside the attention the HEADS are sharded: every rank attends
 * n_heads / world heads over all tokens. The exchange is done by the kernels themselves with
 * stores into peer memory: one kernel normalises + rotates Q and K and scatters Q, K, V by head
 * (exchange_in); the attention kernel's epilogue writes every output row into the buffer of the
 * rank that owns the token (attend). Traffic per GPU and step is 4 * (world-1)/world shards
 * against 2 * (world-1) shards for the ring above. batch must be 1; world must divide n_heads.
 * Uses f2k_seqpar_config; buffers are exported/attached like the ring's. No reference
 * counterpart. Call order per step, all on one stream: exchange_in, attend, output; a call out of
 * that order is refused (the stream wait of output is what makes the two buffer sets safe to
 * reuse, so a step may not be left unfinished). */
typedef struct f2k_hx f2k_hx; /* opaque */
int         f2k_hx_create(const f2k_seqpar_config* cfg, f2k_hx** out);
void        f2k_hx_destroy(f2k_hx* h);
const char* f2k_hx_last_error(const f2k_hx* h);
int f2k_hx_buffer(f2k_hx* h, void** base, size_t* bytes);
int f2k_hx_attach(f2k_hx* h, void* const* peer_bases);
/* q_raw, k_raw, v: this rank's [seq_local, n_heads, 128] bf16 (raw projections); gains [128] bf16;
 * cos_local/sin_local: this rank's rows of the RoPE tables, [seq_local, 64] fp32. */
int f2k_hx_exchange_in(f2k_hx* h, const void* q_raw, const void* k_raw, const void* v,
                       const void* gamma_q, const void* gamma_k,
                       const float* cos_local, const float* sin_local, float eps, void* stream);
/* exchange_in with the COPY ENGINES doing the transfers: one prologue kernel normalises + rotates Q
 * and K of all heads locally, then strided copies on streams the handle owns deliver every rank's
 * head columns of K, V and Q, nearest consumer first, each followed by a stream write of the
 * arrival word. No SM is busy with the exchange, so the attention kernel that f2k_hx_attend
 * launches right behind it (segments in ring order, local tokens first) runs while the copies are
 * on their way. Same arguments and call order as exchange_in. Every copy stream needs a hardware
 * queue of its own (a copy queued behind the caller's stream would wait for the peers while they
 * wait for it): the process must run with CUDA_DEVICE_MAX_CONNECTIONS >= world + 8, set before CUDA
 * is initialised, or the call is refused with F2K_ERR_UNSUPPORTED. Several ranks on ONE GPU (the
 * tests' emulation): call it for every rank before the first attend. */
int f2k_hx_exchange_in_copy(f2k_hx* h, const void* q_raw, const void* k_raw, const void* v,
                            const void* gamma_q, const void* gamma_k,
                            const float* cos_local, const float* sin_local, float eps, void* stream);
int f2k_hx_attend(f2k_hx* h, void* stream);
/* exchange_in and attend as ONE kernel: the attention kernel's spare warps do the exchange (same
 * arithmetic, same peer stores) while its other warps already attend to what has arrived, local
 * tokens first, so that the exchange's NVLink time hides under the attention. Same arguments as
 * exchange_in; followed by f2k_hx_output like attend. For one process per GPU: several ranks on
 * ONE GPU cannot run this form side by side (each kernel fills the GPU and would wait for the
 * others' exchange); world == 1 works anywhere. */
int f2k_hx_forward(f2k_hx* h, const void* q_raw, const void* k_raw, const void* v,
                   const void* gamma_q, const void* gamma_k,
                   const float* cos_local, const float* sin_local, float eps, void* stream);
/* Makes `stream` wait until every rank has written its heads of this rank's rows; *o_local is
 * then this rank's [seq_local, n_heads, 128] bf16 output (inside the exchange buffer; valid
 * until the exchange_in after next). */
int f2k_hx_output(f2k_hx* h, void** o_local, void* stream);
/* F2K_ERR_DEVICE when a bounded wait of this rank's kernels expired, when a PEER's attention
 * kernel gave up during the last step (it marks this rank's control words before it publishes
 * "done", so stale rows cannot be taken for valid ones), or after f2k_hx_abort. */
int f2k_hx_device_status(f2k_hx* h, int* status_out);
int f2k_hx_set_wait_limits(f2k_hx* h, long long in_cta_clk, long long peer_clk);
/* Releases the stream waits f2k_hx_output queued when a peer is gone (writes this rank's "done"
 * words of the current step itself, on a stream of its own). The step's output is invalid;
 * f2k_hx_device_status then returns F2K_ERR_DEVICE once, and the next exchange_in is accepted. */
int f2k_hx_abort(f2k_hx* h);

/* Introspection of f2k_hx_forward's host-side planning; pure arithmetic, no GPU needed (the
 * tests check its invariants on CPU). No reference counterpart.
 * f2k_hx_exchange_plan: the order in which a rank's exchange warps take their work: up to
 * max_ranges entries {kind (0 = Q rows, 1 = K and V rows), ring step (destination = rank - step),
 * first 16-token block, number of blocks} are written to ranges[4 * i ..], the number of entries
 * to *n_ranges. Every (kind, step, block) occurs exactly once.
 * f2k_hx_kv_walk_tile: the 128-token tile of rank dst_rank's K/V walk (its own tokens to the end
 * of the sequence, then the start) that `token` of the whole sequence belongs to. */
int f2k_hx_exchange_plan(int world, int seq_local, int heads_per_rank, int n_sms, int* ranges, int max_ranges,
                         int* n_ranges);
int f2k_hx_kv_walk_tile(int world, int seq_local, int dst_rank, int token, int* tile);

/* CUDA IPC for the shard buffers: 64-byte handles to pass between the rank processes. */
int f2k_ipc_export(const void* base, void* handle64);
int f2k_ipc_open(const void* handle64, void** base);
int f2k_ipc_close(void* base);

/* The fused prologue kernel on its own: y = RoPE(RMSNorm(x) * gamma) per 128-element head row of
 * x [batch, seq, n_heads, 128], position of a token = its index in seq (pass the rank's slice of
 * the tables). Same arithmetic as the prologue inside f2k_attn_forward_fused; stands in for
 * rmsnorm_bf16 + rope_4axis_inplace_bf16 + fill_pos_ids_expanded of the reference callers
 * (src/backend/cuda/double_stream_block.cu:290-372). y may alias x. */
int f2k_qk_norm_rope_bf16(const void* x, void* y, const void* gamma, const float* cos_table,
                          const float* sin_table, int batch, int seq, int n_heads, float eps,
                          void* stream);

/* Library identification string (static storage). */
const char* f2k_attn_version(void);

#ifdef __cplusplus
}
#endif
#endif /* F2K_ATTN_H */
