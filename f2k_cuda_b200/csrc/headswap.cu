// Token-sharded in, token-sharded out, heads sharded inside: sequence-parallel attention by head
// exchange over NVLink peer memory ("all-to-all" form). The reference has no multi-GPU code; this
// layer is new, and is the low-traffic alternative to the ring of seqpar.cu: per step a GPU sends
// and receives 4 * (world-1)/world shards instead of 2 * (world-1) shards.
//
// Rank r holds Q, K, V of its s_loc tokens, all heads. Per step:
//
//  1. exchange_in: ONE kernel (qkv_scatter_kernel) reads the rank's raw Q, K, V once, applies
//     QK-RMSNorm + RoPE to Q and K, and stores every head row directly into the memory of the rank
//     that owns the head (peer stores): rank d receives [world * s_loc tokens, heads/world, 128]
//     for Q, K and V. Its last CTA publishes an "arrived" word on every rank.
//  2. attend: the attention kernel over heads/world heads and all tokens. Its TMA producer waits
//     (bounded) for the "arrived" word of a source rank before the first tile of that rank's
//     token range, so it starts on what has arrived. Queries are cut into one segment per
//     source rank, and a segment's output pointer is the SOURCE rank's token-sharded output
//     buffer: the epilogue's stores are the exchange back. The last CTA publishes "done".
//  3. output: stream waits for every rank's "done" word; the rank's [s_loc, heads, 128] output
//     is then complete in its own buffer.
//
// No collective, no copy engine, no kernel that spins on another kernel's progress on the same
// GPU (waits are on words written by other GPUs). Two buffer sets alternate from step to step; a
// peer can be at most one step ahead, because its next exchange needs this rank's "arrived".
//
// One allocation per rank, exported to the peers by CUDA IPC:
//     [2 sets] { Qh, Kh, Vh : [world * s_loc, heads/world, 128] ; O : [s_loc, heads, 128] }
//     control words: arrived[2][world], done[2][world], two counters, failed[2][world];
//     fused form: the chunk queue's counter and delivered-chunk counters [2][world][Q | KV][tiles].
//
// Fused form (f2k_hx_forward): steps 1 and 2 are ONE kernel. The attention kernel's two spare warps
// per CTA do the exchange (same arithmetic, same peer stores), in chunks of 16 tokens taken from a
// queue in the order the consumers need them, while the other roles of every CTA already attend to
// the tiles that have arrived (a counter per 128-token tile says how much of it has been
// delivered): segments are walked in ring order starting with the rank's own tokens, and CTAs are
// numbered so that those of the local query tokens run first. The exchange (NVLink time of 3
// shards) then hides under the attention instead of preceding it. On ONE GPU several ranks cannot
// run this form side by side (a rank's kernel fills the GPU and would wait for a kernel that
// cannot start), so the in-process emulation of the tests uses the two-kernel form; the fused form
// is tested with world 1 on one GPU and with one process per GPU.
//
// Copy-engine form (f2k_hx_exchange_in_copy, then attend): step 1 is a local prologue kernel plus
// strided copies by the copy engines, which need no SM: the attention kernel of step 2 is launched
// right behind the prologue and overlaps the transfers (segments in ring order, the rank's own
// heads put in place on the caller's stream). See the comment at the function.

#include "f2k_attn.h"

#include "attn_launch.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

namespace {
using namespace f2k;

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);
using WaitValue32Fn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);

void* driver_entry(const char* name) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
        return nullptr;
    return p;
}
}  // namespace

struct f2k_hx {
    f2k_seqpar_config cfg{};
    float  scale = 0.f;
    bool   valid = false;
    std::string err;
    unsigned char* buf = nullptr;
    size_t shard_bytes = 0, total_bytes = 0, flags_off = 0;
    int    hpr = 0;                          // heads per rank
    int*   d_status = nullptr;
    std::vector<unsigned char*> peer;
    unsigned int epoch = 0;
    enum Phase { kIdle, kExchanged, kAttended } phase = kIdle;   // exchange_in -> attend -> output -> ...
    long long wait_clk = 0, peer_wait_clk = 0;                   // 0 = the defaults of attn_params.h
    bool   aborted = false;
    unsigned int fail_reported = 0;                              // step whose peer failure was already reported
    cudaStream_t abort_stream = nullptr;
    using WriteValue32Fn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
    WriteValue32Fn write32 = nullptr;
    EncodeTiledFn encode = nullptr;
    WaitValue32Fn wait32 = nullptr;
    AttnParams params[2];                    // per buffer set; only the call number changes between steps
    bool       have_params[2] = {false, false};

    // set layout: Qh | Kh | Vh | O, each shard_bytes
    unsigned char* part(unsigned char* base, int set, int which) const {
        return base + ((size_t)set * 4 + which) * shard_bytes;
    }
    unsigned int* words(unsigned char* base) const { return reinterpret_cast<unsigned int*>(base + flags_off); }
    unsigned int* arrived(unsigned char* base, int set, int src) const { return words(base) + set * 8 + src; }
    unsigned int* done(unsigned char* base, int set, int src) const { return words(base) + 16 + set * 8 + src; }
    unsigned int* counter(int i) const { return words(buf) + 32 + i; }
    // failed[set][src]: rank src stores the step number here when a CTA of its attention kernel gave
    // up, before it publishes done[set][src]: its heads of this rank's rows were not all written
    unsigned int* failed(unsigned char* base, int set, int src) const { return words(base) + 40 + set * 8 + src; }
    // fused form (f2k_hx_forward): the chunk queue's counter, and behind the control header one
    // counter of delivered chunks per (buffer set, source rank, Q | K+V, 128-token tile)
    unsigned int* next_chunk() const { return words(buf) + 96; }
    static constexpr size_t kControlBytes = 1024;
    int n_tiles = 0;
    unsigned int set_uses[2] = {0, 0};       // fused steps run on each buffer set so far
    unsigned int* tile_words(unsigned char* base, int set, int src) const {   // [Q tiles | KV tiles]
        return reinterpret_cast<unsigned int*>(base + flags_off + kControlBytes) + ((size_t)set * cfg.world + src) * 2 * n_tiles;
    }
    // fused form, K/V walked as two segments of the whole buffer: one counter per tile of the walk
    // and buffer set, shared by all sources (behind the per-source counters)
    unsigned int* walk_words(unsigned char* base, int set) const {
        return tile_words(base, 2, 0) + (size_t)set * cfg.world * n_tiles;
    }
    AttnParams fparams[2];                   // fused form, per buffer set
    bool       have_fparams[2] = {false, false};
    // copy-engine form (f2k_hx_exchange_in_copy): normalised Q and K of all heads staged locally,
    // one copy stream per destination, and launch parameters with the segments in ring order
    unsigned char* stage = nullptr;          // [Qn | Kn], each shard_bytes
    cudaStream_t   copy_stream[8] = {};
    cudaEvent_t    ev_prologue = nullptr;
    AttnParams cparams[2];
    bool       have_cparams[2] = {false, false};
    bool       copy_mode = false;            // which exchange the pending attend follows
};

namespace {
int fail(f2k_hx* h, int code, std::string msg) {
    h->err = std::move(msg);
    return code;
}
int fail_cuda(f2k_hx* h, const char* what, cudaError_t e) {
    return fail(h, F2K_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}
// [1, len, heads, 128] bf16 with the given token stride (elements)
bool encode(f2k_hx* h, CUtensorMap* map, const void* base, int len, int heads, long long tok_stride) {
    const cuuint64_t dims[4]    = {(cuuint64_t)kHeadDim, (cuuint64_t)heads, (cuuint64_t)len, 1};
    const cuuint64_t strides[3] = {(cuuint64_t)kHeadDim * 2, (cuuint64_t)tok_stride * 2,
                                   (cuuint64_t)tok_stride * (cuuint64_t)len * 2};
    const cuuint32_t box[4]     = {64, 1, (cuuint32_t)kTileM, 1};
    const cuuint32_t estr[4]    = {1, 1, 1, 1};
    return h->encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace

extern "C" {

int f2k_hx_create(const f2k_seqpar_config* cfg, f2k_hx** out) {
    if (!out) return F2K_ERR_INVALID;
    *out = nullptr;
    f2k_hx* h = new (std::nothrow) f2k_hx();
    if (!h) return F2K_ERR_CUDA;
    *out = h;
    if (!cfg) return fail(h, F2K_ERR_INVALID, "null config");
    h->cfg = *cfg;
    if (cfg->batch != 1) return fail(h, F2K_ERR_UNSUPPORTED, "head exchange: batch must be 1");
    if (cfg->seq_local <= 0 || cfg->n_heads <= 0 || cfg->head_dim <= 0)
        return fail(h, F2K_ERR_INVALID, "head exchange: zero/negative dim");
    if (cfg->world <= 0 || cfg->world > 8 || cfg->rank < 0 || cfg->rank >= cfg->world)
        return fail(h, F2K_ERR_INVALID, "head exchange: world must be 1..8 and 0 <= rank < world");
    if (cfg->n_heads % cfg->world != 0) return fail(h, F2K_ERR_INVALID, "head exchange: world must divide n_heads");
    if (cfg->head_dim != kHeadDim) return fail(h, F2K_ERR_UNSUPPORTED, "head_dim must be 128");
    h->hpr   = cfg->n_heads / cfg->world;
    h->scale = cfg->scale > 0.f ? cfg->scale : 1.0f / std::sqrt((float)cfg->head_dim);
    h->shard_bytes = (size_t)cfg->seq_local * cfg->n_heads * kHeadDim * 2;     // = world*s_loc*hpr*256
    h->flags_off   = 8 * h->shard_bytes;
    h->n_tiles     = (cfg->seq_local + kTileM - 1) / kTileM;
    h->total_bytes = h->flags_off + f2k_hx::kControlBytes +
                     ((size_t)2 * cfg->world * 3 * h->n_tiles * sizeof(unsigned int) + 255) / 256 * 256;

    int dev = 0, major = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail_cuda(h, "cudaGetDevice", e);
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return fail_cuda(h, "cudaDeviceGetAttribute", e);
    if (major != 10) return fail(h, F2K_ERR_UNSUPPORTED, "this library contains sm_100a code only");
    h->encode = reinterpret_cast<EncodeTiledFn>(driver_entry("cuTensorMapEncodeTiled"));
    h->wait32 = reinterpret_cast<WaitValue32Fn>(driver_entry("cuStreamWaitValue32"));
    h->write32 = reinterpret_cast<f2k_hx::WriteValue32Fn>(driver_entry("cuStreamWriteValue32"));
    if (!h->encode || !h->wait32 || !h->write32) return fail(h, F2K_ERR_CUDA, "driver entry points unavailable");
    e = attn_fwd_prepare();
    if (e == cudaSuccess) e = qk_prologue_prepare();
    if (e != cudaSuccess) return fail_cuda(h, "kernel load", e);
    e = cudaMalloc(reinterpret_cast<void**>(&h->buf), h->total_bytes);
    if (e != cudaSuccess) return fail_cuda(h, "cudaMalloc(exchange buffer)", e);
    e = cudaMemset(h->buf + h->flags_off, 0, h->total_bytes - h->flags_off);
    if (e != cudaSuccess) return fail_cuda(h, "cudaMemset(flags)", e);
    e = cudaMalloc(reinterpret_cast<void**>(&h->d_status), kStatusBytes);
    if (e == cudaSuccess) e = cudaMemset(h->d_status, 0, kStatusBytes);
    if (e != cudaSuccess) return fail_cuda(h, "cudaMalloc(status)", e);
    e = cudaStreamCreateWithFlags(&h->abort_stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) return fail_cuda(h, "cudaStreamCreate", e);
    h->peer.assign(cfg->world, nullptr);
    h->peer[cfg->rank] = h->buf;
    h->valid = true;
    return F2K_OK;
}

void f2k_hx_destroy(f2k_hx* h) {
    if (!h) return;
    if (h->abort_stream) cudaStreamDestroy(h->abort_stream);
    for (cudaStream_t cs : h->copy_stream)
        if (cs) { cudaStreamSynchronize(cs); cudaStreamDestroy(cs); }
    if (h->ev_prologue) cudaEventDestroy(h->ev_prologue);
    if (h->stage) cudaFree(h->stage);
    if (h->d_status) cudaFree(h->d_status);
    if (h->buf) cudaFree(h->buf);
    delete h;
}

const char* f2k_hx_last_error(const f2k_hx* h) { return h ? h->err.c_str() : "no handle"; }

int f2k_hx_buffer(f2k_hx* h, void** base, size_t* bytes) {
    if (!h || !h->valid) return F2K_ERR_INVALID;
    if (base) *base = h->buf;
    if (bytes) *bytes = h->total_bytes;
    return F2K_OK;
}

int f2k_hx_attach(f2k_hx* h, void* const* peer_bases) {
    if (!h || !h->valid || !peer_bases) return F2K_ERR_INVALID;
    for (int r = 0; r < h->cfg.world; ++r) {
        if (r == h->cfg.rank) continue;
        if (!peer_bases[r]) return fail(h, F2K_ERR_INVALID, "null peer buffer");
        h->peer[r] = static_cast<unsigned char*>(peer_bases[r]);
    }
    h->have_params[0] = h->have_params[1] = false;
    h->have_fparams[0] = h->have_fparams[1] = false;
    h->have_cparams[0] = h->have_cparams[1] = false;
    return F2K_OK;
}

int f2k_hx_exchange_in(f2k_hx* h, const void* q_raw, const void* k_raw, const void* v, const void* gamma_q,
                       const void* gamma_k, const float* cos_local, const float* sin_local, float eps,
                       void* stream) {
    if (!h || !h->valid) return F2K_ERR_INVALID;
    if (!q_raw || !k_raw || !v || !gamma_q || !gamma_k || !cos_local || !sin_local)
        return fail(h, F2K_ERR_INVALID, "null tensor pointer");
    for (const void* ptr : {q_raw, k_raw, v, gamma_q, gamma_k, static_cast<const void*>(cos_local),
                            static_cast<const void*>(sin_local)})
        if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0)
            return fail(h, F2K_ERR_INVALID, "tensor, gain and table pointers must be 16-byte aligned");
    const f2k_seqpar_config& c = h->cfg;
    for (int r = 0; r < c.world; ++r)
        if (!h->peer[r]) return fail(h, F2K_ERR_INVALID, "peers not attached");
    // The two buffer sets are safe to reuse only if every step is completed: the stream wait of
    // output() is what keeps this rank from overwriting a set its peers still write into.
    if (h->phase != f2k_hx::kIdle)
        return fail(h, F2K_ERR_INVALID, "exchange_in before the previous step's attend and output");
    h->epoch += 1;
    const int set = h->epoch & 1;
    QkvScatterParams p;
    std::memset(&p, 0, sizeof p);
    p.q = q_raw; p.k = k_raw; p.v = v;
    p.gamma_q = gamma_q; p.gamma_k = gamma_k;
    p.cos_tab = cos_local; p.sin_tab = sin_local;
    for (int r = 0; r < c.world; ++r) {
        p.dst_q[r] = h->part(h->peer[r], set, 0);
        p.dst_k[r] = h->part(h->peer[r], set, 1);
        p.dst_v[r] = h->part(h->peer[r], set, 2);
        p.flag[r]  = h->arrived(h->peer[r], set, c.rank);
    }
    p.counter = h->counter(0);
    p.value   = h->epoch;
    p.s_loc = c.seq_local; p.n_heads = c.n_heads; p.heads_per_rank = h->hpr; p.world = c.world; p.rank = c.rank;
    p.eps = eps;
    const cudaError_t e = qkv_scatter_launch(p, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail_cuda(h, "exchange kernel launch", e);
    h->phase = f2k_hx::kExchanged;
    h->copy_mode = false;
    return F2K_OK;
}

// The exchange with the copy engines doing the transfers: one prologue kernel normalises + rotates
// Q and K of ALL heads into a local staging area; then, per destination rank and on a stream of its
// own, three strided copies pick the destination's head columns of K, V (straight from the caller's
// tensor) and Q and put them into the destination's buffers, local or peer, followed by a stream
// write of the step number into the destination's "arrived" word for this source. Destinations are
// served nearest consumer first (rank - 1, rank - 2, ...); the rank's own heads go in on the caller's
// stream. Nothing occupies an SM after that, so the attention kernel, launched by attend() right behind it, runs while the
// copies are still on their way and waits, per source rank, for what it needs next.
int f2k_hx_exchange_in_copy(f2k_hx* h, const void* q_raw, const void* k_raw, const void* v, const void* gamma_q,
                            const void* gamma_k, const float* cos_local, const float* sin_local, float eps,
                            void* stream) {
    if (!h || !h->valid) return F2K_ERR_INVALID;
    if (!q_raw || !k_raw || !v || !gamma_q || !gamma_k || !cos_local || !sin_local)
        return fail(h, F2K_ERR_INVALID, "null tensor pointer");
    for (const void* ptr : {q_raw, k_raw, v, gamma_q, gamma_k, static_cast<const void*>(cos_local),
                            static_cast<const void*>(sin_local)})
        if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0)
            return fail(h, F2K_ERR_INVALID, "tensor, gain and table pointers must be 16-byte aligned");
    const f2k_seqpar_config& c = h->cfg;
    for (int r = 0; r < c.world; ++r)
        if (!h->peer[r]) return fail(h, F2K_ERR_INVALID, "peers not attached");
    if (h->phase != f2k_hx::kIdle)
        return fail(h, F2K_ERR_INVALID, "exchange_in before the previous step's attend and output");
    cudaError_t e = cudaSuccess;
    if (!h->stage) {                                   // first use: staging area, streams, event
        // Every copy stream needs a hardware queue of its own: a copy that shares a queue with the
        // caller's stream sits behind that stream's wait for the peers' "done" words, while the
        // peers wait for the copy. The CUDA default is 8 queues per device for all streams of the
        // process; more have to be asked for before the CUDA context exists.
        const char* mc = std::getenv("CUDA_DEVICE_MAX_CONNECTIONS");
        if (c.world > 1 && (!mc || std::atoi(mc) < c.world + 8))
            return fail(h, F2K_ERR_UNSUPPORTED,
                        "the copy-engine exchange needs CUDA_DEVICE_MAX_CONNECTIONS >= world + 8 in the environment "
                        "before CUDA is initialised (one hardware queue per copy stream)");
        e = cudaMalloc(reinterpret_cast<void**>(&h->stage), 2 * h->shard_bytes);
        for (int i = 0; i < c.world && e == cudaSuccess; ++i)
            e = cudaStreamCreateWithFlags(&h->copy_stream[i], cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->ev_prologue, cudaEventDisableTiming);
        if (e != cudaSuccess) return fail_cuda(h, "copy-engine exchange set-up", e);
    }
    h->epoch += 1;
    const int set = h->epoch & 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned char* qn = h->stage;
    unsigned char* kn = h->stage + h->shard_bytes;
    QkPrologueParams pp;
    std::memset(&pp, 0, sizeof pp);
    const long long rows = (long long)c.seq_local * c.n_heads;
    pp.job[0].x = q_raw; pp.job[0].y = qn; pp.job[0].gamma = gamma_q;
    pp.job[1].x = k_raw; pp.job[1].y = kn; pp.job[1].gamma = gamma_k;
    for (int j = 0; j < 2; ++j) {
        pp.job[j].cos_tab = cos_local; pp.job[j].sin_tab = sin_local; pp.job[j].seq = c.seq_local; pp.job[j].rows = rows;
    }
    pp.row_start[0] = 0; pp.row_start[1] = rows; pp.row_start[2] = 2 * rows;
    pp.n_jobs = 2; pp.n_heads = c.n_heads; pp.eps = eps;
    e = qk_prologue_launch(pp, s);
    if (e == cudaSuccess) e = cudaEventRecord(h->ev_prologue, s);
    if (e != cudaSuccess) return fail_cuda(h, "prologue launch", e);
    const size_t spitch = (size_t)c.n_heads * kHeadDim * 2;        // a token of all heads
    const size_t width  = (size_t)h->hpr * kHeadDim * 2;           // a token of one rank's heads
    const size_t seg_bytes = (size_t)c.seq_local * width;
    // The rank's own heads stay on this GPU and go in on the caller's stream, ahead of the
    // attention kernel: a same-device strided copy may run as a kernel, and a kernel queued on
    // another stream would find every SM taken by an attention kernel that waits for it.
    {
        QkPrologueParams po;
        std::memset(&po, 0, sizeof po);
        const long long own_rows = (long long)c.seq_local * h->hpr;
        const size_t col = (size_t)c.rank * width;
        po.job[0].x = static_cast<const unsigned char*>(q_raw) + col; po.job[0].gamma = gamma_q;
        po.job[0].y = h->part(h->buf, set, 0) + (size_t)c.rank * seg_bytes;
        po.job[1].x = static_cast<const unsigned char*>(k_raw) + col; po.job[1].gamma = gamma_k;
        po.job[1].y = h->part(h->buf, set, 1) + (size_t)c.rank * seg_bytes;
        for (int j = 0; j < 2; ++j) {
            po.job[j].x_tok_stride = (long long)c.n_heads * kHeadDim;
            po.job[j].cos_tab = cos_local; po.job[j].sin_tab = sin_local; po.job[j].seq = c.seq_local; po.job[j].rows = own_rows;
        }
        po.row_start[0] = 0; po.row_start[1] = own_rows; po.row_start[2] = 2 * own_rows;
        po.n_jobs = 2; po.n_heads = h->hpr; po.eps = eps;
        e = qk_prologue_launch(po, s);
        if (e == cudaSuccess)
            e = cudaMemcpy2DAsync(h->part(h->buf, set, 2) + (size_t)c.rank * seg_bytes, width,
                                  static_cast<const unsigned char*>(v) + col, spitch, width, (size_t)c.seq_local,
                                  cudaMemcpyDeviceToDevice, s);
        if (e != cudaSuccess) return fail_cuda(h, "own heads", e);
    }
    for (int i = 1; i < c.world; ++i) {
        const int d = (c.rank - i + c.world) % c.world;            // nearest consumer first
        cudaStream_t cs = h->copy_stream[i];
        e = cudaStreamWaitEvent(cs, h->ev_prologue, 0);
        const unsigned char* src[3] = {kn, static_cast<const unsigned char*>(v), qn};
        const int part_of[3] = {1, 2, 0};
        for (int t = 0; t < 3 && e == cudaSuccess; ++t)
            e = cudaMemcpy2DAsync(h->part(h->peer[d], set, part_of[t]) + (size_t)c.rank * seg_bytes, width,
                                  src[t] + (size_t)d * width, spitch, width, (size_t)c.seq_local,
                                  cudaMemcpyDeviceToDevice, cs);
        if (e != cudaSuccess) return fail_cuda(h, "exchange copy", e);
        if (h->write32(reinterpret_cast<CUstream>(cs), reinterpret_cast<CUdeviceptr>(h->arrived(h->peer[d], set, c.rank)),
                       h->epoch, 0) != CUDA_SUCCESS)
            return fail(h, F2K_ERR_CUDA, "cuStreamWriteValue32 failed");
    }
    h->phase = f2k_hx::kExchanged;
    h->copy_mode = true;
    return F2K_OK;
}

int f2k_hx_attend(f2k_hx* h, void* stream) {
    if (!h || !h->valid) return F2K_ERR_INVALID;
    if (h->phase != f2k_hx::kExchanged) return fail(h, F2K_ERR_INVALID, "attend without exchange_in");
    const f2k_seqpar_config& c = h->cfg;
    const int set = h->epoch & 1;
    // After the scatter kernel: segment s = the tokens of rank s, and the rank's own rows need no
    // wait (they come from the kernel just before on the same stream). After the copy-engine
    // exchange: ring order starting with the rank's own tokens (what is nearest arrives first), and
    // CTAs numbered head-fastest so that those of the first segments run first.
    const bool ring = h->copy_mode;
    AttnParams& p = ring ? h->cparams[set] : h->params[set];
    bool& have = ring ? h->have_cparams[set] : h->have_params[set];
    if (!have) {
        std::memset(&p, 0, sizeof p);
        const long long tok_h = (long long)h->hpr * kHeadDim;          // token stride of the head-sharded tensors
        const long long tok_o = (long long)c.n_heads * kHeadDim;       // token stride of the token-sharded output
        const int tiles_per_seg = (c.seq_local + kTileM - 1) / kTileM;
        const size_t seg_bytes = (size_t)c.seq_local * h->hpr * kHeadDim * 2;
        for (int s = 0; s < c.world; ++s) {
            const int src = ring ? (c.rank + s) % c.world : s;         // whose tokens segment s holds
            if (!encode(h, &p.tm_q[s], h->part(h->buf, set, 0) + src * seg_bytes, c.seq_local, h->hpr, tok_h) ||
                !encode(h, &p.tm_k[s], h->part(h->buf, set, 1) + src * seg_bytes, c.seq_local, h->hpr, tok_h) ||
                !encode(h, &p.tm_v[s], h->part(h->buf, set, 2) + src * seg_bytes, c.seq_local, h->hpr, tok_h))
                return fail(h, F2K_ERR_CUDA, "tensor map failed");
            // the output rows of the segment go to the rank that owns its tokens, into the columns of this rank's heads
            p.o_ptr[s] = h->part(h->peer[src], set, 3) + (size_t)c.rank * h->hpr * kHeadDim * 2;
            p.o_tok_stride[s]   = tok_o;
            p.o_batch_stride[s] = tok_o * c.seq_local;
            p.q_len[s] = p.kv_len[s] = c.seq_local;
            p.q_tile_start[s] = p.kv_tile_start[s] = s * tiles_per_seg;
            if (src != c.rank) p.q_ready[s] = p.kv_ready[s] = h->arrived(h->buf, set, src);
            p.done_flag[s] = h->done(h->peer[src], set, c.rank);
            p.fail_flag[s] = h->failed(h->peer[src], set, c.rank);
        }
        p.grid_head_fastest = ring ? 1 : 0;
        p.q_tile_start[c.world] = p.kv_tile_start[c.world] = c.world * tiles_per_seg;
        p.n_qseg = p.n_kvseg = c.world;
        p.n_q_tiles = p.n_kv_tiles = c.world * tiles_per_seg;
        if (!ring && c.world > 1) {
            // After the scatter kernel all sources arrive at about the same time and the segments
            // lie back to back in rank order: K/V are walked as ONE segment (no padded tile per
            // source), once every source's arrival word is there - the rank's own included, its
            // exchange kernel writes it too.
            const int all = c.world * c.seq_local;
            if (!encode(h, &p.tm_k[0], h->part(h->buf, set, 1), all, h->hpr, tok_h) ||
                !encode(h, &p.tm_v[0], h->part(h->buf, set, 2), all, h->hpr, tok_h))
                return fail(h, F2K_ERR_CUDA, "tensor map failed");
            for (int s = 0; s < c.world; ++s) { p.kv_ready[s] = nullptr; p.kv_len[s] = 0; p.kv_tile_start[s + 1] = 0; }
            p.kv_len[0] = all;
            p.kv_tile_start[0] = 0;
            p.kv_tile_start[1] = (all + kTileN - 1) / kTileN;
            p.n_kvseg = 1;
            p.n_kv_tiles = p.kv_tile_start[1];
            p.kv_ready[0] = h->arrived(h->buf, set, 0);
            p.kv_ready_words = c.world;
        }
        p.kv_ready_heads_per_group = h->hpr;                            // one word per source rank
        p.n_heads = h->hpr;
        p.batch = 1;
        p.scale_log2 = h->scale * 1.4426950408889634f;
        p.status = h->d_status;
        p.done_counter = h->counter(1);
        p.n_done = c.world;
        have = true;
    }
    p.kv_ready_value = h->epoch;
    p.done_value = h->epoch;
    p.wait_limit_clk      = h->wait_clk;
    p.peer_wait_limit_clk = h->peer_wait_clk;
    const cudaError_t e = attn_fwd_launch(p, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail_cuda(h, "attention launch", e);
    h->phase = f2k_hx::kAttended;
    return F2K_OK;
}

namespace {
// The chunk queue of the fused exchange. CTAs start in index order, head fastest, so the first
// `sms` of them hold the first 2 * ceil(sms / heads) query tiles in ring order: their Q rows go
// first, then the K/V of the first two ring steps, then the other Q rows (the CTAs that need them
// start a wave later), then K/V step by step - delivery is faster than the kernel's walk.
void fill_exchange_order(ExchangeParams& x, int world, int seq_local, int heads_per_rank, int sms) {
    const int n_sub = (seq_local + kExchangeTokens - 1) / kExchangeTokens;
    const int tiles_per_seg = (seq_local + kTileM - 1) / kTileM;
    const int first_tiles = std::min(2 * ((sms + heads_per_rank - 1) / heads_per_rank), world * tiles_per_seg);
    x.n_ranges = 0;
    x.total_chunks = 0;
    auto add = [&x](int kind, int step, int sub0, int n) {
        if (n <= 0) return;
        x.order[x.n_ranges++] = ExchangeRange{(short)kind, (short)step, sub0, n};
        x.total_chunks += (unsigned int)n;
    };
    int q_first[kMaxQSeg];
    for (int i = 0; i < world; ++i) {
        const int tiles = std::max(0, std::min(tiles_per_seg, first_tiles - i * tiles_per_seg));
        q_first[i] = std::min(n_sub, tiles * (kTileM / kExchangeTokens));
        add(0, i, 0, q_first[i]);
    }
    for (int i = 0; i < std::min(2, world); ++i) add(1, i, 0, n_sub);
    for (int i = 0; i < world; ++i) add(0, i, q_first[i], n_sub - q_first[i]);
    for (int i = 2; i < world; ++i) add(1, i, 0, n_sub);
}
}  // namespace

int f2k_hx_forward(f2k_hx* h, const void* q_raw, const void* k_raw, const void* v, const void* gamma_q,
                   const void* gamma_k, const float* cos_local, const float* sin_local, float eps, void* stream) {
    if (!h || !h->valid) return F2K_ERR_INVALID;
    if (!q_raw || !k_raw || !v || !gamma_q || !gamma_k || !cos_local || !sin_local)
        return fail(h, F2K_ERR_INVALID, "null tensor pointer");
    for (const void* ptr : {q_raw, k_raw, v, gamma_q, gamma_k, static_cast<const void*>(cos_local),
                            static_cast<const void*>(sin_local)})
        if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0)
            return fail(h, F2K_ERR_INVALID, "tensor, gain and table pointers must be 16-byte aligned");
    const f2k_seqpar_config& c = h->cfg;
    for (int r = 0; r < c.world; ++r)
        if (!h->peer[r]) return fail(h, F2K_ERR_INVALID, "peers not attached");
    if (h->phase != f2k_hx::kIdle)
        return fail(h, F2K_ERR_INVALID, "forward before the previous step's output");
    h->epoch += 1;
    const int set = h->epoch & 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    AttnParams& p = h->fparams[set];
    if (!h->have_fparams[set]) {
        std::memset(&p, 0, sizeof p);
        const long long tok_h = (long long)h->hpr * kHeadDim;          // token stride of the head-sharded tensors
        const long long tok_o = (long long)c.n_heads * kHeadDim;       // token stride of the token-sharded output
        const int tiles_per_seg = (c.seq_local + kTileM - 1) / kTileM;
        const size_t seg_bytes = (size_t)c.seq_local * h->hpr * kHeadDim * 2;
        for (int i = 0; i < c.world; ++i) {                            // segment i = the tokens of rank (rank + i) % world
            const int src = (c.rank + i) % c.world;
            if (!encode(h, &p.tm_q[i], h->part(h->buf, set, 0) + src * seg_bytes, c.seq_local, h->hpr, tok_h) ||
                !encode(h, &p.tm_k[i], h->part(h->buf, set, 1) + src * seg_bytes, c.seq_local, h->hpr, tok_h) ||
                !encode(h, &p.tm_v[i], h->part(h->buf, set, 2) + src * seg_bytes, c.seq_local, h->hpr, tok_h))
                return fail(h, F2K_ERR_CUDA, "tensor map failed");
            p.o_ptr[i] = h->part(h->peer[src], set, 3) + (size_t)c.rank * h->hpr * kHeadDim * 2;
            p.o_tok_stride[i]   = tok_o;
            p.o_batch_stride[i] = tok_o * c.seq_local;
            p.q_len[i] = p.kv_len[i] = c.seq_local;
            p.q_tile_start[i] = p.kv_tile_start[i] = i * tiles_per_seg;
            p.q_ready[i]  = h->tile_words(h->buf, set, src);            // own rows too: the exchange is part of this kernel
            p.kv_ready[i] = h->tile_words(h->buf, set, src) + h->n_tiles;
            p.done_flag[i] = h->done(h->peer[src], set, c.rank);
            p.fail_flag[i] = h->failed(h->peer[src], set, c.rank);
        }
        p.q_tile_start[c.world] = p.kv_tile_start[c.world] = c.world * tiles_per_seg;
        p.n_qseg = p.n_kvseg = c.world;
        p.n_q_tiles = p.n_kv_tiles = c.world * tiles_per_seg;
        // K/V: the sources' rows lie back to back in rank order, so the ring walk is two pieces of
        // the whole buffer, tokens [start, end) and [0, start) - one padded tile per piece instead
        // of one per source. Needs chunks that never straddle a tile of the walk.
        const bool walk = c.world > 1 && c.seq_local % kExchangeTokens == 0;
        if (walk) {
            const int all = c.world * c.seq_local, start = c.rank * c.seq_local;
            const size_t start_bytes = (size_t)start * h->hpr * kHeadDim * 2;
            const int len[2] = {all - start, start};
            const size_t off[2] = {start_bytes, 0};
            for (int i = 0; i < c.world; ++i) { p.kv_ready[i] = nullptr; p.kv_len[i] = 0; p.kv_tile_start[i + 1] = 0; }
            int n = 0, tiles = 0;
            for (int i = 0; i < 2; ++i) {
                if (len[i] == 0) continue;
                if (!encode(h, &p.tm_k[n], h->part(h->buf, set, 1) + off[i], len[i], h->hpr, tok_h) ||
                    !encode(h, &p.tm_v[n], h->part(h->buf, set, 2) + off[i], len[i], h->hpr, tok_h))
                    return fail(h, F2K_ERR_CUDA, "tensor map failed");
                p.kv_len[n] = len[i];
                p.kv_tile_start[n] = tiles;
                p.kv_ready[n] = h->walk_words(h->buf, set) + tiles;
                tiles += (len[i] + kTileN - 1) / kTileN;
                ++n;
            }
            p.kv_tile_start[n] = tiles;
            p.n_kvseg = n;
            p.n_kv_tiles = tiles;
        }
        p.kv_ready_heads_per_group = h->hpr;
        p.n_heads = h->hpr;
        p.batch = 1;
        p.scale_log2 = h->scale * 1.4426950408889634f;
        p.status = h->d_status;
        p.done_counter = h->counter(1);
        p.n_done = c.world;
        p.grid_head_fastest = 1;
        p.ready_per_tile = 1;
        ExchangeParams& x = p.xchg;
        for (int d = 0; d < c.world; ++d) {
            x.dst_q[d] = h->part(h->peer[d], set, 0);
            x.dst_k[d] = h->part(h->peer[d], set, 1);
            x.dst_v[d] = h->part(h->peer[d], set, 2);
            x.tile_words[d] = h->tile_words(h->peer[d], set, c.rank);
            x.kv_walk_words[d] = walk ? h->walk_words(h->peer[d], set) : nullptr;
        }
        x.next_chunk = h->next_chunk();
        x.s_loc = c.seq_local; x.n_heads_total = c.n_heads; x.heads_per_rank = h->hpr; x.world = c.world; x.rank = c.rank;
        x.unit_rows = 1;
        for (int r = 2; r <= 16; ++r)
            if (h->hpr % r == 0) x.unit_rows = r;
        x.tokens_per_buf = std::min(4, 16 / x.unit_rows);
        int sms = 148, dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        x.n_sms = (unsigned int)sms;
        fill_exchange_order(x, c.world, c.seq_local, h->hpr, sms);
        x.enabled = 1;
        h->have_fparams[set] = true;
    }
    p.kv_ready_value = h->epoch;
    p.done_value = h->epoch;
    p.wait_limit_clk      = h->wait_clk;
    p.peer_wait_limit_clk = h->peer_wait_clk;
    p.xchg.q = q_raw; p.xchg.k = k_raw; p.xchg.v = v;
    p.xchg.gamma_q = gamma_q; p.xchg.gamma_k = gamma_k;
    p.xchg.cos_tab = cos_local; p.xchg.sin_tab = sin_local;
    p.xchg.eps = eps;
    p.ready_uses = ++h->set_uses[set];
    cudaError_t e = cudaMemsetAsync(h->next_chunk(), 0, sizeof(unsigned int), s);   // the chunk queue starts at its head
    if (e != cudaSuccess) return fail_cuda(h, "cudaMemsetAsync(chunk counters)", e);
    e = attn_fwd_launch(p, s);
    if (e != cudaSuccess) return fail_cuda(h, "attention launch", e);
    h->phase = f2k_hx::kAttended;
    return F2K_OK;
}

int f2k_hx_exchange_plan(int world, int seq_local, int heads_per_rank, int n_sms, int* ranges, int max_ranges,
                         int* n_ranges) {
    if (world < 1 || world > kMaxQSeg || seq_local < 1 || heads_per_rank < 1 || n_sms < 1 || !n_ranges ||
        (!ranges && max_ranges > 0))
        return F2K_ERR_INVALID;
    ExchangeParams x;
    std::memset(&x, 0, sizeof x);
    fill_exchange_order(x, world, seq_local, heads_per_rank, n_sms);
    for (int i = 0; i < x.n_ranges && i < max_ranges; ++i) {
        ranges[4 * i + 0] = x.order[i].kind;
        ranges[4 * i + 1] = x.order[i].step;
        ranges[4 * i + 2] = x.order[i].sub0;
        ranges[4 * i + 3] = x.order[i].n;
    }
    *n_ranges = x.n_ranges;
    return F2K_OK;
}

int f2k_hx_kv_walk_tile(int world, int seq_local, int dst_rank, int token, int* tile) {
    if (world < 1 || world > kMaxQSeg || seq_local < 1 || dst_rank < 0 || dst_rank >= world || token < 0 ||
        token >= world * seq_local || !tile)
        return F2K_ERR_INVALID;
    *tile = kv_walk_tile(token, dst_rank * seq_local, world * seq_local);
    return F2K_OK;
}

int f2k_hx_output(f2k_hx* h, void** o_local, void* stream) {
    if (!h || !h->valid) return F2K_ERR_INVALID;
    if (h->phase != f2k_hx::kAttended) return fail(h, F2K_ERR_INVALID, "output without attend");
    const int set = h->epoch & 1;
    for (int s = 0; s < h->cfg.world; ++s)
        if (h->wait32(static_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(h->done(h->buf, set, s)), h->epoch,
                      0 /* CU_STREAM_WAIT_VALUE_GEQ */) != CUDA_SUCCESS)
            return fail(h, F2K_ERR_CUDA, "cuStreamWaitValue32 failed");
    if (o_local) *o_local = h->part(h->buf, set, 3);
    h->phase = f2k_hx::kIdle;
    return F2K_OK;
}

int f2k_hx_device_status(f2k_hx* h, int* status_out) {
    if (!h || !h->valid) return F2K_ERR_INVALID;
    int st = 0;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail_cuda(h, "cudaDeviceSynchronize", e);
    e = cudaMemcpy(&st, h->d_status, sizeof st, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail_cuda(h, "status read", e);
    if (st != 0) cudaMemset(h->d_status, 0, sizeof st);
    // did a peer give up during the last step? its kernel says so in this rank's control words
    if (h->epoch > 0 && h->fail_reported != h->epoch) {
        unsigned int words[8] = {};
        const int set = h->epoch & 1;
        e = cudaMemcpy(words, h->failed(h->buf, set, 0), sizeof words, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return fail_cuda(h, "status read", e);
        for (int s = 0; s < h->cfg.world; ++s)
            if (words[s] == h->epoch) st |= kStatusPeerFailed;
        if (st & kStatusPeerFailed) h->fail_reported = h->epoch;      // reported once, like the status word
    }
    if (h->aborted) {
        st |= kStatusAborted;
        h->aborted = false;
    }
    if (status_out) *status_out = st;
    if (st & kStatusAborted) return fail(h, F2K_ERR_DEVICE, "the step was aborted by the host: a peer never delivered");
    if (st & kStatusWaitExpired) return fail(h, F2K_ERR_DEVICE, "a bounded wait inside the attention kernel expired");
    if (st & kStatusPeerFailed)
        return fail(h, F2K_ERR_DEVICE, "a peer's attention kernel gave up: some heads of this rank's output rows are stale");
    return F2K_OK;
}

int f2k_hx_set_wait_limits(f2k_hx* h, long long in_cta_clk, long long peer_clk) {
    if (!h || !h->valid) return F2K_ERR_INVALID;
    if (in_cta_clk < 0 || peer_clk < 0) return fail(h, F2K_ERR_INVALID, "wait limits must not be negative");
    h->wait_clk = in_cta_clk;
    h->peer_wait_clk = peer_clk;
    return F2K_OK;
}

// output() parks the stream on waits for every rank's "done" word. If a peer is gone the words
// never come. This writes them for the current step from the host side, on a stream of its own,
// so that the parked waits fall through; the step's output is invalid and device_status reports
// F2K_ERR_DEVICE once. Does not synchronise with the caller's stream.
int f2k_hx_abort(f2k_hx* h) {
    if (!h || !h->valid) return F2K_ERR_INVALID;
    if (h->epoch == 0) return F2K_OK;
    const int set = h->epoch & 1;
    for (int s = 0; s < h->cfg.world; ++s)
        if (h->write32(reinterpret_cast<CUstream>(h->abort_stream), reinterpret_cast<CUdeviceptr>(h->done(h->buf, set, s)),
                       h->epoch, 0) != CUDA_SUCCESS)
            return fail(h, F2K_ERR_CUDA, "cuStreamWriteValue32 failed");
    const cudaError_t e = cudaStreamSynchronize(h->abort_stream);
    if (e != cudaSuccess) return fail_cuda(h, "abort stream", e);
    h->aborted = true;
    h->phase = f2k_hx::kIdle;
    return F2K_OK;
}

}  // extern "C"
