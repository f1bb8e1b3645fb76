// Sequence-parallel joint attention across the GPUs of one NVLink/NVSwitch box as an all-gather of
// the K/V shards by pull (peers are visited in ring order; nothing rotates), and the stand-alone
// entry point of the QK prologue kernel it uses.
//
// The reference has no multi-GPU code at all (one process, one GPU, batch 1); this layer is new.
// Tokens are sharded by rank: rank r holds Q, K, V of its `seq_local` tokens. Every rank needs
// every other rank's K and V. Each rank owns ONE device allocation:
//
//     [2 sets][world slots] { K shard, V shard } | control words
//
// A rank writes its own normalised K and its V into slot `rank` of the current set (the set
// alternates from call to call) and calls forward(). No collective runs inside a step:
//
//  * forward() launches the attention kernel at once on the compute stream, with one key/value
//    segment per rank: its own first, then rank+1, rank+2, ... The kernel needs nothing remote
//    for its first segment.
//  * On the copy stream the rank tells every peer "my slot of this set is written" (a 32-bit
//    stream write into the peer's allocation), then, peer by peer in the same ring order, waits
//    for that peer's word (a stream wait on local memory), pulls the peer's slot into its own
//    allocation with the COPY ENGINES (no SMs) and writes an arrival word. K and V of a slot are
//    adjacent, so one copy moves both: a copy costs about 10 us on top of its bytes, and copies
//    of one stream pair do not run side by side, so fewer and larger copies win.
//  * When the kernel is the longer leg, pulls go head group by head group (all peers for the
//    heads of the first wave of CTAs, then the next wave's heads; one 3-D copy takes a group's
//    columns of K and V): CTAs are dispatched head-major, so what a CTA needs arrives before it
//    gets there. When the transfer is the longer leg a slot moves whole, in one linear copy.
//  * The kernel's TMA producer waits (bounded) on the arrival word of (segment, head group)
//    before the first tile of a remote segment. Remote data is only ever read from local
//    memory by ordinary single-CTA TMA loads, and nothing waits on another kernel.
//
// With overlap off the compute stream waits for all pulls before the kernel starts.
//
// Two sets: a rank may write the next call's K/V while slower peers still pull the current set.
// A peer's "written" word for call n+1 is sent after its kernel of call n (stream order), and a
// kernel cannot finish before its pulls have landed, so when this rank's kernel of call n+1 is
// done every peer has finished pulling set n from it, and call n+2 may overwrite it.

#include "f2k_attn.h"

#include "attn_launch.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

namespace {
using namespace f2k;
constexpr size_t kAlign = 256;
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);
using WriteValue32Fn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);

void* driver_fn(const char* name) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
        return nullptr;
    return p;
}
}  // namespace

struct f2k_seqpar {
    f2k_seqpar_config cfg{};
    float  scale = 0.f;
    bool   valid = false;
    std::string err;
    unsigned char* buf = nullptr;       // the allocation described above
    size_t shard_bytes = 0, set_bytes = 0, total_bytes = 0, flags_off = 0;
    using WaitValue32Fn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
    WaitValue32Fn wait32 = nullptr;
    cudaEvent_t written = nullptr;      // compute stream -> copy stream: this rank's K/V are in place
    cudaStream_t own_copy_stream = nullptr;   // used when the caller passes no copy stream
    static constexpr int kMaxGroups = 8;
    int*   d_status = nullptr;
    std::vector<unsigned char*> peer;   // base of every rank's allocation as mapped here
    unsigned int epoch = 0;             // call counter; arrival words carry it
    cudaEvent_t pulled = nullptr;
    EncodeTiledFn  encode = nullptr;
    WriteValue32Fn write32 = nullptr;

    long long wait_clk = 0, peer_wait_clk = 0;   // 0 = the defaults of attn_params.h
    bool aborted = false;               // f2k_seqpar_abort released the stream waits of the current step
    cudaStream_t abort_stream = nullptr;

    bool peer_write32 = true;           // stream writes straight into a peer's words work here
    unsigned char* k_slot(unsigned char* base, int set, int slot) const {
        return base + ((size_t)set * cfg.world + slot) * 2 * shard_bytes;
    }
    unsigned char* v_slot(unsigned char* base, int set, int slot) const {
        return k_slot(base, set, slot) + shard_bytes;      // V directly behind K: one copy moves both
    }
    // control words (uint32), all inside this rank's allocation so that peers can reach them:
    //   arrival[set][slot][group]  written locally after a pull        (2 * world * 8 words)
    //   ready[set][peer]           written by `peer` into THIS buffer  (2 * world words)
    //   epoch_word                 source of the 4-byte "written" copies (1 word)
    unsigned int* arrival(int set, int slot) const {
        return reinterpret_cast<unsigned int*>(buf + flags_off) + ((size_t)set * cfg.world + slot) * kMaxGroups;
    }
    static size_t ready_index(int world, int set, int peer) {
        return (size_t)2 * world * kMaxGroups + (size_t)set * world + peer;
    }
    unsigned int* ready(unsigned char* base, int set, int peer) const {
        return reinterpret_cast<unsigned int*>(base + flags_off) + ready_index(cfg.world, set, peer);
    }
    unsigned int* epoch_word() const {
        return reinterpret_cast<unsigned int*>(buf + flags_off) + (size_t)2 * cfg.world * kMaxGroups + (size_t)2 * cfg.world;
    }
};

namespace {
int fail(f2k_seqpar* h, int code, std::string msg) {
    h->err = std::move(msg);
    return code;
}
int fail_cuda(f2k_seqpar* h, const char* what, cudaError_t e) {
    return fail(h, F2K_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}
bool encode(f2k_seqpar* h, CUtensorMap* map, const void* base, int len) {
    const f2k_seqpar_config& c = h->cfg;
    const cuuint64_t tok = (cuuint64_t)c.n_heads * kHeadDim;
    const cuuint64_t dims[4]    = {(cuuint64_t)kHeadDim, (cuuint64_t)c.n_heads, (cuuint64_t)len, (cuuint64_t)c.batch};
    const cuuint64_t strides[3] = {(cuuint64_t)kHeadDim * 2, tok * 2, tok * (cuuint64_t)len * 2};
    const cuuint32_t box[4]     = {64, 1, (cuuint32_t)kTileM, 1};
    const cuuint32_t estr[4]    = {1, 1, 1, 1};
    return h->encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace

extern "C" {

int f2k_seqpar_create(const f2k_seqpar_config* cfg, f2k_seqpar** out) {
    if (!out) return F2K_ERR_INVALID;
    *out = nullptr;
    f2k_seqpar* h = new (std::nothrow) f2k_seqpar();
    if (!h) return F2K_ERR_CUDA;
    *out = h;
    if (!cfg) return fail(h, F2K_ERR_INVALID, "null config");
    h->cfg = *cfg;
    if (cfg->batch <= 0 || cfg->seq_local <= 0 || cfg->n_heads <= 0 || cfg->head_dim <= 0)
        return fail(h, F2K_ERR_INVALID, "sequence-parallel attention: zero/negative dim");
    if (cfg->world <= 0 || cfg->world > kMaxKvSeg || cfg->rank < 0 || cfg->rank >= cfg->world)
        return fail(h, F2K_ERR_INVALID, "sequence-parallel attention: world must be 1..8 and 0 <= rank < world");
    if (cfg->head_dim != kHeadDim) return fail(h, F2K_ERR_UNSUPPORTED, "head_dim must be 128");
    h->scale = cfg->scale > 0.f ? cfg->scale : 1.0f / std::sqrt((float)cfg->head_dim);
    h->shard_bytes = (size_t)cfg->batch * cfg->seq_local * cfg->n_heads * kHeadDim * 2;   // a multiple of 256
    h->set_bytes   = (size_t)cfg->world * h->shard_bytes;
    h->flags_off   = 4 * h->set_bytes;
    h->total_bytes = h->flags_off +
                     align_up(((size_t)2 * cfg->world * (f2k_seqpar::kMaxGroups + 1) + 1) * sizeof(unsigned int), kAlign);

    int dev = 0, major = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail_cuda(h, "cudaGetDevice", e);
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return fail_cuda(h, "cudaDeviceGetAttribute", e);
    if (major != 10) return fail(h, F2K_ERR_UNSUPPORTED, "this library contains sm_100a code only");
    h->encode  = reinterpret_cast<EncodeTiledFn>(driver_fn("cuTensorMapEncodeTiled"));
    h->write32 = reinterpret_cast<WriteValue32Fn>(driver_fn("cuStreamWriteValue32"));
    h->wait32  = reinterpret_cast<f2k_seqpar::WaitValue32Fn>(driver_fn("cuStreamWaitValue32"));
    if (!h->encode || !h->write32 || !h->wait32) return fail(h, F2K_ERR_CUDA, "driver entry points unavailable");
    e = attn_fwd_prepare();           // code is loaded now, never under a pending stream wait
    if (e == cudaSuccess) e = qk_prologue_prepare();
    if (e != cudaSuccess) return fail_cuda(h, "kernel load", e);
    e = cudaMalloc(reinterpret_cast<void**>(&h->buf), h->total_bytes);
    if (e != cudaSuccess) return fail_cuda(h, "cudaMalloc(shards)", e);
    e = cudaMemset(h->buf + h->flags_off, 0, h->total_bytes - h->flags_off);
    if (e != cudaSuccess) return fail_cuda(h, "cudaMemset(flags)", e);
    e = cudaMalloc(reinterpret_cast<void**>(&h->d_status), kStatusBytes);
    if (e == cudaSuccess) e = cudaMemset(h->d_status, 0, kStatusBytes);
    if (e != cudaSuccess) return fail_cuda(h, "cudaMalloc(status)", e);
    e = cudaEventCreateWithFlags(&h->pulled, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->written, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->own_copy_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->abort_stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) return fail_cuda(h, "cudaEventCreate/cudaStreamCreate", e);
    h->peer.assign(cfg->world, nullptr);
    h->peer[cfg->rank] = h->buf;
    h->valid = true;
    return F2K_OK;
}

void f2k_seqpar_destroy(f2k_seqpar* h) {
    if (!h) return;
    if (h->pulled) cudaEventDestroy(h->pulled);
    if (h->written) cudaEventDestroy(h->written);
    if (h->own_copy_stream) cudaStreamDestroy(h->own_copy_stream);
    if (h->abort_stream) cudaStreamDestroy(h->abort_stream);
    if (h->d_status) cudaFree(h->d_status);
    if (h->buf) cudaFree(h->buf);
    delete h;
}

const char* f2k_seqpar_last_error(const f2k_seqpar* h) { return h ? h->err.c_str() : "no handle"; }

int f2k_seqpar_buffer(f2k_seqpar* h, void** base, size_t* bytes) {
    if (!h || !h->valid) return F2K_ERR_INVALID;
    if (base) *base = h->buf;
    if (bytes) *bytes = h->total_bytes;
    return F2K_OK;
}

int f2k_seqpar_attach(f2k_seqpar* h, void* const* peer_bases) {
    if (!h || !h->valid || !peer_bases) return F2K_ERR_INVALID;
    for (int r = 0; r < h->cfg.world; ++r) {
        if (r == h->cfg.rank) continue;
        if (!peer_bases[r]) return fail(h, F2K_ERR_INVALID, "null peer buffer");
        h->peer[r] = static_cast<unsigned char*>(peer_bases[r]);
    }
    return F2K_OK;
}

int f2k_seqpar_local_kv(f2k_seqpar* h, void** k, void** v) {
    if (!h || !h->valid) return F2K_ERR_INVALID;
    const int set = (h->epoch + 1) & 1;   // the set the NEXT forward call reads
    if (k) *k = h->k_slot(h->buf, set, h->cfg.rank);
    if (v) *v = h->v_slot(h->buf, set, h->cfg.rank);
    return F2K_OK;
}

int f2k_seqpar_forward(f2k_seqpar* h, const void* q_local, void* o_local, int overlap,
                       void* compute_stream, void* copy_stream) {
    if (!h || !h->valid) return F2K_ERR_INVALID;
    if (!q_local || !o_local) return fail(h, F2K_ERR_INVALID, "null tensor pointer");
    if ((reinterpret_cast<uintptr_t>(q_local) & 15u) || (reinterpret_cast<uintptr_t>(o_local) & 15u))
        return fail(h, F2K_ERR_INVALID, "q_local and o_local must be 16-byte aligned");
    const f2k_seqpar_config& c = h->cfg;
    for (int r = 0; r < c.world; ++r)
        if (!h->peer[r]) return fail(h, F2K_ERR_INVALID, "peers not attached");
    h->epoch += 1;
    const int set = h->epoch & 1;
    cudaStream_t cs = static_cast<cudaStream_t>(compute_stream);
    cudaStream_t ps = copy_stream ? static_cast<cudaStream_t>(copy_stream) : h->own_copy_stream;
    if (c.world > 1 && ps == cs && overlap)
        return fail(h, F2K_ERR_INVALID, "overlap needs a copy stream different from the compute stream");

    AttnParams p;
    std::memset(&p, 0, sizeof p);
    const long long tok = (long long)c.n_heads * kHeadDim;
    if (!encode(h, &p.tm_q[0], q_local, c.seq_local)) return fail(h, F2K_ERR_CUDA, "tensor map (Q) failed");
    p.o_ptr[0] = o_local;
    p.o_tok_stride[0] = tok;
    p.o_batch_stride[0] = tok * c.seq_local;
    p.q_len[0] = c.seq_local;
    const int tiles_per_seg = (c.seq_local + kTileM - 1) / kTileM;
    p.q_tile_start[0] = 0;
    p.q_tile_start[1] = tiles_per_seg;
    p.n_qseg = 1;
    p.n_q_tiles = tiles_per_seg;

    // Head groups. If the kernel is clearly the longer leg: as many groups as it has waves of
    // CTAs (a power of two that divides the head count, at most 8, copies of 8 MB or more), so
    // that the heads of the first wave arrive first. If the transfer is: whole slots.
    int groups = 1;
    if (overlap && c.world > 1) {
        int sms = 148;
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const long long ctas = (long long)((tiles_per_seg + 1) / 2) * c.n_heads * c.batch;
        const long long waves = (ctas + sms - 1) / sms;
        const double s_all = (double)c.seq_local * c.world;
        const double t_kernel = 4.0 * c.batch * c.n_heads * c.seq_local * s_all * kHeadDim / 1.1e15;
        const double t_copy = (c.world - 1) * (2.0 * h->shard_bytes / 7.4e11 + 10e-6);
        if (t_copy < 0.85 * t_kernel)
            while (groups < waves && groups < f2k_seqpar::kMaxGroups && c.n_heads % (groups * 2) == 0 &&
                   2 * h->shard_bytes / (groups * 2) >= ((size_t)8 << 20))
                groups *= 2;
        if (const char* env = std::getenv("F2K_SEQPAR_GROUPS")) {       // measurement knob
            const int g = std::atoi(env);
            if (g >= 1 && g <= f2k_seqpar::kMaxGroups && c.n_heads % g == 0) groups = g;
        }
    }
    const int hpg = c.n_heads / groups;

    // key/value segment i of the kernel is rank (rank + i) % world
    for (int i = 0; i < c.world; ++i) {
        const int src = (c.rank + i) % c.world;
        if (!encode(h, &p.tm_k[i], h->k_slot(h->buf, set, src), c.seq_local) ||
            !encode(h, &p.tm_v[i], h->v_slot(h->buf, set, src), c.seq_local))
            return fail(h, F2K_ERR_CUDA, "tensor map (K/V) failed");
        p.kv_len[i] = c.seq_local;
        p.kv_tile_start[i] = i * tiles_per_seg;
        if (i > 0 && overlap) p.kv_ready[i] = h->arrival(set, src);
    }
    p.kv_tile_start[c.world] = c.world * tiles_per_seg;
    p.n_kvseg = c.world;
    p.n_kv_tiles = c.world * tiles_per_seg;
    p.kv_ready_value = h->epoch;
    p.kv_ready_heads_per_group = hpg;
    p.n_heads = c.n_heads;
    p.batch = c.batch;
    p.scale_log2 = h->scale * 1.4426950408889634f;
    p.status = h->d_status;
    p.wait_limit_clk      = h->wait_clk;
    p.peer_wait_limit_clk = h->peer_wait_clk;

    if (c.world > 1) {
        const cudaError_t we = cudaEventRecord(h->written, cs);   // everything before this call on cs: K/V written
        if (we != cudaSuccess) return fail_cuda(h, "event", we);
    }
    // With overlap the kernel goes first: its first segment is local, and the host then queues
    // the pulls while the kernel is already running.
    bool launched = false;
    if (overlap || c.world == 1) {
        const cudaError_t le = attn_fwd_launch(p, cs);
        if (le != cudaSuccess) return fail_cuda(h, "attention launch", le);
        launched = true;
    }
    if (c.world > 1) {
        // (1) the copy stream may go once this rank's K/V are in place (event recorded above,
        //     before the kernel launch)
        cudaError_t e = cudaStreamWaitEvent(ps, h->written, 0);
        if (e != cudaSuccess) return fail_cuda(h, "event", e);
        // (2) tell every peer: the call number goes into the peer's allocation, by a stream write
        //     where the driver takes a peer address for one, else by a 4-byte copy
        if (h->write32(reinterpret_cast<CUstream>(ps), reinterpret_cast<CUdeviceptr>(h->epoch_word()), h->epoch, 0) != CUDA_SUCCESS)
            return fail(h, F2K_ERR_CUDA, "cuStreamWriteValue32 failed");
        for (int i = 1; i < c.world; ++i) {
            const int dstr = (c.rank + i) % c.world;
            unsigned int* word = h->ready(h->peer[dstr], set, c.rank);
            if (h->peer_write32 &&
                h->write32(reinterpret_cast<CUstream>(ps), reinterpret_cast<CUdeviceptr>(word), h->epoch, 0) != CUDA_SUCCESS)
                h->peer_write32 = false;
            if (!h->peer_write32) {
                e = cudaMemcpyAsync(word, h->epoch_word(), sizeof(unsigned int), cudaMemcpyDeviceToDevice, ps);
                if (e != cudaSuccess) return fail_cuda(h, "peer notify", e);
            }
        }
        // (3) pulls: head group by head group, peers in ring order; K and V in one copy
        const size_t pitch = (size_t)c.n_heads * kHeadDim * 2;
        const size_t width = (size_t)hpg * kHeadDim * 2;
        const size_t rows  = (size_t)c.batch * c.seq_local;
        for (int g = 0; g < groups; ++g) {
            for (int i = 1; i < c.world; ++i) {
                const int src = (c.rank + i) % c.world;
                if (g == 0 &&
                    h->wait32(reinterpret_cast<CUstream>(ps), reinterpret_cast<CUdeviceptr>(h->ready(h->buf, set, src)),
                              h->epoch, 0 /* CU_STREAM_WAIT_VALUE_GEQ */) != CUDA_SUCCESS)
                    return fail(h, F2K_ERR_CUDA, "cuStreamWaitValue32 failed");
                unsigned char* dst_k = h->k_slot(h->buf, set, src);
                unsigned char* src_k = h->k_slot(h->peer[src], set, src);
                if (groups == 1) {
                    e = cudaMemcpyAsync(dst_k, src_k, 2 * h->shard_bytes, cudaMemcpyDeviceToDevice, ps);
                } else {
                    // columns [g * width, (g + 1) * width) of every token row, planes K and V
                    cudaMemcpy3DParms cp;
                    std::memset(&cp, 0, sizeof cp);
                    cp.srcPtr = make_cudaPitchedPtr(src_k + (size_t)g * width, pitch, width, rows);
                    cp.dstPtr = make_cudaPitchedPtr(dst_k + (size_t)g * width, pitch, width, rows);
                    cp.extent = make_cudaExtent(width, rows, 2);
                    cp.kind   = cudaMemcpyDeviceToDevice;
                    e = cudaMemcpy3DAsync(&cp, ps);
                }
                if (e != cudaSuccess) return fail_cuda(h, "peer copy", e);
                if (h->write32(reinterpret_cast<CUstream>(ps), reinterpret_cast<CUdeviceptr>(h->arrival(set, src) + g),
                               h->epoch, 0) != CUDA_SUCCESS)
                    return fail(h, F2K_ERR_CUDA, "cuStreamWriteValue32 failed");
            }
        }
        if (!overlap) {
            e = cudaEventRecord(h->pulled, ps);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(cs, h->pulled, 0);
            if (e != cudaSuccess) return fail_cuda(h, "event", e);
        }
    }
    if (!launched) {
        const cudaError_t le = attn_fwd_launch(p, cs);
        if (le != cudaSuccess) return fail_cuda(h, "attention launch", le);
    }
    return F2K_OK;
}

int f2k_seqpar_device_status(f2k_seqpar* h, int* status_out) {
    if (!h || !h->valid) return F2K_ERR_INVALID;
    int st = 0;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail_cuda(h, "cudaDeviceSynchronize", e);
    e = cudaMemcpy(&st, h->d_status, sizeof st, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail_cuda(h, "status read", e);
    if (st != 0) cudaMemset(h->d_status, 0, sizeof st);
    if (h->aborted) {
        st |= kStatusAborted;
        h->aborted = false;
    }
    if (status_out) *status_out = st;
    if (st & kStatusAborted)
        return fail(h, F2K_ERR_DEVICE, "the step was aborted by the host: a peer never announced its K/V");
    if (st != 0) return fail(h, F2K_ERR_DEVICE, "a bounded wait inside the attention kernel expired");
    return F2K_OK;
}

int f2k_seqpar_set_wait_limits(f2k_seqpar* h, long long in_cta_clk, long long peer_clk) {
    if (!h || !h->valid) return F2K_ERR_INVALID;
    if (in_cta_clk < 0 || peer_clk < 0) return fail(h, F2K_ERR_INVALID, "wait limits must not be negative");
    h->wait_clk = in_cta_clk;
    h->peer_wait_clk = peer_clk;
    return F2K_OK;
}

// The copy stream of a step is parked on stream waits for the peers' "written" words. If a peer is
// gone those words never come, and neither the stream nor anything that synchronises with it
// (device_status, destroy) would return. This writes the awaited words of the current step from the
// host side, on a stream of its own, so that the parked waits fall through: the pulls then copy
// whatever the peers' slots hold (mapped memory, stale values) and the arrival words are written.
// The step's output is invalid; device_status reports F2K_ERR_DEVICE once. Does not synchronise
// with the compute or copy stream.
int f2k_seqpar_abort(f2k_seqpar* h) {
    if (!h || !h->valid) return F2K_ERR_INVALID;
    if (h->epoch == 0) return F2K_OK;            // nothing was ever queued
    const int set = h->epoch & 1;
    for (int r = 0; r < h->cfg.world; ++r) {
        if (r == h->cfg.rank) continue;
        if (h->write32(reinterpret_cast<CUstream>(h->abort_stream),
                       reinterpret_cast<CUdeviceptr>(h->ready(h->buf, set, r)), h->epoch, 0) != CUDA_SUCCESS)
            return fail(h, F2K_ERR_CUDA, "cuStreamWriteValue32 failed");
    }
    const cudaError_t e = cudaStreamSynchronize(h->abort_stream);
    if (e != cudaSuccess) return fail_cuda(h, "abort stream", e);
    h->aborted = true;
    return F2K_OK;
}

// ---- CUDA IPC helpers (one process per GPU: the allocation of a rank, mapped into its peers) ----
int f2k_ipc_export(const void* base, void* handle64) {
    if (!base || !handle64) return F2K_ERR_INVALID;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t hd;
    if (cudaIpcGetMemHandle(&hd, const_cast<void*>(base)) != cudaSuccess) return F2K_ERR_CUDA;
    std::memcpy(handle64, &hd, 64);
    return F2K_OK;
}
int f2k_ipc_open(const void* handle64, void** base) {
    if (!handle64 || !base) return F2K_ERR_INVALID;
    cudaIpcMemHandle_t hd;
    std::memcpy(&hd, handle64, 64);
    return cudaIpcOpenMemHandle(base, hd, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? F2K_OK : F2K_ERR_CUDA;
}
int f2k_ipc_close(void* base) {
    if (!base) return F2K_ERR_INVALID;
    return cudaIpcCloseMemHandle(base) == cudaSuccess ? F2K_OK : F2K_ERR_CUDA;
}

// ---- the prologue kernel on its own: y = RoPE(RMSNorm(x) * gamma), position = token index ----
int f2k_qk_norm_rope_bf16(const void* x, void* y, const void* gamma, const float* cos_table,
                          const float* sin_table, int batch, int seq, int n_heads, float eps, void* stream) {
    if (!x || !y || !gamma || !cos_table || !sin_table) return F2K_ERR_INVALID;
    if (batch <= 0 || seq <= 0 || n_heads <= 0) return F2K_ERR_INVALID;
    for (const void* ptr : {x, static_cast<const void*>(y), gamma, static_cast<const void*>(cos_table),
                            static_cast<const void*>(sin_table)})
        if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0) return F2K_ERR_INVALID;   // the kernel uses 16-byte accesses
    QkPrologueParams pp;
    std::memset(&pp, 0, sizeof pp);
    pp.job[0].x = x; pp.job[0].y = y; pp.job[0].gamma = gamma;
    pp.job[0].cos_tab = cos_table; pp.job[0].sin_tab = sin_table; pp.job[0].seq = seq;
    pp.job[0].rows = (long long)batch * seq * n_heads;
    pp.row_start[0] = 0; pp.row_start[1] = pp.job[0].rows;
    pp.n_jobs = 1; pp.n_heads = n_heads; pp.eps = eps;
    return qk_prologue_launch(pp, static_cast<cudaStream_t>(stream)) == cudaSuccess ? F2K_OK : F2K_ERR_CUDA;
}

}  // extern "C"
