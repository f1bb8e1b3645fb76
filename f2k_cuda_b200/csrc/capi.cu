// Implementation of the C ABI declared in include/f2k_attn.h: argument checking,
// TMA tensor-map construction, workspace carving and kernel launches. Everything that
// touches the GPU lives in the kernels (attn_fwd_sm100.cu, qk_prologue.cu); there is
// no CPU path here and none is reachable from these entry points.

#include "f2k_attn.h"

#include "attn_launch.h"

#include <algorithm>
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

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The kernels read Q, K, gains and tables with 16-byte loads: a pointer that is not 16-byte aligned
// would be a misaligned-address fault on the GPU, so it is refused here, before any launch.
inline bool misaligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }

// The driver entry point is fetched through the runtime so that the library carries no
// link-time dependency on libcuda.
EncodeTiledFn encode_tiled_fn(std::string& err) {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
        err = std::string("cuTensorMapEncodeTiled unavailable: ") + cudaGetErrorString(e);
        return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
    return fn;
}

// One segment: bf16 [batch, len, heads, 128], token stride and batch stride in elements.
bool encode_segment(CUtensorMap* map, const void* base, int len, int heads, int batch,
                    long long tok_stride, long long batch_stride, std::string& err) {
    EncodeTiledFn fn = encode_tiled_fn(err);
    if (!fn) return false;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) {
        err = "tensor base pointer is not 16-byte aligned";
        return false;
    }
    const cuuint64_t dims[4]    = {(cuuint64_t)kHeadDim, (cuuint64_t)heads, (cuuint64_t)len,
                                   (cuuint64_t)batch};
    const cuuint64_t strides[3] = {(cuuint64_t)kHeadDim * 2, (cuuint64_t)tok_stride * 2,
                                   (cuuint64_t)batch_stride * 2};
    const cuuint32_t box[4]     = {64, 1, (cuuint32_t)kTileM, 1};
    const cuuint32_t estr[4]    = {1, 1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims,
                          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char buf[96];
        std::snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed (CUresult %d)", (int)r);
        err = buf;
        return false;
    }
    return true;
}

}  // namespace

struct f2k_attn {
    f2k_attn_config cfg{};
    float           scale = 0.f;
    bool            valid = false;
    std::string     err;
    int             device = -1;
    int*            d_status = nullptr;
    long long       wait_clk = 0, peer_wait_clk = 0;   // 0 = the defaults of attn_params.h

    // Descriptors of the last forward call; rebuilt only when a pointer changes.
    const void* last_in[6] = {};
    void*       last_out[2] = {};
    long long   last_vo[4] = {};
    bool        have_params = false;
    AttnParams  params;

    // Host-buffer entry point: device staging, and the pipeline that overlaps the transfers of
    // one head group with the kernels of another (children: one handle per head group, each for
    // n_heads / groups heads; two extra streams, one per transfer direction).
    void*  stage = nullptr;
    size_t stage_bytes = 0;
    std::vector<f2k_attn*>   child;
    std::vector<AttnParams>  chunk_params;   // batch 1: one launch per chunk of query rows
    cudaEvent_t  ev_k = nullptr, ev_v = nullptr;
    std::vector<cudaEvent_t> arrived, computed;
    cudaStream_t s_in = nullptr, s_out = nullptr;
    cudaEvent_t  ev_start = nullptr, ev_out = nullptr;

    size_t bytes_txt() const {
        return (size_t)cfg.batch * cfg.seq_txt * cfg.n_heads * cfg.head_dim * 2;
    }
    size_t bytes_img() const {
        return (size_t)cfg.batch * cfg.seq_img * cfg.n_heads * cfg.head_dim * 2;
    }
    size_t fused_ws() const { return 2 * align_up(bytes_txt(), kAlign) + 2 * align_up(bytes_img(), kAlign); }
};

namespace {

int fail(f2k_attn* h, int code, std::string msg) {
    h->err = std::move(msg);
    return code;
}
int fail_cuda(f2k_attn* h, const char* what, cudaError_t e) {
    return fail(h, F2K_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

// token strides in elements; 0 = dense (heads * 128)
struct QSeg  { const void* q; void* o; int len; long long q_stride = 0, o_stride = 0; };
struct KvSeg { const void* k; const void* v; int len; long long k_stride = 0, v_stride = 0; };

// Launch parameters for attention of the given query segments over the given key/value segments;
// every segment is bf16 [batch, len, heads, 128], dense.
int build_params(f2k_attn* h, AttnParams& p, const QSeg* qs, int nq, const KvSeg* kvs, int nkv) {
    const f2k_attn_config& c = h->cfg;
    std::memset(&p, 0, sizeof p);
    const long long tok = (long long)c.n_heads * kHeadDim;
    if (nq < 1 || nq > kMaxQSeg || nkv < 1 || nkv > kMaxKvSeg) return fail(h, F2K_ERR_INVALID, "segment count");
    int tiles = 0;
    for (int s = 0; s < nq; ++s) {
        const QSeg& g = qs[s];
        if (!g.q || !g.o) return fail(h, F2K_ERR_INVALID, "null tensor pointer");
        if ((reinterpret_cast<uintptr_t>(g.o) & 15u) != 0)
            return fail(h, F2K_ERR_INVALID, "output pointer is not 16-byte aligned");
        const long long qs_ = g.q_stride ? g.q_stride : tok, os_ = g.o_stride ? g.o_stride : tok;
        if (!encode_segment(&p.tm_q[s], g.q, g.len, c.n_heads, c.batch, qs_, (long long)g.len * qs_, h->err))
            return F2K_ERR_CUDA;
        p.o_ptr[s]          = g.o;
        p.o_tok_stride[s]   = os_;
        p.o_batch_stride[s] = (long long)g.len * os_;
        p.q_len[s]          = g.len;
        p.q_tile_start[s]   = tiles;
        tiles += (g.len + kTileM - 1) / kTileM;
    }
    p.q_tile_start[nq] = tiles;
    p.n_qseg    = nq;
    p.n_q_tiles = tiles;
    tiles = 0;
    for (int s = 0; s < nkv; ++s) {
        const KvSeg& g = kvs[s];
        if (!g.k || !g.v) return fail(h, F2K_ERR_INVALID, "null tensor pointer");
        const long long ks_ = g.k_stride ? g.k_stride : tok, vs_ = g.v_stride ? g.v_stride : tok;
        if (!encode_segment(&p.tm_k[s], g.k, g.len, c.n_heads, c.batch, ks_, (long long)g.len * ks_, h->err) ||
            !encode_segment(&p.tm_v[s], g.v, g.len, c.n_heads, c.batch, vs_, (long long)g.len * vs_, h->err))
            return F2K_ERR_CUDA;
        p.kv_len[s]        = g.len;
        p.kv_tile_start[s] = tiles;
        tiles += (g.len + kTileN - 1) / kTileN;
    }
    p.kv_tile_start[nkv] = tiles;
    p.n_kvseg    = nkv;
    p.n_kv_tiles = tiles;
    p.n_heads    = c.n_heads;
    p.batch      = c.batch;
    p.scale_log2 = h->scale * 1.4426950408889634f;
    p.status     = h->d_status;
    p.wait_limit_clk      = h->wait_clk;
    p.peer_wait_limit_clk = h->peer_wait_clk;
    return F2K_OK;
}

// Builds (or reuses) the launch parameters for attention over the text||image
// segments held at the given pointers.
// vo_strides: token strides of v_txt, o_txt, v_img, o_img (0 = dense); Q and K are dense here.
int prepare_params(f2k_attn* h, const void* q_txt, const void* k_txt, const void* v_txt,
                   const void* q_img, const void* k_img, const void* v_img, void* o_txt,
                   void* o_img, const long long* vo_strides = nullptr) {
    const void* in[6] = {q_txt, k_txt, v_txt, q_img, k_img, v_img};
    void* out[2]      = {o_txt, o_img};
    long long vo[4]   = {0, 0, 0, 0};
    if (vo_strides) std::memcpy(vo, vo_strides, sizeof vo);
    if (h->have_params && std::memcmp(in, h->last_in, sizeof in) == 0 &&
        std::memcmp(out, h->last_out, sizeof out) == 0 && std::memcmp(vo, h->last_vo, sizeof vo) == 0)
        return F2K_OK;
    h->have_params = false;
    const f2k_attn_config& c = h->cfg;
    QSeg  qs[2];
    KvSeg kvs[2];
    int n = 0;
    if (c.seq_txt > 0) {
        qs[n]  = {q_txt, o_txt, c.seq_txt, 0, vo[1]};
        kvs[n] = {k_txt, v_txt, c.seq_txt, 0, vo[0]};
        ++n;
    }
    qs[n]  = {q_img, o_img, c.seq_img, 0, vo[3]};
    kvs[n] = {k_img, v_img, c.seq_img, 0, vo[2]};
    ++n;
    for (int i = 0; i < n; ++i)
        if (!qs[i].q || !kvs[i].k || !kvs[i].v || !qs[i].o) return fail(h, F2K_ERR_INVALID, "null tensor pointer");
    const int rc = build_params(h, h->params, qs, n, kvs, n);
    if (rc != F2K_OK) return rc;
    std::memcpy(h->last_in, in, sizeof in);
    std::memcpy(h->last_out, out, sizeof out);
    std::memcpy(h->last_vo, vo, sizeof vo);
    h->have_params = true;
    return F2K_OK;
}

// ---- host-buffer entry point: set-up shared by its two pipelines ----
cudaError_t ensure_pipe(f2k_attn* h, int n_stages) {
    cudaError_t e = cudaSuccess;
    while ((int)h->arrived.size() < n_stages && e == cudaSuccess) {
        cudaEvent_t a = nullptr, b = nullptr;
        e = cudaEventCreateWithFlags(&a, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&b, cudaEventDisableTiming);
        if (e == cudaSuccess) { h->arrived.push_back(a); h->computed.push_back(b); }
    }
    for (cudaEvent_t* ev : {&h->ev_start, &h->ev_out, &h->ev_k, &h->ev_v})
        if (e == cudaSuccess && !*ev) e = cudaEventCreateWithFlags(ev, cudaEventDisableTiming);
    if (e == cudaSuccess && !h->s_in) e = cudaStreamCreateWithFlags(&h->s_in, cudaStreamNonBlocking);
    if (e == cudaSuccess && !h->s_out) e = cudaStreamCreateWithFlags(&h->s_out, cudaStreamNonBlocking);
    return e;
}

constexpr int kChunkRows = 1024;   // query rows per launch of the batch-1 pipeline: 4 CTA pairs per head

// Batch 1: every transfer is one linear copy. K and V go in first, whole; then the query rows in
// chunks of kChunkRows of the joint (text, then image) sequence. A chunk's rows are normalised,
// attended over all keys and sent back while the next chunk's rows are still coming in, so the step
// takes the host-to-device time of Q, K, V plus the last chunk's kernels and output copy.
int host_row_chunks(f2k_attn* h, const void* hq_txt, const void* hk_txt, const void* hv_txt,
                    const void* hq_img, const void* hk_img, const void* hv_img, const void* gamma_q_txt,
                    const void* gamma_k_txt, const void* gamma_q_img, const void* gamma_k_img,
                    const float* cos_txt, const float* sin_txt, const float* cos_img, const float* sin_img,
                    float eps, void* ho_txt, void* ho_img, cudaStream_t s) {
    const f2k_attn_config& c = h->cfg;
    const int St = c.seq_txt, Si = c.seq_img, S = St + Si;
    const int n_chunks = (S + kChunkRows - 1) / kChunkRows;
    cudaError_t e = ensure_pipe(h, n_chunks);
    if (e != cudaSuccess) return fail_cuda(h, "host pipeline set-up", e);
    const size_t bt = align_up(h->bytes_txt(), kAlign), bi = align_up(h->bytes_img(), kAlign);
    const size_t need = 4 * bt + 4 * bi + h->fused_ws();
    if (h->stage_bytes < need) {
        if (h->stage) cudaFree(h->stage);
        h->stage = nullptr;
        h->stage_bytes = 0;
        h->chunk_params.clear();
        e = cudaMalloc(&h->stage, need);
        if (e != cudaSuccess) return fail_cuda(h, "cudaMalloc(staging)", e);
        h->stage_bytes = need;
    }
    uint8_t* d = static_cast<uint8_t*>(h->stage);
    uint8_t *dq_t = d, *dk_t = d + bt, *dv_t = d + 2 * bt, *do_t = d + 3 * bt;
    uint8_t* di = d + 4 * bt;
    uint8_t *dq_i = di, *dk_i = di + bi, *dv_i = di + 2 * bi, *do_i = di + 3 * bi;
    uint8_t* ws = di + 4 * bi;
    uint8_t *qn_t = ws, *kn_t = ws + bt, *qn_i = ws + 2 * bt, *kn_i = ws + 2 * bt + bi;
    const size_t tokb = (size_t)c.n_heads * kHeadDim * 2;       // bytes of one token, all heads

    // the rows of chunk i: [t0, t1) of the text stream and [i0, i1) of the image stream
    auto chunk_rows = [&](int i, int& t0, int& t1, int& i0, int& i1) {
        const int r0 = i * kChunkRows, r1 = std::min(S, r0 + kChunkRows);
        t0 = std::min(r0, St); t1 = std::min(r1, St);
        i0 = std::max(r0, St) - St; i1 = std::max(r1, St) - St;
    };
    if ((int)h->chunk_params.size() != n_chunks) {
        h->chunk_params.assign(n_chunks, AttnParams{});
        KvSeg kvs[2];
        int nkv = 0;
        if (St > 0) kvs[nkv++] = {kn_t, dv_t, St};
        kvs[nkv++] = {kn_i, dv_i, Si};
        for (int i = 0; i < n_chunks; ++i) {
            int t0, t1, i0, i1;
            chunk_rows(i, t0, t1, i0, i1);
            QSeg qs[2];
            int nq = 0;
            if (t1 > t0) qs[nq++] = {qn_t + t0 * tokb, do_t + t0 * tokb, t1 - t0};
            if (i1 > i0) qs[nq++] = {qn_i + i0 * tokb, do_i + i0 * tokb, i1 - i0};
            const int rc = build_params(h, h->chunk_params[i], qs, nq, kvs, nkv);
            if (rc != F2K_OK) { h->chunk_params.clear(); return rc; }
        }
    }

    auto copy = [&](void* dst, const void* src, size_t n, cudaMemcpyKind kind, cudaStream_t st) {
        if (e == cudaSuccess && n) e = cudaMemcpyAsync(dst, src, n, kind, st);
    };
    QkPrologueParams pp;
    long long rows = 0;
    auto reset_jobs = [&]() { std::memset(&pp, 0, sizeof pp); rows = 0; pp.n_heads = c.n_heads; pp.eps = eps; };
    auto add_job = [&](const void* x, void* y, const void* g, const float* ct, const float* sn, int len) {
        QkPrologueJob& j = pp.job[pp.n_jobs];
        j.x = x; j.y = y; j.gamma = g; j.cos_tab = ct; j.sin_tab = sn; j.seq = len;
        j.rows = (long long)len * c.n_heads;
        pp.row_start[pp.n_jobs] = rows;
        rows += j.rows;
        pp.row_start[++pp.n_jobs] = rows;
    };

    e = cudaEventRecord(h->ev_start, s);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(h->s_in, h->ev_start, 0);
    copy(dk_t, hk_txt, h->bytes_txt(), cudaMemcpyHostToDevice, h->s_in);
    copy(dk_i, hk_img, h->bytes_img(), cudaMemcpyHostToDevice, h->s_in);
    if (e == cudaSuccess) e = cudaEventRecord(h->ev_k, h->s_in);
    copy(dv_t, hv_txt, h->bytes_txt(), cudaMemcpyHostToDevice, h->s_in);
    copy(dv_i, hv_img, h->bytes_img(), cudaMemcpyHostToDevice, h->s_in);
    if (e == cudaSuccess) e = cudaEventRecord(h->ev_v, h->s_in);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(s, h->ev_k, 0);
    if (e != cudaSuccess) return fail_cuda(h, "host-to-device copy (K, V)", e);
    reset_jobs();
    if (St > 0) add_job(dk_t, kn_t, gamma_k_txt, cos_txt, sin_txt, St);
    add_job(dk_i, kn_i, gamma_k_img, cos_img, sin_img, Si);
    e = qk_prologue_launch(pp, s);
    if (e != cudaSuccess) return fail_cuda(h, "prologue launch (K)", e);

    for (int i = 0; i < n_chunks; ++i) {
        int t0, t1, i0, i1;
        chunk_rows(i, t0, t1, i0, i1);
        if (t1 > t0) copy(dq_t + t0 * tokb, static_cast<const uint8_t*>(hq_txt) + t0 * tokb, (t1 - t0) * tokb,
                          cudaMemcpyHostToDevice, h->s_in);
        if (i1 > i0) copy(dq_i + i0 * tokb, static_cast<const uint8_t*>(hq_img) + i0 * tokb, (i1 - i0) * tokb,
                          cudaMemcpyHostToDevice, h->s_in);
        if (e == cudaSuccess) e = cudaEventRecord(h->arrived[i], h->s_in);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(s, h->arrived[i], 0);
        if (e == cudaSuccess && i == 0) e = cudaStreamWaitEvent(s, h->ev_v, 0);
        if (e != cudaSuccess) return fail_cuda(h, "host-to-device copy (Q)", e);
        reset_jobs();
        if (t1 > t0) add_job(dq_t + t0 * tokb, qn_t + t0 * tokb, gamma_q_txt, cos_txt + (size_t)t0 * 64,
                             sin_txt + (size_t)t0 * 64, t1 - t0);
        if (i1 > i0) add_job(dq_i + i0 * tokb, qn_i + i0 * tokb, gamma_q_img, cos_img + (size_t)i0 * 64,
                             sin_img + (size_t)i0 * 64, i1 - i0);
        e = qk_prologue_launch(pp, s);
        if (e == cudaSuccess) e = attn_fwd_launch(h->chunk_params[i], s);
        if (e != cudaSuccess) return fail_cuda(h, "kernel launch", e);
        e = cudaEventRecord(h->computed[i], s);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(h->s_out, h->computed[i], 0);
        if (t1 > t0) copy(static_cast<uint8_t*>(ho_txt) + t0 * tokb, do_t + t0 * tokb, (t1 - t0) * tokb,
                          cudaMemcpyDeviceToHost, h->s_out);
        if (i1 > i0) copy(static_cast<uint8_t*>(ho_img) + i0 * tokb, do_i + i0 * tokb, (i1 - i0) * tokb,
                          cudaMemcpyDeviceToHost, h->s_out);
        if (e != cudaSuccess) return fail_cuda(h, "device-to-host copy", e);
    }
    e = cudaEventRecord(h->ev_out, h->s_out);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(s, h->ev_out, 0);
    if (e != cudaSuccess) return fail_cuda(h, "event", e);
    return F2K_OK;
}

}  // namespace

extern "C" {

int f2k_attn_create(const f2k_attn_config* cfg, f2k_attn** out) {
    if (!out) return F2K_ERR_INVALID;
    *out = nullptr;
    f2k_attn* h = new (std::nothrow) f2k_attn();
    if (!h) return F2K_ERR_CUDA;
    *out = h;
    if (!cfg) return fail(h, F2K_ERR_INVALID, "null config");
    h->cfg = *cfg;
    // Same refusals, same wording, as the reference constructors.
    if (cfg->batch <= 0 || cfg->seq_txt < 0 || cfg->seq_img <= 0 || cfg->n_heads <= 0 ||
        cfg->head_dim <= 0)
        return fail(h, F2K_ERR_INVALID,
                    cfg->seq_txt != 0 ? "JointAttention: zero/negative dim" : "Attention: zero/negative dim");
    if (cfg->head_dim != kHeadDim)
        return fail(h, F2K_ERR_UNSUPPORTED,
                    "head_dim must be 128: this engine implements only the MMDiT attention shape "
                    "and has no fallback kernel for other head dims");
    h->scale = cfg->scale > 0.f ? cfg->scale : 1.0f / std::sqrt((float)cfg->head_dim);

    cudaError_t e = cudaGetDevice(&h->device);
    if (e != cudaSuccess) return fail_cuda(h, "cudaGetDevice", e);
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, h->device);
    if (e != cudaSuccess) return fail_cuda(h, "cudaDeviceGetAttribute", e);
    if (major != 10)
        return fail(h, F2K_ERR_UNSUPPORTED, "this library contains sm_100a code only (needs a B200-class GPU)");
    e = attn_fwd_prepare();          // load the kernels now rather than inside the first forward call
    if (e == cudaSuccess) e = qk_prologue_prepare();
    if (e != cudaSuccess) return fail_cuda(h, "kernel load", e);
    e = cudaMalloc(reinterpret_cast<void**>(&h->d_status), kStatusBytes);
    if (e != cudaSuccess) return fail_cuda(h, "cudaMalloc(status)", e);
    e = cudaMemset(h->d_status, 0, kStatusBytes);
    if (e != cudaSuccess) return fail_cuda(h, "cudaMemset(status)", e);
    h->valid = true;
    return F2K_OK;
}

void f2k_attn_destroy(f2k_attn* h) {
    if (!h) return;
    for (f2k_attn* c : h->child) f2k_attn_destroy(c);
    for (cudaEvent_t e : h->arrived) cudaEventDestroy(e);
    for (cudaEvent_t e : h->computed) cudaEventDestroy(e);
    if (h->ev_start) cudaEventDestroy(h->ev_start);
    if (h->ev_k) cudaEventDestroy(h->ev_k);
    if (h->ev_v) cudaEventDestroy(h->ev_v);
    if (h->ev_out) cudaEventDestroy(h->ev_out);
    if (h->s_in) cudaStreamDestroy(h->s_in);
    if (h->s_out) cudaStreamDestroy(h->s_out);
    if (h->d_status) cudaFree(h->d_status);
    if (h->stage) cudaFree(h->stage);
    delete h;
}

const char* f2k_attn_last_error(const f2k_attn* h) { return h ? h->err.c_str() : "no handle"; }

size_t f2k_attn_workspace_bytes(const f2k_attn* h) {
    (void)h;
    return 0;
}

size_t f2k_attn_fused_workspace_bytes(const f2k_attn* h) { return (h && h->valid) ? h->fused_ws() : 0; }

int f2k_attn_forward(f2k_attn* h, const void* q_txt, const void* k_txt, const void* v_txt,
                     const void* q_img, const void* k_img, const void* v_img, void* o_txt,
                     void* o_img, void* workspace, size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;  // nothing to check: this path needs no workspace
    if (!h) return F2K_ERR_INVALID;
    if (!h->valid) return F2K_ERR_INVALID;  // keeps the creation error as last_error
    const int rc = prepare_params(h, q_txt, k_txt, v_txt, q_img, k_img, v_img, o_txt, o_img);
    if (rc != F2K_OK) return rc;
    const cudaError_t e = attn_fwd_launch(h->params, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail_cuda(h, "attention launch", e);
    return F2K_OK;
}

int f2k_attn_forward_fused(f2k_attn* h, const void* q_txt, const void* k_txt, const void* v_txt,
                           const void* q_img, const void* k_img, const void* v_img,
                           const void* gamma_q_txt, const void* gamma_k_txt,
                           const void* gamma_q_img, const void* gamma_k_img, const float* cos_txt,
                           const float* sin_txt, const float* cos_img, const float* sin_img,
                           float eps, void* o_txt, void* o_img, void* workspace,
                           size_t workspace_bytes, void* stream) {
    return f2k_attn_forward_fused_strided(h, q_txt, k_txt, v_txt, q_img, k_img, v_img, gamma_q_txt, gamma_k_txt,
                                          gamma_q_img, gamma_k_img, cos_txt, sin_txt, cos_img, sin_img, eps, o_txt,
                                          o_img, nullptr, workspace, workspace_bytes, stream);
}

int f2k_attn_forward_fused_strided(f2k_attn* h, const void* q_txt, const void* k_txt, const void* v_txt,
                                   const void* q_img, const void* k_img, const void* v_img,
                                   const void* gamma_q_txt, const void* gamma_k_txt,
                                   const void* gamma_q_img, const void* gamma_k_img, const float* cos_txt,
                                   const float* sin_txt, const float* cos_img, const float* sin_img,
                                   float eps, void* o_txt, void* o_img, const f2k_attn_strides* strides,
                                   void* workspace, size_t workspace_bytes, void* stream) {
    if (!h) return F2K_ERR_INVALID;
    if (!h->valid) return F2K_ERR_INVALID;
    if (workspace_bytes < h->fused_ws() || !workspace)
        return fail(h, F2K_ERR_WORKSPACE, "workspace too small");
    const f2k_attn_config& c = h->cfg;
    const bool has_txt = c.seq_txt > 0;
    f2k_attn_strides st{};
    if (strides) {
        st = *strides;
        const long long dense = (long long)c.n_heads * kHeadDim;
        const long long all[8] = {st.q_txt, st.k_txt, st.v_txt, st.o_txt, st.q_img, st.k_img, st.v_img, st.o_img};
        for (long long v : all)
            if (v != 0 && (v < dense || v % 8 != 0))
                return fail(h, F2K_ERR_INVALID, "token stride must be 0 or a multiple of 8 that is >= n_heads * 128");
    }
    if (!q_img || !k_img || !gamma_q_img || !gamma_k_img || !cos_img || !sin_img ||
        (has_txt && (!q_txt || !k_txt || !gamma_q_txt || !gamma_k_txt || !cos_txt || !sin_txt)))
        return fail(h, F2K_ERR_INVALID, "null tensor pointer");
    {
        // V and O are checked where their tensor maps / output pointers are set up (build_params)
        const void* vec[12] = {q_img, k_img, gamma_q_img, gamma_k_img, cos_img, sin_img,
                               q_txt, k_txt, gamma_q_txt, gamma_k_txt, cos_txt, sin_txt};
        for (int i = 0; i < (has_txt ? 12 : 6); ++i)
            if (misaligned16(vec[i]))
                return fail(h, F2K_ERR_INVALID,
                            "Q, K, gain and RoPE-table pointers must be 16-byte aligned (the kernels use 16-byte loads)");
    }

    uint8_t* ws = static_cast<uint8_t*>(workspace);
    void* qn_txt = ws;
    void* kn_txt = ws + align_up(h->bytes_txt(), kAlign);
    void* qn_img = ws + 2 * align_up(h->bytes_txt(), kAlign);
    void* kn_img = static_cast<uint8_t*>(qn_img) + align_up(h->bytes_img(), kAlign);

    QkPrologueParams pp;
    std::memset(&pp, 0, sizeof pp);
    int n = 0;
    long long rows = 0;
    auto add = [&](const void* x, long long x_stride, void* y, const void* g, const float* ct, const float* sn,
                   int seq) {
        QkPrologueJob& j = pp.job[n];
        j.x = x; j.x_tok_stride = x_stride; j.y = y; j.gamma = g; j.cos_tab = ct; j.sin_tab = sn; j.seq = seq;
        j.rows = (long long)c.batch * seq * c.n_heads;
        pp.row_start[n] = rows;
        rows += j.rows;
        ++n;
    };
    if (has_txt) {
        add(q_txt, st.q_txt, qn_txt, gamma_q_txt, cos_txt, sin_txt, c.seq_txt);
        add(k_txt, st.k_txt, kn_txt, gamma_k_txt, cos_txt, sin_txt, c.seq_txt);
    }
    add(q_img, st.q_img, qn_img, gamma_q_img, cos_img, sin_img, c.seq_img);
    add(k_img, st.k_img, kn_img, gamma_k_img, cos_img, sin_img, c.seq_img);
    pp.row_start[n] = rows;
    pp.n_jobs  = n;
    pp.n_heads = c.n_heads;
    pp.eps     = eps;

    const long long vo[4] = {st.v_txt, st.o_txt, st.v_img, st.o_img};
    const int rc = prepare_params(h, has_txt ? qn_txt : nullptr, has_txt ? kn_txt : nullptr, v_txt,
                                  qn_img, kn_img, v_img, o_txt, o_img, vo);
    if (rc != F2K_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = qk_prologue_launch(pp, s);
    if (e != cudaSuccess) return fail_cuda(h, "prologue launch", e);
    e = attn_fwd_launch(h->params, s);
    if (e != cudaSuccess) return fail_cuda(h, "attention launch", e);
    return F2K_OK;
}

// Host buffers in, host buffers out, as a pipeline on two transfer streams of the handle and the
// caller's stream. Batch 1 splits the query rows (host_row_chunks above). Larger batches split the
// heads, which are independent: while the copy engine brings in Q, K, V of group g+1 (2-D copies that pick the
// group's columns out of the [batch, seq, heads, 128] host tensors), the SMs run the prologue and
// the attention of group g on a contiguous [batch, seq, heads/groups, 128] staging copy, and the
// other copy engine sends the output of group g-1 back. The host-to-device leg is the long one
// (three inputs per output), so the step takes about its time plus the last group's kernels and
// output copy. Stream order as seen by the caller is unchanged: the call starts after earlier work
// on `stream`, and later work on `stream` starts after the last output copy.
int f2k_attn_forward_fused_host(f2k_attn* h, const void* hq_txt, const void* hk_txt,
                                const void* hv_txt, const void* hq_img, const void* hk_img,
                                const void* hv_img, const void* gamma_q_txt,
                                const void* gamma_k_txt, const void* gamma_q_img,
                                const void* gamma_k_img, const float* cos_txt,
                                const float* sin_txt, const float* cos_img, const float* sin_img,
                                float eps, void* ho_txt, void* ho_img, void* stream) {
    if (!h) return F2K_ERR_INVALID;
    if (!h->valid) return F2K_ERR_INVALID;
    const f2k_attn_config& c = h->cfg;
    const bool has_txt = c.seq_txt > 0;
    if (!hq_img || !hk_img || !hv_img || !ho_img ||
        (has_txt && (!hq_txt || !hk_txt || !hv_txt || !ho_txt)))
        return fail(h, F2K_ERR_INVALID, "null host pointer");
    const bool big = 3 * h->bytes_img() >= ((size_t)4 << 20);    // small problems: one pass
    const char* mode = std::getenv("F2K_HOST_PIPELINE");         // measurement knob: "heads" or "rows"
    const bool want_rows = mode ? std::strcmp(mode, "rows") == 0 : (c.batch == 1 && big);
    if (!gamma_q_img || !gamma_k_img || !cos_img || !sin_img ||
        (has_txt && (!gamma_q_txt || !gamma_k_txt || !cos_txt || !sin_txt)))
        return fail(h, F2K_ERR_INVALID, "null tensor pointer");
    {
        const void* vec[8] = {gamma_q_img, gamma_k_img, cos_img, sin_img, gamma_q_txt, gamma_k_txt, cos_txt, sin_txt};
        for (int i = 0; i < (has_txt ? 8 : 4); ++i)
            if (misaligned16(vec[i]))
                return fail(h, F2K_ERR_INVALID, "gain and RoPE-table pointers must be 16-byte aligned");
    }
    if (want_rows && c.batch == 1)
        return host_row_chunks(h, hq_txt, hk_txt, hv_txt, hq_img, hk_img, hv_img, gamma_q_txt, gamma_k_txt,
                               gamma_q_img, gamma_k_img, cos_txt, sin_txt, cos_img, sin_img, eps, ho_txt, ho_img,
                               static_cast<cudaStream_t>(stream));
    cudaError_t e = cudaSuccess;
    if (h->child.empty()) {
        // first call: split into head groups (none for small problems, where the extra copies cost
        // more than the overlap gains), make the children, streams and events
        int groups = 1;
        if (big) {
            if (c.n_heads % 8 == 0 && c.n_heads >= 16) groups = 8;      // measured best for 32 heads
            else if (c.n_heads % 4 == 0 && c.n_heads >= 8) groups = 4;
            else if (c.n_heads % 2 == 0 && c.n_heads >= 4) groups = 2;
        }
        if (const char* env = std::getenv("F2K_HOST_GROUPS")) {          // measurement knob
            const int g = std::atoi(env);
            if (g >= 1 && c.n_heads % g == 0) groups = g;
        }
        f2k_attn_config cc = c;
        cc.n_heads = c.n_heads / groups;
        cc.scale   = h->scale;
        for (int g = 0; g < groups; ++g) {
            f2k_attn* ch = nullptr;
            const int rc = f2k_attn_create(&cc, &ch);
            if (ch) h->child.push_back(ch);
            if (rc != F2K_OK) {
                const std::string msg = std::string("head-group handle: ") + f2k_attn_last_error(ch);
                for (f2k_attn* x : h->child) f2k_attn_destroy(x);
                h->child.clear();
                return fail(h, rc, msg);
            }
        }
        e = ensure_pipe(h, groups);
        if (e != cudaSuccess) {
            for (f2k_attn* x : h->child) f2k_attn_destroy(x);
            h->child.clear();
            return fail_cuda(h, "host pipeline set-up", e);
        }
    }
    const int groups = (int)h->child.size();
    f2k_attn* c0 = h->child[0];
    const int nh = c0->cfg.n_heads;
    const size_t bt = align_up(c0->bytes_txt(), kAlign), bi = align_up(c0->bytes_img(), kAlign);
    const size_t per_group = 4 * bt + 4 * bi + c0->fused_ws();
    const size_t need = per_group * groups;
    if (h->stage_bytes < need) {
        if (h->stage) cudaFree(h->stage);
        h->stage = nullptr;
        h->stage_bytes = 0;
        h->chunk_params.clear();
        e = cudaMalloc(&h->stage, need);
        if (e != cudaSuccess) return fail_cuda(h, "cudaMalloc(staging)", e);
        h->stage_bytes = need;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t hpitch = (size_t)c.n_heads * kHeadDim * 2;   // one token of all heads on the host
    const size_t dpitch = (size_t)nh * kHeadDim * 2;          // one token of the group on the device
    const size_t rows_t = (size_t)c.batch * c.seq_txt, rows_i = (size_t)c.batch * c.seq_img;
    auto h2d = [&](void* dst, const void* src, size_t rows, int g) {
        if (e == cudaSuccess && rows)
            e = cudaMemcpy2DAsync(dst, dpitch, static_cast<const uint8_t*>(src) + g * dpitch, hpitch, dpitch, rows,
                                  cudaMemcpyHostToDevice, h->s_in);
    };
    auto d2h = [&](void* dst, const void* src, size_t rows, int g) {
        if (e == cudaSuccess && rows)
            e = cudaMemcpy2DAsync(static_cast<uint8_t*>(dst) + g * dpitch, hpitch, src, dpitch, dpitch, rows,
                                  cudaMemcpyDeviceToHost, h->s_out);
    };
    e = cudaEventRecord(h->ev_start, s);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(h->s_in, h->ev_start, 0);
    if (e != cudaSuccess) return fail_cuda(h, "event", e);
    for (int g = 0; g < groups; ++g) {
        uint8_t* d = static_cast<uint8_t*>(h->stage) + g * per_group;
        void* dq_t = d;            void* dk_t = d + bt;       void* dv_t = d + 2 * bt;  void* do_t = d + 3 * bt;
        uint8_t* di = d + 4 * bt;
        void* dq_i = di;           void* dk_i = di + bi;      void* dv_i = di + 2 * bi; void* do_i = di + 3 * bi;
        void* ws = di + 4 * bi;
        if (has_txt) {
            h2d(dq_t, hq_txt, rows_t, g);
            h2d(dk_t, hk_txt, rows_t, g);
            h2d(dv_t, hv_txt, rows_t, g);
        }
        h2d(dq_i, hq_img, rows_i, g);
        h2d(dk_i, hk_img, rows_i, g);
        h2d(dv_i, hv_img, rows_i, g);
        if (e == cudaSuccess) e = cudaEventRecord(h->arrived[g], h->s_in);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(s, h->arrived[g], 0);
        if (e != cudaSuccess) return fail_cuda(h, "host-to-device copy", e);
        f2k_attn* ch = h->child[g];
        const int rc = f2k_attn_forward_fused(ch, has_txt ? dq_t : nullptr, has_txt ? dk_t : nullptr,
                                              has_txt ? dv_t : nullptr, dq_i, dk_i, dv_i, gamma_q_txt,
                                              gamma_k_txt, gamma_q_img, gamma_k_img, cos_txt, sin_txt,
                                              cos_img, sin_img, eps, has_txt ? do_t : nullptr, do_i, ws,
                                              ch->fused_ws(), stream);
        if (rc != F2K_OK) return fail(h, rc, ch->err);
        e = cudaEventRecord(h->computed[g], s);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(h->s_out, h->computed[g], 0);
        if (has_txt) d2h(ho_txt, do_t, rows_t, g);
        d2h(ho_img, do_i, rows_i, g);
        if (e != cudaSuccess) return fail_cuda(h, "device-to-host copy", e);
    }
    e = cudaEventRecord(h->ev_out, h->s_out);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(s, h->ev_out, 0);
    if (e != cudaSuccess) return fail_cuda(h, "event", e);
    return F2K_OK;
}

int f2k_attn_device_status(f2k_attn* h, int* status_out) {
    if (!h || !h->valid) return F2K_ERR_INVALID;
    int st = 0;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail_cuda(h, "cudaDeviceSynchronize", e);
    e = cudaMemcpy(&st, h->d_status, sizeof st, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail_cuda(h, "status read", e);
    if (st != 0) {
        e = cudaMemset(h->d_status, 0, sizeof st);
        if (e != cudaSuccess) return fail_cuda(h, "status clear", e);
    }
    for (f2k_attn* ch : h->child) {      // head-group handles of the host-buffer entry point
        int cst = 0;
        f2k_attn_device_status(ch, &cst);
        st |= cst;
    }
    if (status_out) *status_out = st;
    if (st != 0) return fail(h, F2K_ERR_DEVICE, "a bounded wait inside the attention kernel expired");
    return F2K_OK;
}

int f2k_attn_set_wait_limits(f2k_attn* h, long long in_cta_clk, long long peer_clk) {
    if (!h || !h->valid) return F2K_ERR_INVALID;
    if (in_cta_clk < 0 || peer_clk < 0) return fail(h, F2K_ERR_INVALID, "wait limits must not be negative");
    h->wait_clk = in_cta_clk;
    h->peer_wait_clk = peer_clk;
    h->have_params = false;          // the limits travel inside the cached launch parameters
    h->chunk_params.clear();
    for (f2k_attn* ch : h->child) f2k_attn_set_wait_limits(ch, in_cta_clk, peer_clk);
    return F2K_OK;
}

int f2k_rmsnorm_bf16(const void* x, const void* gamma, void* y, int rows, int dim, float eps,
                     void* stream) {
    // Same refusals as the reference wrapper (kernels/rmsnorm.cu:76-77).
    if (rows <= 0 || dim <= 0) return F2K_ERR_INVALID;
    if (dim % 8 != 0) return F2K_ERR_INVALID;
    if (!x || !gamma || !y) return F2K_ERR_INVALID;
    if (misaligned16(x) || misaligned16(gamma) || misaligned16(y)) return F2K_ERR_INVALID;   // 16-byte loads
    return rmsnorm_rows_launch(x, gamma, y, rows, dim, eps, static_cast<cudaStream_t>(stream)) == cudaSuccess
               ? F2K_OK : F2K_ERR_CUDA;
}

int f2k_rope_4axis_inplace_bf16(void* x, const float* cos_table, const float* sin_table,
                                const int32_t* pos_ids, int rows, int head_dim, int seq_max,
                                void* stream) {
    // Same refusals as the reference wrapper (kernels/rope_4axis.cu:48-49).
    if (rows <= 0 || head_dim <= 0 || (head_dim & 1)) return F2K_ERR_INVALID;
    if (head_dim > 512) return F2K_ERR_INVALID;
    if (!x || !cos_table || !sin_table || !pos_ids || seq_max <= 0) return F2K_ERR_INVALID;
    // head_dim 128 rows go through 16-byte loads (x, and a token's 64 cos / sin values as float4);
    // other head dims through 4-byte loads of x
    if (head_dim == 128 ? (misaligned16(x) || misaligned16(cos_table) || misaligned16(sin_table))
                        : (reinterpret_cast<uintptr_t>(x) & 3u) != 0)
        return F2K_ERR_INVALID;
    if ((reinterpret_cast<uintptr_t>(cos_table) & 3u) || (reinterpret_cast<uintptr_t>(sin_table) & 3u) ||
        (reinterpret_cast<uintptr_t>(pos_ids) & 3u))
        return F2K_ERR_INVALID;
    return rope4_rows_launch(x, cos_table, sin_table, pos_ids, rows, head_dim, seq_max,
                             static_cast<cudaStream_t>(stream)) == cudaSuccess
               ? F2K_OK : F2K_ERR_CUDA;
}

int f2k_build_rope_4axis_tables(const int* axes_dim, int n_axes, const int* positions, int seq,
                                float theta, float* cos_out, float* sin_out) {
    if (!axes_dim || n_axes <= 0 || seq < 0 || (seq > 0 && (!positions || !cos_out || !sin_out)))
        return F2K_ERR_INVALID;
    int head_dim = 0;
    for (int a = 0; a < n_axes; ++a) {
        if (axes_dim[a] < 0) return F2K_ERR_INVALID;
        head_dim += axes_dim[a];
    }
    const int half = head_dim / 2;
    // Per axis a, pair k: frequency theta^(-2k/d_a) in double; angle = position * frequency;
    // an axis fills d_a/2 consecutive pair slots of the token's row.
    std::vector<double> freq((size_t)half > 0 ? half : 1);
    std::vector<int> axis_of((size_t)half > 0 ? half : 1);
    int off = 0;
    for (int a = 0; a < n_axes; ++a) {
        const int pairs = axes_dim[a] / 2;
        for (int k = 0; k < pairs && off + k < half; ++k) {
            freq[off + k]    = std::pow((double)theta, -2.0 * k / (double)axes_dim[a]);
            axis_of[off + k] = a;
        }
        off += pairs;
    }
    const int filled = off < half ? off : half;
    for (int s = 0; s < seq; ++s) {
        float* cr = cos_out + (size_t)s * half;
        float* sr = sin_out + (size_t)s * half;
        for (int k = 0; k < half; ++k) {
            if (k < filled) {
                const double ang = (double)positions[(size_t)s * n_axes + axis_of[k]] * freq[k];
                cr[k] = (float)std::cos(ang);
                sr[k] = (float)std::sin(ang);
            } else {  // odd axis widths leave trailing slots; the reference leaves them 0
                cr[k] = 0.f;
                sr[k] = 0.f;
            }
        }
    }
    return F2K_OK;
}

const char* f2k_attn_version(void) { return "f2k_attn sm_100a 0.2"; }

}  // extern "C"
