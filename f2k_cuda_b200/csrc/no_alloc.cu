// f2k_attn_forward_fused_noalloc: the fused call (per-head RMSNorm + RoPE, then joint
// attention) for callers that must not allocate device memory, and the reader of its status word.
//
// Who that is: code that runs where the CUDA allocator is off limits - a real-time loop that
// may not take the allocator's locks or risk its latency, a plug-in whose host application
// forbids device allocations after start-up, or a process whose device memory was handed out
// completely at start-up and that has no pool left to carve a workspace (or a handle's status
// word) from. Such a caller cannot use f2k_attn_create (it calls cudaMalloc once) nor provide
// the workspace f2k_attn_forward_fused wants.
//
// What replaces the workspace: a fixed array in the library's own device image
// (`g_scratch`, 32 MiB). It holds the status word and the normalised + rotated copies of Q and K
// that the prologue kernel hands to the attention kernel. Shapes that need more are refused.
//
// When the 32 MiB are taken. The array belongs to this file's device module. The CUDA runtime
// loads a module into a context when something of it is first used there (lazy loading, the
// default since CUDA 12.2; with CUDA_MODULE_LOADING=EAGER it happens when the context is
// created). Device memory for the array is reserved at that moment - for this library, inside
// the first call of either entry point of this file on a device - and is held until the
// process exits. That first call is therefore the one that can fail for lack of memory, and a
// caller that hands all device memory out at start-up has to make it BEFORE doing so:
// f2k_attn_noalloc_device_status(NULL, ...) is enough. After it, no call of this file
// allocates, frees or loads anything.
//
// On the host `g_scratch` is only a stand-in for the symbol: the device address is obtained
// with cudaGetSymbolAddress, once per device, on that device, in that first call, which should
// therefore also come before any stream capture begins.
//
// Every call uses the same array and finds whatever the previous call left in it. The status
// word is the only part that has to start at zero: it is cleared once when the device is set
// up and again by f2k_attn_noalloc_device_status when it reads a non-zero value, so a failure
// stays visible until it is read. The Q/K copies are overwritten in full before they are read.
// Two calls whose GPU work can overlap (different streams, or different host threads) race on
// the array: keep the calls of one device on one stream, or serialise them yourself.

#include "f2k_attn.h"

#include "attn_launch.h"

#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>

namespace {

using namespace f2k;

constexpr size_t kScratchBytes = 32u << 20;   // the stated maximum: 32 MiB per GPU
constexpr size_t kAlign        = 256;         // kStatusBytes (attn_params.h) keeps the tensors 256-aligned

static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct PerDevice {
    unsigned char* scratch = nullptr;   // device address of g_scratch on this device
    CUresult (*encode)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
};
constexpr int kMaxDevices = 64;
PerDevice  g_dev[kMaxDevices];
std::mutex g_setup_mutex;

int fail(char* errbuf, size_t errbuf_len, int code, const char* msg) {
    if (errbuf && errbuf_len) std::snprintf(errbuf, errbuf_len, "%s", msg);
    return code;
}

// Once per device, with that device current: device address of the scratch array (this is what
// makes the runtime load the module and reserve the array), the driver's tensor-map encoder,
// the kernels' one-time configuration, and a zero status word.
int setup_device(int dev, char* errbuf, size_t errbuf_len) {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    PerDevice& d = g_dev[dev];
    if (d.scratch && d.encode) return F2K_OK;
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
        char msg[160];
        std::snprintf(msg, sizeof msg, "cudaGetSymbolAddress(scratch) failed: %s", cudaGetErrorString(e));
        return fail(errbuf, errbuf_len, F2K_ERR_CUDA, msg);
    }
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    const cudaError_t e2 = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e2 != cudaSuccess || q != cudaDriverEntryPointSuccess || fn == nullptr)
        return fail(errbuf, errbuf_len, F2K_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if (attn_fwd_prepare() != cudaSuccess || qk_prologue_prepare() != cudaSuccess)
        return fail(errbuf, errbuf_len, F2K_ERR_CUDA, "loading the kernels failed");
    if (cudaMemset(ptr, 0, kStatusBytes) != cudaSuccess)
        return fail(errbuf, errbuf_len, F2K_ERR_CUDA, "clearing the status word failed");
    d.scratch = static_cast<unsigned char*>(ptr);
    d.encode  = reinterpret_cast<decltype(d.encode)>(fn);
    return F2K_OK;
}

// Current device, checked: index in range and compute capability 10.x.
int current_device(int* dev_out, char* errbuf, size_t errbuf_len) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return fail(errbuf, errbuf_len, F2K_ERR_CUDA, "cudaGetDevice failed");
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess || major != 10)
        return fail(errbuf, errbuf_len, F2K_ERR_UNSUPPORTED, "this library contains sm_100a code only");
    *dev_out = dev;
    return F2K_OK;
}

// bf16 [batch, len, heads, 128] -> 4-D tiled map, box 64 x 1 x 128 x 1, 128-byte swizzle.
bool encode_segment(const PerDevice& d, CUtensorMap* map, const void* base, int len, int heads, int batch) {
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return false;
    const cuuint64_t tok = (cuuint64_t)heads * kHeadDim;
    const cuuint64_t dims[4]    = {(cuuint64_t)kHeadDim, (cuuint64_t)heads, (cuuint64_t)len, (cuuint64_t)batch};
    const cuuint64_t strides[3] = {(cuuint64_t)kHeadDim * 2, tok * 2, tok * (cuuint64_t)len * 2};
    const cuuint32_t box[4]     = {64, 1, (cuuint32_t)kTileM, 1};
    const cuuint32_t estr[4]    = {1, 1, 1, 1};
    return d.encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" int f2k_attn_forward_fused_noalloc(
    const f2k_attn_config* cfg,
    const void* q_txt, const void* k_txt, const void* v_txt,
    const void* q_img, const void* k_img, const void* v_img,
    const void* gamma_q_txt, const void* gamma_k_txt, const void* gamma_q_img, const void* gamma_k_img,
    const float* cos_txt, const float* sin_txt, const float* cos_img, const float* sin_img,
    float eps, void* o_txt, void* o_img, void* stream, char* errbuf, size_t errbuf_len) {
    if (errbuf && errbuf_len) errbuf[0] = '\0';
    if (!cfg) return fail(errbuf, errbuf_len, F2K_ERR_INVALID, "null config");
    if (cfg->batch <= 0 || cfg->seq_txt < 0 || cfg->seq_img <= 0 || cfg->n_heads <= 0 || cfg->head_dim <= 0)
        return fail(errbuf, errbuf_len, F2K_ERR_INVALID, "zero/negative dim");
    if (cfg->head_dim != kHeadDim)
        return fail(errbuf, errbuf_len, F2K_ERR_UNSUPPORTED, "head_dim must be 128");
    const bool has_txt = cfg->seq_txt > 0;
    if (!q_img || !k_img || !v_img || !o_img || !gamma_q_img || !gamma_k_img || !cos_img || !sin_img ||
        (has_txt && (!q_txt || !k_txt || !v_txt || !o_txt || !gamma_q_txt || !gamma_k_txt || !cos_txt || !sin_txt)))
        return fail(errbuf, errbuf_len, F2K_ERR_INVALID, "null tensor pointer");
    {
        // 16-byte loads and stores everywhere: refuse here what would fault on the GPU
        const void* vec[16] = {q_img, k_img, v_img, o_img, gamma_q_img, gamma_k_img, cos_img, sin_img,
                               q_txt, k_txt, v_txt, o_txt, gamma_q_txt, gamma_k_txt, cos_txt, sin_txt};
        for (int i = 0; i < (has_txt ? 16 : 8); ++i)
            if ((reinterpret_cast<uintptr_t>(vec[i]) & 15u) != 0)
                return fail(errbuf, errbuf_len, F2K_ERR_INVALID, "tensor, gain and table pointers must be 16-byte aligned");
    }

    const size_t bt = align_up((size_t)cfg->batch * cfg->seq_txt * cfg->n_heads * kHeadDim * 2, kAlign);
    const size_t bi = align_up((size_t)cfg->batch * cfg->seq_img * cfg->n_heads * kHeadDim * 2, kAlign);
    const size_t need = kStatusBytes + 2 * bt + 2 * bi;
    if (need > kScratchBytes) {
        char msg[200];
        std::snprintf(msg, sizeof msg,
                      "shape needs %zu bytes of scratch but the built-in array holds %zu (32 MiB): "
                      "use f2k_attn_forward_fused with a caller-provided workspace",
                      need, kScratchBytes);
        return fail(errbuf, errbuf_len, F2K_ERR_WORKSPACE, msg);
    }

    int dev = 0;
    int rc = current_device(&dev, errbuf, errbuf_len);
    if (rc == F2K_OK) rc = setup_device(dev, errbuf, errbuf_len);
    if (rc != F2K_OK) return rc;
    const PerDevice& d = g_dev[dev];

    unsigned char* base = d.scratch;
    int*  status = reinterpret_cast<int*>(base);
    void* qn_txt = base + kStatusBytes;
    void* kn_txt = base + kStatusBytes + bt;
    void* qn_img = base + kStatusBytes + 2 * bt;
    void* kn_img = base + kStatusBytes + 2 * bt + bi;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    // The array keeps what the last call left. Nothing has to be cleared here: the Q/K copies are
    // written in full by the prologue kernel before the attention kernel reads them, and the status
    // word is zero unless an earlier call failed and nobody has read it yet.

    QkPrologueParams pp;
    std::memset(&pp, 0, sizeof pp);
    int n = 0;
    long long rows = 0;
    auto add = [&](const void* x, void* y, const void* g, const float* ct, const float* st, int seq) {
        QkPrologueJob& j = pp.job[n];
        j.x = x; j.y = y; j.gamma = g; j.cos_tab = ct; j.sin_tab = st; j.seq = seq;
        j.rows = (long long)cfg->batch * seq * cfg->n_heads;
        pp.row_start[n] = rows;
        rows += j.rows;
        ++n;
    };
    if (has_txt) {
        add(q_txt, qn_txt, gamma_q_txt, cos_txt, sin_txt, cfg->seq_txt);
        add(k_txt, kn_txt, gamma_k_txt, cos_txt, sin_txt, cfg->seq_txt);
    }
    add(q_img, qn_img, gamma_q_img, cos_img, sin_img, cfg->seq_img);
    add(k_img, kn_img, gamma_k_img, cos_img, sin_img, cfg->seq_img);
    pp.row_start[n] = rows;
    pp.n_jobs  = n;
    pp.n_heads = cfg->n_heads;
    pp.eps     = eps;

    AttnParams ap;
    std::memset(&ap, 0, sizeof ap);
    struct Seg { const void *q, *k, *v; void* o; int len; };
    Seg segs[2];
    int ns = 0;
    if (has_txt) segs[ns++] = {qn_txt, kn_txt, v_txt, o_txt, cfg->seq_txt};
    segs[ns++] = {qn_img, kn_img, v_img, o_img, cfg->seq_img};
    const long long tok = (long long)cfg->n_heads * kHeadDim;
    int tiles = 0;
    for (int i = 0; i < ns; ++i) {
        const Seg& g = segs[i];
        if ((reinterpret_cast<uintptr_t>(g.o) & 15u) != 0 ||
            !encode_segment(d, &ap.tm_q[i], g.q, g.len, cfg->n_heads, cfg->batch) ||
            !encode_segment(d, &ap.tm_k[i], g.k, g.len, cfg->n_heads, cfg->batch) ||
            !encode_segment(d, &ap.tm_v[i], g.v, g.len, cfg->n_heads, cfg->batch))
            return fail(errbuf, errbuf_len, F2K_ERR_INVALID, "tensor pointers must be 16-byte aligned device pointers");
        ap.o_ptr[i]          = g.o;
        ap.o_tok_stride[i]   = tok;
        ap.o_batch_stride[i] = tok * g.len;
        ap.q_len[i] = ap.kv_len[i] = g.len;
        ap.q_tile_start[i] = ap.kv_tile_start[i] = tiles;
        tiles += (g.len + kTileM - 1) / kTileM;
    }
    ap.q_tile_start[ns] = ap.kv_tile_start[ns] = tiles;
    ap.n_qseg = ap.n_kvseg = ns;
    ap.n_q_tiles = ap.n_kv_tiles = tiles;
    ap.n_heads    = cfg->n_heads;
    ap.batch      = cfg->batch;
    ap.scale_log2 = (cfg->scale > 0.f ? cfg->scale : 1.0f / std::sqrt((float)cfg->head_dim)) * 1.4426950408889634f;
    ap.status     = status;

    if (qk_prologue_launch(pp, s) != cudaSuccess)
        return fail(errbuf, errbuf_len, F2K_ERR_CUDA, "prologue launch failed");
    if (attn_fwd_launch(ap, s) != cudaSuccess)
        return fail(errbuf, errbuf_len, F2K_ERR_CUDA, "attention launch failed");
    return F2K_OK;
}

// Reads the status word of the allocation-free call on the current device and clears it when it
// is not zero. Synchronises the device. status_out may be NULL. Allocates nothing; on its first
// call on a device it does the same one-time set-up as the forward call.
extern "C" int f2k_attn_noalloc_device_status(int* status_out, char* errbuf, size_t errbuf_len) {
    if (errbuf && errbuf_len) errbuf[0] = '\0';
    int dev = 0;
    int rc = current_device(&dev, errbuf, errbuf_len);
    if (rc == F2K_OK) rc = setup_device(dev, errbuf, errbuf_len);
    if (rc != F2K_OK) return rc;
    int st = 0;
    if (cudaDeviceSynchronize() != cudaSuccess ||
        cudaMemcpy(&st, g_dev[dev].scratch, sizeof st, cudaMemcpyDeviceToHost) != cudaSuccess)
        return fail(errbuf, errbuf_len, F2K_ERR_CUDA, "reading the status word failed");
    if (st != 0 && cudaMemset(g_dev[dev].scratch, 0, sizeof st) != cudaSuccess)
        return fail(errbuf, errbuf_len, F2K_ERR_CUDA, "clearing the status word failed");
    if (status_out) *status_out = st;
    if (st != 0)
        return fail(errbuf, errbuf_len, F2K_ERR_DEVICE,
                    "a bounded wait inside the attention kernel expired: the outputs of the calls since the last "
                    "status read must not be used");
    return F2K_OK;
}
