// Non-causal flash-attention forward for head_dim 128, bf16, written for sm_100a.
//
// One CTA owns a pair of 128-row query tiles of one (batch, head) and walks every
// key/value tile of the attended sequence. Three warpgroups:
//
//   warps 0-3 / 4-7     softmax group for tile 0 / tile 1: one thread per query
//                       row (= TMEM lane). Reads S_t with tcgen05.ld, keeps the
//                       row in registers, exponentiates in the log2 domain, writes
//                       bf16 P_t over the first 64 columns of S_t (handed to the MMA
//                       warp in parts, so P_t V_j starts before the row is finished)
//                       and accumulates the row sum from the unrounded fp32 values.
//   warp 8  (one lane)  TMA producer: Q tiles once, then K_j, V_j into a 4-slot
//                       ring of 32 KiB shared-memory slots (mbarrier full/empty).
//   warp 9  (converged) tcgen05.mma issuer:  S_t = Q_t K_j^T  (A, B from shared
//                       memory, K-major, 128-byte swizzle) and O_t += P_t V_j
//                       (A = P_t from tensor memory, B = V_j MN-major). S_0, S_1,
//                       O_0, O_1 are 128-column fp32 accumulators in TMEM.
//   warps 10-11         give their registers to the softmax groups (setmaxnreg: 208 registers
//                       per softmax thread, 88 elsewhere). In head-exchange use they do the
//                       exchange: QK-norm + RoPE of this rank's raw Q, K and peer stores of every
//                       head row to the rank that attends it, while the other roles already work
//                       on what has arrived (ExchangeParams). Idle otherwise.
//
// Issue order per key/value tile j:  S0_j, PV1_{j-1}, S1_j, PV0_j.  While one
// softmax group works on its S, the tensor pipe runs the other tile's two MMAs.
//
// Online softmax with a lazy reference maximum: the exponent reference of a row
// only moves when some row of the warp sees a tile maximum more than 2^8 above it;
// then the group rescales its O rows in TMEM itself. That window is safe because
// the commit that published S_t for tile j also covers PV_t of tile j-1, and
// PV_t of tile j is not issued before the group hands over P_t.
//
// Arithmetic follows the reference flash kernel (F2K_CUDA
// src/backend/cuda/attention.cu:601-757): scores scaled by `scale`, P rounded to
// bf16 for the P.V product, the row sum taken from fp32 P, one bf16 rounding of O.
//
// Every wait is bounded; when one expires the CTA sets the status word, drains its
// own copies and MMAs, frees its tensor memory and returns.

#include "attn_launch.h"
#include "ptx.cuh"
#include "row_math.cuh"
#include "softmax_row.cuh"

#include <cuda_bf16.h>

namespace f2k {

using namespace f2k::ptx;

namespace {

constexpr int kThreads     = 384;
constexpr int kLoaderWarp  = 8;
constexpr int kMmaWarp     = 9;
constexpr int kStages      = 4;
constexpr uint32_t kTileBytes = kTileM * kHeadDim * 2;  // 32 KiB: one Q, K or V tile
constexpr uint32_t kBoxBytes  = kTileBytes / 2;         // one 128 x 64 TMA box
constexpr uint32_t kTmemCols  = 512;
constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO0 = 256, kColO1 = 384;
constexpr float kLazyThreshold = 8.0f;  // log2 units

// Tuning switches (compile-time; the defaults are what ships).
#ifndef F2K_OPT_SETMAXNREG
#define F2K_OPT_SETMAXNREG 1   // softmax warpgroups take registers from the load/MMA warpgroup
#endif
#ifndef F2K_OPT_P_PARTS
#define F2K_OPT_P_PARTS 4      // P is handed to the MMA warp in this many parts (1, 2 or 4)
#endif
#ifndef F2K_OPT_POLY_OF8
#define F2K_OPT_POLY_OF8 0     // of every 8 key pairs, how many take 2^x on the FMA pipe (0..8); see softmax_row.cuh
#endif
constexpr int kPParts = F2K_OPT_P_PARTS;
#ifndef F2K_OPT_REGS_SOFTMAX
#define F2K_OPT_REGS_SOFTMAX 208
#endif
// registers per thread after setmaxnreg: softmax warpgroups / the load+MMA warpgroup;
// 2 * 128 * softmax + 128 * other must stay within the 384 * 168 the CTA is launched with
constexpr int kRegsSoftmax = F2K_OPT_REGS_SOFTMAX, kRegsOther = (384 * 168 - 256 * F2K_OPT_REGS_SOFTMAX) / 128 / 8 * 8;
static_assert(kRegsOther >= 40, "the load and MMA warps need some registers too");

struct SmemCtl {
    uint64_t q_full[2];
    uint64_t kv_full[kStages];
    uint64_t kv_empty[kStages];
    uint64_t s_full[2];
    uint64_t p_full[2][kPParts];   // [tile][part of the key tile]
    uint64_t o_full[2];
    uint64_t drain;
    uint64_t xchg_full[2][2];      // head exchange: [warp][staging buffer] loaded
    uint32_t tmem_base;
    uint32_t abort;
    uint32_t softmax_done;         // softmax warps that have finished (head exchange: the spare warps then stop)
};

constexpr uint32_t kSmemQ    = 0;
constexpr uint32_t kSmemRing = 2 * kTileBytes;
constexpr uint32_t kSmemCtl  = kSmemRing + kStages * kTileBytes;
constexpr uint32_t kSmemStage = (kSmemCtl + sizeof(SmemCtl) + 127u) & ~127u;   // head exchange staging (bulk copies)
constexpr uint32_t kSmemUsed = kSmemStage + 2 * 2 * (16 * 256 + 4 * 512);

template <int kMax>
__device__ __forceinline__ void locate_tile(const int* tile_start, const int* len, int nseg,
                                            int tile, int& seg, int& row0, int& valid) {
    seg = 0;
#pragma unroll
    for (int i = 1; i < kMax; ++i)
        if (i < nseg && tile >= tile_start[i]) seg = i;
    row0  = (tile - tile_start[seg]) * kTileN;
    valid = min(kTileN, len[seg] - row0);
}

// The MMA-issuing thread is a single lane that shares its scheduler with softmax warps, so every
// instruction it needs per MMA delays the tensor pipe. Descriptors are therefore built once and
// advanced by adding a compile-time constant to their low word (the start-address field counts
// 16-byte units and never carries out of its 14 bits inside the CTA's shared memory).

// S_t = Q_t K^T: 8 k-steps of 16 over head_dim; both operands K-major, 128-byte swizzle, stored as
// two 128 x 64 boxes (k-steps 0-3 in the first, 4-7 in the second).
__device__ __forceinline__ void issue_qk(uint32_t d_tmem, uint64_t q_desc, uint64_t k_desc) {
    constexpr uint32_t idesc = umma_idesc_bf16(kTileM, kTileN, /*b_mn_major=*/false);
#pragma unroll
    for (int kk = 0; kk < kHeadDim / 16; ++kk) {
        constexpr uint32_t kBox16 = kBoxBytes >> 4;
        const uint32_t off = (kk >> 2) * kBox16 + (kk & 3) * 2;   // in 16-byte units
        umma_ss(d_tmem, q_desc + off, k_desc + off, idesc, kk > 0 ? 1u : 0u);
    }
}

// O_t (+)= P_t V: 8 k-steps of 16 keys. A = P_t in TMEM (two bf16 per 32-bit column, 8 columns per
// k-step); B = V tile, MN-major: head_dim contiguous in 64-element (128-byte) swizzled rows, one
// row per key, the second 64 head-dim elements one box (16 KiB) further on; 8-key groups are
// 1024 bytes apart. `part` selects 8 / kPParts consecutive k-steps.
__device__ __forceinline__ void issue_pv_part(uint32_t d_tmem, uint32_t p_tmem, uint64_t v_desc,
                                              int part, uint32_t accumulate) {
    constexpr uint32_t idesc = umma_idesc_bf16(kTileM, kHeadDim, /*b_mn_major=*/true);
    constexpr int kSteps = 8 / kPParts;
#pragma unroll
    for (int k4 = 0; k4 < kSteps; ++k4) {
        const int kk = part * kSteps + k4;
        umma_ts(d_tmem, p_tmem + kk * 8, v_desc + kk * (2048 >> 4), idesc, kk > 0 ? 1u : accumulate);
    }
}

// Head exchange by one of the CTA's two spare warps (see ExchangeParams). A chunk is 16 tokens of
// Q, or of K and V, for one destination. The queue walks the ranges of ExchangeParams::order: ring
// step i sends to rank - i (0 = this rank itself), which is the order in which the destinations
// get to this rank's segment.
//
// Two warps per CTA cannot keep enough loads in flight from registers (measured: 86 GB/s per
// GPU), so the rows travel as bulk copies through a small staging area in shared memory: one lane
// issues cp.async.bulk loads of up to 4 KiB of head rows (plus the tokens' cos/sin rows) into one
// of the warp's two buffers, the warp normalises + rotates the rows in place (a half-warp per
// row, as the prologue kernel does), and one bulk store sends them to the destination, local or
// peer. The loads of the next buffer are in flight while this one is worked on.
constexpr uint32_t kStageRowBytes = 16 * 256;                 // 16 head rows
constexpr uint32_t kStageTabBytes = 4 * 512;                  // cos + sin rows of up to 4 tokens
constexpr uint32_t kStageBufBytes = kStageRowBytes + kStageTabBytes;

// The warp stops taking chunks once its CTA's softmax groups are done (`softmax_done` reaches 8) if
// a later CTA will take the CTA's place (`may_stop`: CTAs start in index order, one per SM): that
// one brings exchange warps of its own. The CTAs of the last wave serve the queue until it is
// empty, so everything this rank owes its peers is sent. A CTA that waits for rows is running, so
// its own spare warps keep serving the queue: nothing can stall.
__device__ __forceinline__ bool exchange_role(const ExchangeParams& x, int lane, uint32_t stage_u32, uint8_t* stage_ptr,
                                              uint32_t bar0, volatile uint32_t* abort_flag, long long wait_limit,
                                              volatile uint32_t* softmax_done, bool may_stop) {
    const int hl = lane & 15, hw = lane >> 4;
    const int n_tiles = (x.s_loc + kTileM - 1) / kTileM;
    const int hpr = x.heads_per_rank, R = x.unit_rows, tpb = x.tokens_per_buf;
    const int n_hg = hpr / R;
    unsigned int fills = 0;                                    // buffers filled so far by this warp: buffer and parity
    bool ok = true;

    struct Chunk { int dst_rank, kind, tok0, tok1, n_tb, per_pass, n_fill; bool valid; };
    // Next chunk of the queue. The queue is a list of ranges (x.order): what the CTAs that run first
    // need first - their own query rows - comes first, then K/V in the order the kernel walks them.
    auto grab = [&]() {
        Chunk ch;
        unsigned int c = 0xffffffffu;
        if (lane == 0 && !(may_stop && *softmax_done >= 8u)) c = atomicAdd(x.next_chunk, 1u);
        c = __shfl_sync(0xffffffffu, c, 0);
        ch.valid = c < x.total_chunks;
        if (!ch.valid) return ch;
        int e = 0;
        unsigned int first = 0;
        while (e + 1 < x.n_ranges && c >= first + (unsigned int)x.order[e].n) { first += (unsigned int)x.order[e].n; ++e; }
        ch.kind = x.order[e].kind;                             // 0: Q rows, 1: K and V rows
        ch.dst_rank = (x.rank - (int)x.order[e].step + x.world) % x.world;
        ch.tok0 = (x.order[e].sub0 + (int)(c - first)) * kExchangeTokens;
        ch.tok1 = min(ch.tok0 + kExchangeTokens, x.s_loc);
        ch.n_tb = (ch.tok1 - ch.tok0 + tpb - 1) / tpb;
        ch.per_pass = n_hg * ch.n_tb;
        ch.n_fill = (ch.kind + 1) * ch.per_pass;
        return ch;
    };
    // fill f of a chunk: tensor, head group, token block
    auto issue = [&](const Chunk& ch, int f) {                 // lane 0 only
        const int pass = f / ch.per_pass, rem = f % ch.per_pass, hg = rem / ch.n_tb, t0 = ch.tok0 + (rem % ch.n_tb) * tpb;
        const int nt = min(tpb, ch.tok1 - t0);
        const bool rot = !(ch.kind == 1 && pass == 1);
        const __nv_bfloat16* xin = static_cast<const __nv_bfloat16*>(ch.kind == 0 ? x.q : (pass == 0 ? x.k : x.v));
        const unsigned int n = fills;
        const uint32_t buf = stage_u32 + (n & 1u) * kStageBufBytes, bar = bar0 + (n & 1u) * 8;
        bulk_wait_read<0>();                                   // the store that last used this buffer has read it
        mbar_arrive_expect_tx(bar, (uint32_t)nt * (uint32_t)(R * 256 + (rot ? 512 : 0)));
        for (int i = 0; i < nt; ++i) {
            bulk_load(buf + i * R * 256, xin + ((long long)(t0 + i) * x.n_heads_total + ch.dst_rank * hpr + hg * R) * kHeadDim,
                      R * 256, bar);
            if (rot) {
                bulk_load(buf + kStageRowBytes + i * 512, x.cos_tab + (long long)(t0 + i) * 64, 256, bar);
                bulk_load(buf + kStageRowBytes + i * 512 + 256, x.sin_tab + (long long)(t0 + i) * 64, 256, bar);
            }
        }
    };

    Chunk cur = grab();
    if (cur.valid && lane == 0) issue(cur, 0);
    while (cur.valid) {
        for (int f = 0; f < cur.n_fill; ++f) {
            const unsigned int n = fills;                      // the buffer fill f went into
            ++fills;
            if (f + 1 < cur.n_fill && lane == 0) issue(cur, f + 1);
            __syncwarp();
            ok = mbar_wait(bar0 + (n & 1u) * 8, (n >> 1) & 1u, abort_flag, wait_limit);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const int pass = f / cur.per_pass, rem = f % cur.per_pass, hg = rem / cur.n_tb;
            const int t0 = cur.tok0 + (rem % cur.n_tb) * tpb;
            const int nt = min(tpb, cur.tok1 - t0);
            const bool rot = !(cur.kind == 1 && pass == 1);
            uint8_t* buf = stage_ptr + (n & 1u) * kStageBufBytes;
            if (rot) {
                float g[8];
                unpack8(__ldg(reinterpret_cast<const uint4*>(cur.kind == 0 ? x.gamma_q : x.gamma_k) + hl), g);
                for (int row = hw; row < nt * R; row += 2) {   // a half-warp per row; both halves run the same count
                    const int ti = row / R;
                    uint4* cell = reinterpret_cast<uint4*>(buf + row * 256) + hl;
                    const float4 c4 = *(reinterpret_cast<const float4*>(buf + kStageRowBytes + ti * 512) + hl);
                    const float4 s4 = *(reinterpret_cast<const float4*>(buf + kStageRowBytes + ti * 512 + 256) + hl);
                    const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
                    *cell = norm_rope_row(*cell, g, cs, sn, x.eps);
                }
                fence_proxy_async_smem();                      // the rewritten rows, before the bulk store reads them
            }
            __syncwarp();
            if (lane == 0) {
                unsigned char* base = cur.kind == 0 ? x.dst_q[cur.dst_rank]
                                                    : (pass == 0 ? x.dst_k[cur.dst_rank] : x.dst_v[cur.dst_rank]);
                unsigned char* dst = base + (((long long)x.rank * x.s_loc + t0) * hpr + hg * R) * (long long)(kHeadDim * 2);
                const uint32_t src = stage_u32 + (n & 1u) * kStageBufBytes;
                if (n_hg == 1) {
                    bulk_store(dst, src, (uint32_t)(nt * R * 256));   // the tokens' rows are adjacent at the destination
                } else {
                    for (int i = 0; i < nt; ++i) bulk_store(dst + (long long)i * hpr * 256, src + i * R * 256, R * 256);
                }
                bulk_commit();
            }
        }
        if (!ok) break;
        // The first loads of the next chunk are started before this chunk's stores are waited for.
        const Chunk nxt = grab();
        if (nxt.valid && lane == 0) issue(nxt, 0);
        if (lane == 0) {
            bulk_wait<0>();                    // this chunk's rows are written, wherever they went
            fence_proxy_async_all();
            __threadfence_system();
            unsigned int* word = x.tile_words[cur.dst_rank] + cur.kind * n_tiles + cur.tok0 / kTileM;
            if (cur.kind == 1 && x.kv_walk_words[cur.dst_rank] != nullptr) {
                word = x.kv_walk_words[cur.dst_rank] +
                       kv_walk_tile(x.rank * x.s_loc + cur.tok0, cur.dst_rank * x.s_loc, x.world * x.s_loc);
            }
            atomicAdd_system(word, 1u);
        }
        __syncwarp();
        cur = nxt;
    }
    if (!ok) {
        // Leaving early: the loads of the buffer that was being filled ahead may still be on their way.
        volatile uint32_t never = 0;
        mbar_wait(bar0 + (fills & 1u) * 8, (fills >> 1) & 1u, &never, 40000000ll);
    }
    if (lane == 0) bulk_wait<0>();             // nothing of this warp reads shared memory after the kernel's exit
    return ok;
}

}  // namespace

// kWithExchange: the build of the kernel whose spare warps can run the head exchange (launches
// with p.xchg.enabled). The plain build has no code, shared memory or barriers for it.
template <bool kWithExchange>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_sm100_kernel(const __grid_constant__ AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t smem     = (raw_addr + 1023u) & ~1023u;  // swizzle atoms need 1 KiB
    SmemCtl* ctl = reinterpret_cast<SmemCtl*>(smem_raw + (smem - raw_addr) + kSmemCtl);
    volatile uint32_t* abort_flag = &ctl->abort;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int pair = p.grid_head_fastest ? blockIdx.y : blockIdx.x;
    const int head = p.grid_head_fastest ? blockIdx.x : blockIdx.y;
    const int bidx = blockIdx.z;
    const int n_kv = p.n_kv_tiles;
    // With an odd number of query tiles the last CTA of a (batch, head) has one tile only: its
    // second softmax group, and the MMAs that would feed it, are left out.
    const bool has_t1 = 2 * pair + 1 < p.n_q_tiles;
    const long long peer_limit = p.peer_wait_limit_clk;
    const long long wait_limit = p.wait_limit_clk;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&ctl->q_full[i]), 1);
            mbar_init(smem_u32(&ctl->s_full[i]), 1);
            for (int k = 0; k < kPParts; ++k) mbar_init(smem_u32(&ctl->p_full[i][k]), 128);
            mbar_init(smem_u32(&ctl->o_full[i]), 1);
        }
        for (int i = 0; i < kStages; ++i) {
            mbar_init(smem_u32(&ctl->kv_full[i]), 1);
            mbar_init(smem_u32(&ctl->kv_empty[i]), 1);
        }
        mbar_init(smem_u32(&ctl->drain), 1);
        if constexpr (kWithExchange)
            for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&ctl->xchg_full[0][0]) + i * 8, 1);
        ctl->abort = 0;
        ctl->softmax_done = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);

    if (warp >= 8) {
        // ===================== warpgroup 2: TMA producer, MMA issuer, two idle warps =====================
#if F2K_OPT_SETMAXNREG
        setmaxnreg_dec<kRegsOther>();
#endif
        if (warp == kLoaderWarp) {
            // ------------------------------ TMA producer ------------------------------
            if (lane == 0) {
                int issued = 0, q_issued = 0;
                bool ok = true;
                for (int t = 0; t < 2 && ok; ++t) {
                    const int qt = 2 * pair + t;
                    if (qt >= p.n_q_tiles) break;   // odd tile count: the last CTA of a head has one tile
                    int seg, row0, valid;
                    locate_tile<kMaxQSeg>(p.q_tile_start, p.q_len, p.n_qseg, qt, seg, row0, valid);
                    if (p.q_ready[seg] != nullptr) {   // the segment is written by another GPU's kernel
                        ok = p.ready_per_tile
                                 ? global_flag_wait(p.q_ready[seg] + row0 / kTileM,
                                                    p.ready_uses * (unsigned)((valid + kExchangeTokens - 1) / kExchangeTokens),
                                                    abort_flag, peer_limit)
                                 : global_flag_wait(p.q_ready[seg], p.kv_ready_value, abort_flag, peer_limit);
                        if (!ok) break;
                        asm volatile("fence.proxy.async.global;" ::: "memory");
                    }
                    const uint32_t bar = smem_u32(&ctl->q_full[t]);
                    const uint32_t dst = smem + kSmemQ + t * kTileBytes;
                    mbar_arrive_expect_tx(bar, kTileBytes);
                    tma_load_4d(dst, &p.tm_q[seg], bar, 0, head, row0, bidx);
                    tma_load_4d(dst + kBoxBytes, &p.tm_q[seg], bar, 64, head, row0, bidx);
                    ++q_issued;
                }
                for (int j = 0; j < n_kv && ok; ++j) {
                    int seg, row0, valid;
                    locate_tile<kMaxKvSeg>(p.kv_tile_start, p.kv_len, p.n_kvseg, j, seg, row0, valid);
                    if (p.ready_per_tile && p.kv_ready[seg] != nullptr) {
                        // fused head exchange: every tile has its own counter of delivered chunks
                        ok = global_flag_wait(p.kv_ready[seg] + row0 / kTileN,
                                              p.ready_uses * (unsigned)((valid + kExchangeTokens - 1) / kExchangeTokens),
                                              abort_flag, peer_limit);
                        if (!ok) break;
                        asm volatile("fence.proxy.async.global;" ::: "memory");
                    } else if (row0 == 0 && p.kv_ready[seg] != nullptr) {
                        // first tile of a segment that is being copied in: wait for its arrival word,
                        // then order the copy engine's writes before this thread's TMA reads
                        const unsigned int* word = p.kv_ready[seg] + head / max(1, p.kv_ready_heads_per_group);
                        for (int i = 0; i < max(1, p.kv_ready_words) && ok; ++i)
                            ok = global_flag_wait(word + i, p.kv_ready_value, abort_flag, peer_limit);
                        if (!ok) break;
                        asm volatile("fence.proxy.async.global;" ::: "memory");
                    }
#pragma unroll
                    for (int kv = 0; kv < 2; ++kv) {
                        const int slot = issued % kStages;
                        const uint32_t par = (issued / kStages) & 1;
                        ok = mbar_wait(smem_u32(&ctl->kv_empty[slot]), par ^ 1u, abort_flag, wait_limit);
                        if (!ok) break;
                        const uint32_t bar = smem_u32(&ctl->kv_full[slot]);
                        const uint32_t dst = smem + kSmemRing + slot * kTileBytes;
                        const CUtensorMap* tm = kv == 0 ? &p.tm_k[seg] : &p.tm_v[seg];
                        mbar_arrive_expect_tx(bar, kTileBytes);
                        tma_load_4d(dst, tm, bar, 0, head, row0, bidx);
                        tma_load_4d(dst + kBoxBytes, tm, bar, 64, head, row0, bidx);
                        ++issued;
                    }
                }
                if (!ok) {
                    // Leaving early: let the copies this thread started land first.
                    const long long lim = 40000000ll;  // ~20 ms each, still bounded
                    volatile uint32_t never = 0;
                    for (int t = 0; t < q_issued; ++t) mbar_wait(smem_u32(&ctl->q_full[t]), 0, &never, lim);
                    for (int i = max(0, issued - kStages); i < issued; ++i)
                        mbar_wait(smem_u32(&ctl->kv_full[i % kStages]), (i / kStages) & 1, &never, lim);
                }
            }
        } else if (warp > kMmaWarp) {
            // ------------------------------ head exchange -----------------------------
            if constexpr (kWithExchange) if (p.xchg.enabled) {
                const int xw = warp - kMmaWarp - 1;
                const unsigned int cta_linear = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
                exchange_role(p.xchg, lane, smem + kSmemStage + xw * 2 * kStageBufBytes,
                              smem_raw + (smem - raw_addr) + kSmemStage + xw * 2 * kStageBufBytes,
                              smem_u32(&ctl->xchg_full[xw][0]), abort_flag, wait_limit, &ctl->softmax_done,
                              cta_linear + p.xchg.n_sms < gridDim.x * gridDim.y * gridDim.z);
            }
        } else if (warp == kMmaWarp) {
            // ------------------------------ MMA issuer --------------------------------
            // The whole warp runs this loop converged; umma_* elect one lane per instruction.
            {
                bool ok = true;
                // Descriptors: Q tiles (fixed for the CTA) and ring slot 0 as K (K-major) / V (MN-major).
                const uint64_t q0_desc = umma_smem_desc(smem + kSmemQ, 16, 1024);
                const uint64_t q1_desc = umma_smem_desc(smem + kSmemQ + kTileBytes, 16, 1024);
                const uint64_t k_desc0 = umma_smem_desc(smem + kSmemRing, 16, 1024);
                const uint64_t v_desc0 = umma_smem_desc(smem + kSmemRing, kBoxBytes, 1024);
                const uint32_t bar_full0 = smem_u32(&ctl->kv_full[0]), bar_empty0 = smem_u32(&ctl->kv_empty[0]);
                // Ring slot of K_j is 2j, of V_j is 2j+1.
                auto slot_off16 = [&](int n) { return (uint32_t)(n % kStages) * (kTileBytes >> 4); };
                auto wait_uniform = [&](uint32_t bar, uint32_t parity) {
                    return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, wait_limit)) != 0;
                };
                auto wait_full = [&](int n) {
                    return wait_uniform(bar_full0 + (n % kStages) * 8, (n / kStages) & 1);
                };
                auto release = [&](int n) { umma_commit(bar_empty0 + (n % kStages) * 8); };
                // O_t (+)= P_t V_n, issued part by part as the softmax group hands P over.
                auto issue_pv = [&](int t, int jj) -> bool {
                    const uint32_t d = tmem + (t == 0 ? kColO0 : kColO1);
                    const uint32_t a = tmem + (t == 0 ? kColS0 : kColS1);
                    const uint64_t v_desc = v_desc0 + slot_off16(2 * jj + 1);
                    const uint32_t bar_p = smem_u32(&ctl->p_full[t][0]);
#pragma unroll
                    for (int part = 0; part < kPParts; ++part) {
                        if (!wait_uniform(bar_p + part * 8, jj & 1)) return false;
                        tc_fence_after_sync();
                        issue_pv_part(d, a, v_desc, part, jj > 0 ? 1u : 0u);
                    }
                    return true;
                };

                for (int j = 0; j < n_kv; ++j) {
                    // S0_j
                    if (!(ok = wait_full(2 * j))) break;
                    if (j == 0 && !(ok = wait_uniform(smem_u32(&ctl->q_full[0]), 0))) break;
                    tc_fence_after_sync();
                    issue_qk(tmem + kColS0, q0_desc, k_desc0 + slot_off16(2 * j));
                    umma_commit(smem_u32(&ctl->s_full[0]));
                    if (has_t1) {
                        // PV1_{j-1}
                        if (j > 0) {
                            if (!(ok = issue_pv(1, j - 1))) break;
                            release(2 * j - 1);
                        }
                        // S1_j
                        if (j == 0 && !(ok = wait_uniform(smem_u32(&ctl->q_full[1]), 0))) break;
                        tc_fence_after_sync();
                        issue_qk(tmem + kColS1, q1_desc, k_desc0 + slot_off16(2 * j));
                        umma_commit(smem_u32(&ctl->s_full[1]));
                    }
                    release(2 * j);
                    // PV0_j
                    if (!(ok = wait_full(2 * j + 1))) break;
                    if (!(ok = issue_pv(0, j))) break;
                    if (!has_t1) release(2 * j + 1);
                    if (j == n_kv - 1) umma_commit(smem_u32(&ctl->o_full[0]));
                }
                if (ok && n_kv > 0 && has_t1) {
                    // PV1 of the last tile
                    ok = issue_pv(1, n_kv - 1);
                    if (ok) {
                        release(2 * n_kv - 1);
                        umma_commit(smem_u32(&ctl->o_full[1]));
                    }
                }
                if (!ok) {
                    // Leaving early: wait (bounded) until the MMAs already issued retire, so
                    // tensor memory is idle when it is freed.
                    volatile uint32_t never = 0;
                    __syncwarp();
                    umma_commit(smem_u32(&ctl->drain));
                    mbar_wait(smem_u32(&ctl->drain), 0, &never, 40000000ll);
                }
            }
        }
    } else {
        // ===================== warpgroups 0 and 1: softmax for query tile 0 / 1 =====================
#if F2K_OPT_SETMAXNREG
        setmaxnreg_inc<kRegsSoftmax>();
#endif
        const int t = warp >> 2;                                       // which query tile
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;  // this warp's TMEM lanes
        const uint32_t tS = tmem + lane_base + (t == 0 ? kColS0 : kColS1);
        const uint32_t tO = tmem + lane_base + (t == 0 ? kColO0 : kColO1);
        const float c = p.scale_log2;

        float m_ref = -INFINITY;  // exponent reference, in raw score units
        float l_sum = 0.0f;
        bool ok = true;

        int kv_seg = 0, kv_row0 = 0;
        const int n_iter = (t == 0 || has_t1) ? n_kv : 0;
        for (int j = 0; j < n_iter; ++j) {
            const int valid = min(kTileN, p.kv_len[kv_seg] - kv_row0);
            kv_row0 += kTileN;
            if (kv_row0 >= p.kv_len[kv_seg]) { kv_row0 = 0; ++kv_seg; }

            ok = mbar_wait(smem_u32(&ctl->s_full[t]), j & 1, abort_flag, wait_limit);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();

            // The row is fetched in two halves: the maxima of the first 64 scores are folded while
            // the second 64 are still on their way from tensor memory.
            uint32_t s[128];
            float mx[kMaxChains];
            {
                uint32_t(&s0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[0]);
                uint32_t(&s1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[32]);
                uint32_t(&s2)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[64]);
                uint32_t(&s3)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[96]);
                tmem_ld_x32(tS + 0, s0);
                tmem_ld_x32(tS + 32, s1);
                tmem_wait_ld();
                tmem_ld_x32(tS + 64, s2);
                tmem_ld_x32(tS + 96, s3);
                if (valid < 64) {  // last tile of a segment: keys past its end do not exist
#pragma unroll
                    for (int i = 0; i < 64; ++i)
                        if (i >= valid) s[i] = __float_as_uint(-INFINITY);
                }
                row_max64<true>(&s[0], mx);
                tmem_wait_ld();
            }
            if (valid < kTileN) {
#pragma unroll
                for (int i = 64; i < 128; ++i)
                    if (i >= valid) s[i] = __float_as_uint(-INFINITY);
            }
            row_max64<false>(&s[64], mx);
            const float m_tile = row_max_finish(mx);

            const bool need = (m_tile - m_ref) * c > kLazyThreshold;
            if (__any_sync(0xffffffffu, need)) {
                const float m_new = fmaxf(m_ref, m_tile);
                const float f = ex2_approx((m_ref - m_new) * c);
                l_sum *= f;
                m_ref = m_new;
                if (j > 0) {
                    // Rescale this row of O in place (O_t is idle, see the file header).
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint32_t o[32];
                        tmem_ld_x32(tO + q * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                        tmem_st_x32(tO + q * 32, o);
                    }
                }
            }

            // P = 2^(c s - c m_ref), rounded to bf16 into the first 64 columns of S_t (two keys
            // per column); the row sum keeps the unrounded values.
            const float neg_mc = -m_ref * c;
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
            // A part of P is announced half a chunk after its last store was issued: by then the
            // store has drained, so the wait costs nothing and the special-function unit never
            // idles behind it. Only the last part has to wait for real.
            int pending = -1;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t pk[16];
                exp_chunk16<F2K_OPT_POLY_OF8>(&s[q * 32], pk, c, neg_mc, sum);
                if (pending >= 0) {
                    tmem_wait_st();
                    tc_fence_before_sync();
                    mbar_arrive(smem_u32(&ctl->p_full[t][0]) + pending * 8);
                    pending = -1;
                }
                exp_chunk16<F2K_OPT_POLY_OF8>(&s[q * 32 + 16], pk + 8, c, neg_mc, sum);
                tmem_st_x16(tS + q * 16, pk);
                if ((q + 1) % (4 / kPParts) == 0) pending = (q + 1) / (4 / kPParts) - 1;
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&ctl->p_full[t][kPParts - 1]));
            l_sum += (sum[0] + sum[1]) + (sum[2] + sum[3]);
        }

        // ------------------------------ epilogue ------------------------------------
        if (ok && n_iter > 0) {
            ok = mbar_wait(smem_u32(&ctl->o_full[t]), 0, abort_flag, wait_limit);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok && n_iter > 0) {
            tc_fence_after_sync();
            const int qt = 2 * pair + t;
            int seg = 0, row0 = 0, valid = 0;
            locate_tile<kMaxQSeg>(p.q_tile_start, p.q_len, p.n_qseg, qt, seg, row0, valid);
            const int r = (warp & 3) * 32 + lane;  // row inside the tile
            const float inv = 1.0f / (l_sum + 1e-30f);
            // The rows go out through the shared memory of this tile's Q (no MMA reads it any more:
            // o_full was committed after the last of them). Each thread parks its row there, 16-byte
            // chunk c of row r at chunk position c ^ (r & 15), and the warp then writes its 32 rows
            // two at a time, 16 lanes on the 256 contiguous bytes of one row. To local memory this
            // saves partial-sector writes; to a peer's memory (head exchange) it turns 16-byte
            // packets into 256-byte ones.
            const uint32_t park = smem + kSmemQ + t * kTileBytes;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t o[32];
                tmem_ld_x32(tO + q * 32, o);  // every lane takes part, valid row or not
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 v;
                    v.x = pack_bf16x2(__uint_as_float(o[i + 0]) * inv, __uint_as_float(o[i + 1]) * inv);
                    v.y = pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                    v.z = pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
                    v.w = pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
                    const int c = q * 4 + (i >> 3);
                    st_shared_v4(park + r * 256 + ((c ^ (r & 15)) << 4), v);
                }
            }
            __syncwarp();
            __nv_bfloat16* obase = static_cast<__nv_bfloat16*>(p.o_ptr[seg]) +
                                   (long long)bidx * p.o_batch_stride[seg] + (long long)head * kHeadDim;
            const int c = lane & 15;
#pragma unroll 2
            for (int it = 0; it < 16; ++it) {
                const int row = (warp & 3) * 32 + it * 2 + (lane >> 4);
                const uint4 v = ld_shared_v4(park + row * 256 + ((c ^ (row & 15)) << 4));
                if (row < valid)
                    *reinterpret_cast<uint4*>(obase + (long long)(row0 + row) * p.o_tok_stride[seg] + c * 8) = v;
            }
        }
    }

    if constexpr (kWithExchange)
        if (warp < 8 && lane == 0) atomicAdd(&ctl->softmax_done, 1u);   // (also when the warp left its loop early)

    // ------------------------------ common exit ---------------------------------
    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag != 0u && p.status != nullptr)
        atomicOr(p.status, (int)kStatusWaitExpired);
    if (threadIdx.x == 0 && p.done_counter != nullptr)   // all output rows of this CTA are stored (barrier above)
        grid_done_publish(p.done_counter, gridDim.x * gridDim.y * gridDim.z, p.done_flag, p.fail_flag, p.n_done,
                          p.done_value, p.status);
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, kTmemCols);
    }
}

size_t attn_fwd_smem_bytes() { return kSmemStage + 1024; }                        // plain build
static size_t attn_fwd_smem_bytes_exchange() { return kSmemUsed + 1024; }         // + the exchange's staging area

// Loads the kernel on the current device and raises its shared-memory limit. Called when a
// handle is created, so that the first launch does not have to load code: loading may
// synchronise the device, which must not happen while a stream is parked on a wait that only a
// later call (or another process) can satisfy.
cudaError_t attn_fwd_prepare() {
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && configured[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(attn_fwd_sm100_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)attn_fwd_smem_bytes());
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(attn_fwd_sm100_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)attn_fwd_smem_bytes_exchange());
    if (e != cudaSuccess) return e;
    cudaFuncAttributes attr;
    e = cudaFuncGetAttributes(&attr, attn_fwd_sm100_kernel<false>);
    if (e != cudaSuccess) return e;
    e = cudaFuncGetAttributes(&attr, attn_fwd_sm100_kernel<true>);
    if (e != cudaSuccess) return e;
    if (dev < 64) configured[dev] = true;
    return cudaSuccess;
}

cudaError_t attn_fwd_launch(const AttnParams& params, cudaStream_t stream) {
    cudaError_t e = attn_fwd_prepare();
    if (e != cudaSuccess) return e;
    AttnParams p = params;
    if (p.wait_limit_clk <= 0) p.wait_limit_clk = kDefaultWaitClk;
    if (p.peer_wait_limit_clk <= 0) p.peer_wait_limit_clk = kDefaultPeerWaitClk;
    // An in-CTA wait may sit behind a peer wait of the loader (a softmax group waits for S, the MMA
    // warp for K, the loader for the word), so it has to outlast it where peer words are in use.
    bool peer_words = false;
    for (int i = 0; i < kMaxKvSeg; ++i) peer_words |= p.kv_ready[i] != nullptr;
    for (int i = 0; i < kMaxQSeg; ++i) peer_words |= p.q_ready[i] != nullptr;
    if (peer_words) p.wait_limit_clk += p.peer_wait_limit_clk;
    dim3 grid((p.n_q_tiles + 1) / 2, p.n_heads, p.batch);
    if (p.grid_head_fastest) grid = dim3(p.n_heads, (p.n_q_tiles + 1) / 2, p.batch);
    if (p.xchg.enabled)
        attn_fwd_sm100_kernel<true><<<grid, kThreads, attn_fwd_smem_bytes_exchange(), stream>>>(p);
    else
        attn_fwd_sm100_kernel<false><<<grid, kThreads, attn_fwd_smem_bytes(), stream>>>(p);
    return cudaPeekAtLastError();
}

}  // namespace f2k
