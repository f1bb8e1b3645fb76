// Launch parameters shared by the host side (C ABI) and the sm_100a attention kernel.
//
// The attended sequence is described as a list of *segments*: contiguous runs of
// tokens that live in their own allocation ([batch, len, heads, 128] bf16, token
// stride and batch stride explicit). Joint attention has two (text, then image);
// plain attention has one; sequence-parallel attention has one key/value segment
// per rank. No segment is ever copied into a concatenated buffer: query tiles and
// key/value tiles are cut per segment and each tile is fetched through that
// segment's own TMA tensor map, so a tile never straddles two allocations.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cuda.h>

namespace f2k {

constexpr int kHeadDim  = 128;  // the only head_dim the MMDiT path uses
constexpr int kTileM    = 128;  // query rows per tile (one TMEM lane each)
constexpr int kTileN    = 128;  // keys per tile
constexpr int kMaxQSeg  = 8;
constexpr int kMaxKvSeg = 8;

// Bits of the device status word a launch may set (0 = clean run).
enum AttnStatus : int {
    kStatusOk          = 0,
    kStatusWaitExpired = 1,  // a bounded wait ran out; the output is invalid
    kStatusPeerFailed  = 2,  // head exchange: another rank's kernel gave up; rows it owed are stale
    kStatusAborted     = 4,  // the host released the stream waits of a step (f2k_*_abort)
};

constexpr size_t kStatusBytes = 256;   // every status allocation: the word, padded to the tensor alignment

// Limits of the bounded waits, in SM clock cycles (about 1.9 GHz). A wait inside the CTA (mbarrier:
// a TMA copy, an MMA, another role of the same CTA) has nothing slower than HBM behind it. A wait
// on a word that a copy engine or another GPU writes also covers the skew between the rank
// processes, which the host decides, so its default is much longer.
constexpr long long kDefaultWaitClk     = 2000000000ll;    // ~1 s
constexpr long long kDefaultPeerWaitClk = 40000000000ll;   // ~20 s

// Head exchange done by the attention kernel itself. Rank r holds the raw Q, K, V of its s_loc
// tokens for all heads; the kernel's two spare warps per CTA normalise + rotate Q and K and store
// every head row into the memory of the rank that attends that head (peer stores over NVLink; V is
// copied), while the CTA's other roles already attend to what has arrived. Work is cut into small
// chunks (kExchangeTokens tokens of one destination rank: their Q rows, or their K and V rows)
// handed out through a counter, in the order in which the destinations consume them. A finished
// chunk adds one to the destination's counter of the 128-token tile it belongs to; the consumer's
// TMA producer waits until a tile's counter has reached (number of steps so far) x (chunks of the
// tile). Only CTAs that are running take chunks, so no CTA ever waits for work held by a CTA that
// has not started.
// A run of chunks of the exchange queue: sub-blocks sub0 .. sub0 + n - 1 (16 tokens each) of
// kind 0 (Q) or 1 (K and V), sent at ring step `step` (to rank - step).
struct ExchangeRange { short kind, step; int sub0, n; };
constexpr int kMaxExchangeRanges = 32;

struct ExchangeParams {
    const void*  q; const void* k; const void* v;   // [s_loc, n_heads_total, 128] bf16, dense
    const void*  gamma_q; const void* gamma_k;      // [128] bf16
    const float* cos_tab; const float* sin_tab;     // [s_loc, 64] fp32: this rank's rows
    unsigned char* dst_q[8]; unsigned char* dst_k[8]; unsigned char* dst_v[8];   // per destination rank
    unsigned int*  tile_words[8];                   // destination's counters for this source: [Q | KV][tiles]
    // When not null: the destination walks K/V as at most two segments of its buffer, tokens
    // [start, world * s_loc) then [0, start) with start = destination * s_loc, and has one counter
    // per 128-token tile of that walk, shared by all sources (s_loc is a multiple of 16 then, so a
    // chunk never straddles two tiles). K/V chunks count there instead of tile_words.
    unsigned int*  kv_walk_words[8];
    unsigned int*  next_chunk;                      // local, zero before the launch
    ExchangeRange  order[kMaxExchangeRanges];       // the queue, in the order the attention needs the rows
    int            n_ranges;
    unsigned int   total_chunks;                    // sum of order[].n = 2 * world * ceil(s_loc / 16)
    int   s_loc, n_heads_total, heads_per_rank, world, rank;
    int   unit_rows;        // head rows of one token moved by one bulk copy: the largest divisor of heads_per_rank <= 16
    int   tokens_per_buf;   // tokens per staging buffer: min(4, 16 / unit_rows)
    unsigned int n_sms;     // CTAs that run at a time (one per SM)
    int   enabled;
    float eps;
};
constexpr int kExchangeTokens = 16;   // tokens per chunk: 8 chunks per 128-token tile

#ifdef __CUDACC__
#define F2K_HOST_DEVICE __host__ __device__
#else
#define F2K_HOST_DEVICE
#endif
// Tile of a destination's two-piece K/V walk (tokens [start, all) then [0, start)) that token g
// of the whole sequence falls into: the counter a chunk starting at g counts in.
F2K_HOST_DEVICE inline int kv_walk_tile(int g, int start, int all) {
    const int tiles_a = (all - start + kTileN - 1) / kTileN;
    return g >= start ? (g - start) / kTileN : tiles_a + g / kTileN;
}

struct AttnParams {
    // 4-D tensor maps, dims (fastest first): head_dim, head, token, batch;
    // box = 64 x 1 x 128 x 1 elements, 128-byte swizzle, zero fill out of bounds.
    CUtensorMap tm_q[kMaxQSeg];
    CUtensorMap tm_k[kMaxKvSeg];
    CUtensorMap tm_v[kMaxKvSeg];

    // Output per query segment (bf16), strides in elements.
    void*     o_ptr[kMaxQSeg];
    long long o_tok_stride[kMaxQSeg];
    long long o_batch_stride[kMaxQSeg];

    int q_len[kMaxQSeg];              // tokens in each query segment
    int q_tile_start[kMaxQSeg + 1];   // prefix sum of ceil(len / 128)
    int kv_len[kMaxKvSeg];
    int kv_tile_start[kMaxKvSeg + 1];
    int n_qseg;
    int n_kvseg;
    int n_q_tiles;
    int n_kv_tiles;

    int   n_heads;
    int   batch;
    float scale_log2;                 // softmax scale * log2(e)

    int* status;                      // device word, AttnStatus bits OR-ed in

    long long wait_limit_clk;         // bounded waits inside the CTA (0 = kDefaultWaitClk)
    long long peer_wait_limit_clk;    // bounded waits on kv_ready / q_ready words (0 = kDefaultPeerWaitClk)

    // Sequence-parallel use: key/value segment i may still be on its way into this GPU's memory
    // when the kernel starts (a copy engine is bringing it over NVLink, one group of
    // kv_ready_heads_per_group heads at a time). When kv_ready[i] is not null the TMA producer of
    // a CTA working on head h waits, bounded, until the word kv_ready[i][h / heads_per_group]
    // equals kv_ready_value before it touches the segment. The word is written after the copy,
    // in stream order, by the copying stream. Null for data that is already in place.
    const unsigned int* kv_ready[kMaxKvSeg];
    unsigned int        kv_ready_value;
    int                 kv_ready_heads_per_group;
    // A segment filled by several writers: the producer waits for kv_ready_words consecutive words
    // starting at the one above (0 or 1 = that word alone).
    int                 kv_ready_words;

    // Per-tile readiness (fused head exchange): when ready_per_tile is set, q_ready[i] / kv_ready[i]
    // point at one counter per 128-token tile of segment i; a tile may be fetched once its counter
    // has reached ready_uses * ceil(tokens in the tile / kExchangeTokens) ("not before", modulo 2^32).
    int          ready_per_tile;
    unsigned int ready_uses;

    // Head-exchange use (tokens sharded outside the attention, heads inside): query segment i is
    // written into this GPU's memory by rank i's kernel, which then stores kv_ready_value (or a
    // later call's value) to q_ready[i]; the TMA producer waits for that word, bounded, before it
    // fetches a query tile of the segment. Null for data that is already in place.
    const unsigned int* q_ready[kMaxQSeg];

    // When done_counter is not null, the last CTA to finish stores done_value to each of the
    // n_done words done_flag[] (words in this and in the peers' memory) after every output row of
    // the launch has been written: outputs may go straight into other GPUs' buffers (o_ptr), and
    // this tells their owners. The counter is left at zero for the next launch.
    // If a CTA of the launch gave up on a wait, its output rows were not written: the last CTA then
    // stores done_value to fail_flag[] (same owners as done_flag[]) BEFORE it publishes done, so that
    // nobody who sees "done" can miss the failure.
    unsigned int* done_counter;
    unsigned int* done_flag[8];
    unsigned int* fail_flag[8];
    int           n_done;
    unsigned int  done_value;

    // 0: CTAs are numbered pair-fastest (all tile pairs of a head are neighbours: the K/V of a
    // head are shared through L2 by CTAs that run together). 1: head-fastest, so that the first
    // CTAs to run are those of the first query segments (head exchange: the local tokens).
    int grid_head_fastest;

    ExchangeParams xchg;
};

}  // namespace f2k
