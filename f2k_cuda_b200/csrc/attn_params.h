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
};

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

    // Sequence-parallel use: key/value segment i may still be on its way into this GPU's memory
    // when the kernel starts (a copy engine is bringing it over NVLink, one group of
    // kv_ready_heads_per_group heads at a time). When kv_ready[i] is not null the TMA producer of
    // a CTA working on head h waits, bounded, until the word kv_ready[i][h / heads_per_group]
    // equals kv_ready_value before it touches the segment. The word is written after the copy,
    // in stream order, by the copying stream. Null for data that is already in place.
    const unsigned int* kv_ready[kMaxKvSeg];
    unsigned int        kv_ready_value;
    int                 kv_ready_heads_per_group;

    // Head-exchange use (tokens sharded outside the attention, heads inside): query segment i is
    // written into this GPU's memory by rank i's kernel, which then stores kv_ready_value (or a
    // later call's value) to q_ready[i]; the TMA producer waits for that word, bounded, before it
    // fetches a query tile of the segment. Null for data that is already in place.
    const unsigned int* q_ready[kMaxQSeg];

    // When done_counter is not null, the last CTA to finish stores done_value to each of the
    // n_done words done_flag[] (words in this and in the peers' memory) after every output row of
    // the launch has been written: outputs may go straight into other GPUs' buffers (o_ptr), and
    // this tells their owners. The counter is left at zero for the next launch.
    unsigned int* done_counter;
    unsigned int* done_flag[8];
    int           n_done;
    unsigned int  done_value;
};

}  // namespace f2k
