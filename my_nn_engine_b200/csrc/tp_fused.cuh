// Internal interface of the fused tensor-parallel reduction (tp_fused.cu) and of the DequantMatMul form that feeds it
// (i8_gemm.cu).
//
// Data flow of one reduction over `world` ranks:
//   1. the row-parallel DequantMatMul (o_proj, down_proj) of every rank STORES its f32 partial sums straight into slot
//      [its own rank] of the partial buffer of EVERY rank (plain 4-byte peer stores over NVLink, issued from the GEMM
//      epilogue, 128 contiguous bytes per warp).  A slot that holds no value yet holds the EMPTY word 0xFFFFFFFF, a NaN
//      pattern no product ever stores (a NaN result is delivered as the canonical NaN), so the value itself tells the
//      receiver that it has arrived: no flag, no tag, and no fence on the sender (a system-scope release costs microseconds,
//      and there would be one per CTA and destination);
//   2. one kernel per rank reads the `world` partial rows from its OWN memory, re-reading a 16-byte piece until none of its
//      words is EMPTY, puts EMPTY back, adds the values in rank order (every rank computes the identical sum), and finishes
//      the row: residual add, RMSNorm, activation limbs of the next DequantMatMul in the local workspace.
// One NVLink hop per reduction, 4 bytes per value, no load ever crosses NVLink, no collective call, nothing uses multicast.
// (Measured against it on the same step: every value as an 8-byte {value, number of the reduction} word, which needs no
// EMPTY words but moves twice the bytes over NVLink and through the reducing kernel; reading the peers' partial sums with
// peer loads behind a flag barrier, 3.89 ms per step at 2 ranks against 3.69 with those 8-byte words and 3.47 with these; a reduce-scatter by rows plus an all-gather of
// the finished limb rows, which moves 1/world of the bytes but needs two hops and a system-scope release per hop, 4.24 ms.)
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace mynn {

constexpr int kTpMaxRanks = 8;  // ranks of one NVLink domain; sizes the pointer arrays below

constexpr uint32_t kTpEmpty = 0xFFFFFFFFu;  // "no value yet" in a partial buffer

// Header of the block of device memory every rank shares with its peers.  Before its first use a block's header is zeroed
// and every byte behind it set to 0xFF (mynn_b200_tp_block_init).
struct TpHeader {
    int status;  // 21: a wait for partial sums ran out of time
    uint32_t pad[63];
};
static_assert(sizeof(TpHeader) == 256, "TpHeader is one 256-byte header");

// Geometry of a block; identical on every rank.
struct TpLayout {
    int world, max_rows, hidden;
    size_t part_off[2], bytes;  // each partial buffer: [source rank][row][hidden] f32 words (kTpEmpty: not there yet)
};
TpLayout tp_layout(int max_rows, int hidden, int world);
int tp_block_init(cudaStream_t st, char *block, size_t bytes);  // header zero, every partial-sum word EMPTY

// A rank's view of the group: its own block and every rank's block as mapped into this process (blocks[rank] == own).
struct TpPeers {
    char *blocks[kTpMaxRanks];
    int rank, world;
    TpLayout lay;
};

__host__ __device__ inline TpHeader *tp_header(char *blk) { return reinterpret_cast<TpHeader *>(blk); }

// What the tcgen05 DequantMatMul kernel needs to deliver its outputs as partial sums (passed by value in its parameters).
struct I8Tp {
    int mode;                   // 0: plain output; 1: the outputs go to slot [rank] of every rank's partial buffer
    int world, rank, max_rows;
    uint32_t *part[kTpMaxRanks];  // partial buffer of every rank
    int skip;                   // test aid: deliver nothing
};

// Row-parallel DequantMatMul whose f32 outputs go to every rank as partial sums.  act == nullptr: limbs already in
// `workspace`.  skip_delivery (test aid): run the product but deliver nothing.
int launch_tp_gemm_push(cudaStream_t st, const TpPeers &peers, int buf, const void *act, const int8_t *wq, const float *scale, int M,
                        int N, int K, int act_dtype, void *workspace, size_t workspace_bytes, int skip_delivery);
// sum over ranks of the partial rows -> x = round(x + round(sum)); if w != null: y = round(RMSNorm(x) * w) -> limbs + row
// scales in `workspace` (the DequantMatMul workspace of the product that follows).  after_push: the kernel in front of this
// one on the stream is the delivering DequantMatMul of the same reduction (the two may then overlap).
int launch_tp_reduce_norm_limbs(cudaStream_t st, int dtype, const TpPeers &peers, int buf, void *workspace, size_t workspace_bytes,
                                void *x, const void *w, float eps, int M, bool after_push);

}  // namespace mynn
