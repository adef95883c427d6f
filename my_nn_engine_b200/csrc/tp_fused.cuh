// Internal interface of the fused tensor-parallel reduction (tp_fused.cu) and of the two DequantMatMul forms that feed it
// and are fed by it (i8_gemm.cu).
//
// Data flow of one reduction over `world` ranks (rows m of the step are dealt out: row m belongs to rank m % world):
//   1. the row-parallel DequantMatMul (o_proj, down_proj) of every rank STORES its f32 partial row m straight into slot
//      [its own rank][m / world] of the partial buffer of the rank that owns row m (plain peer stores over NVLink, issued
//      from the GEMM epilogue).  Every value travels as an 8-byte word {value, tag} written with one store, the tag being
//      the number of the reduction: the receiver needs no flag and the sender no fence (a system-scope release costs
//      microseconds, and there would be one per CTA and destination);
//   2. the owner's reduction kernel reads the `world` partial rows from its OWN memory, re-reading a word until it carries
//      the tag of this reduction, adds them in rank order, finishes the row (residual add, RMSNorm, activation limbs) and
//      stores the limbs and the row scale into the limb buffer of EVERY rank, followed by a release increment of a counter
//      in that rank's header (the limbs are read by TMA, so they cannot carry tags);
//   3. the column-parallel DequantMatMul that follows (qkv, gate/up, lm_head) streams its weights at once and only holds
//      its activation (limb) loads back until all rows have arrived.
// Every rank moves rows/world of the partial sums in and 3 bytes per element of its own rows out, instead of reading
// every rank's whole partial tensor; the transfers overlap the GEMM epilogue and the weight prefetch of the next GEMM.
// No load ever crosses NVLink, and nothing here uses multicast.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace mynn {

constexpr int kTpMaxRanks = 8;  // ranks of one NVLink domain; sizes the counter and pointer arrays below

// Header of the block of device memory every rank shares with its peers.  All counters are monotonic (they wrap modulo
// 2^32 and are compared by signed difference); a block must be zeroed once before its first use.
struct TpHeader {
    uint32_t gather_cnt;                // limb rows delivered so far by the reductions of all ranks (peers add)
    // written by this rank only (the last CTA of each of its reduction kernels):
    uint32_t part_tag[2];               // number of reductions run on each partial buffer = tag of the last one
    uint32_t gather_expected;           // value gather_cnt reaches once every reduction completed so far has been delivered
    uint32_t ticket;                    // CTA arrival counter of the running reduction kernel
    int status;                         // 21: a wait for partial sums ran out of time; 22: a wait for limb rows did
    uint32_t pad[64 - 6];
};
static_assert(sizeof(TpHeader) == 256, "TpHeader is one 256-byte header");

// Geometry of a block; identical on every rank.  rows_cap = rows one rank can own = ceil(max_rows / world).
struct TpLayout {
    int world, max_rows, hidden, rows_cap, nc;  // nc = limb rows of the gathered matrix (3 per activation row, padded)
    size_t part_off[2], limb_off, ascale_off, bytes;
};
TpLayout tp_layout(int max_rows, int hidden, int world);

// A rank's view of the group: its own block and every rank's block as mapped into this process (blocks[rank] == own).
struct TpPeers {
    char *blocks[kTpMaxRanks];
    int rank, world;
    TpLayout lay;
};

__host__ __device__ inline TpHeader *tp_header(char *blk) { return reinterpret_cast<TpHeader *>(blk); }

// What the tcgen05 DequantMatMul kernel needs to take part (passed by value in its parameters).
struct I8Tp {
    int mode;                          // 0: plain; 1: scatter partial rows to their owners; 2: activation limbs are gathered rows
    int world, rank, rows_cap;
    uint2 *part[kTpMaxRanks];          // mode 1: partial buffer of every rank, {value, tag} words, layout [source][local row][N]
    const uint32_t *part_tag;          // mode 1: own header's count of reductions on this buffer; this product's tag is that + 1
    const uint32_t *gather_cnt;        // mode 2: own header's counter of delivered limb rows and the value it has to reach
    const uint32_t *gather_expected;
    int *status;                       // own header's status word
};

// Row-parallel DequantMatMul with the scatter epilogue.  act == nullptr: limbs already in `workspace`.
int launch_tp_gemm_scatter(cudaStream_t st, const TpPeers &peers, int buf, const void *act, const int8_t *wq, const float *scale,
                           int M, int N, int K, int act_dtype, void *workspace, size_t workspace_bytes);
// sum over ranks of the partial rows this rank owns -> x[m] = round(x[m] + round(sum)); y = round(RMSNorm(x[m]) * w) -> limbs
// + row scale into every rank's limb buffer.  skip_signal (test aid): do everything except the deliveries to the peers.
int launch_tp_reduce_norm_gather(cudaStream_t st, int dtype, const TpPeers &peers, int buf, void *x, const void *w, float eps, int M,
                                 int skip_signal);
// Column-parallel DequantMatMul over the gathered limb rows.  `workspace` only carries the kernel's status word.
int launch_tp_gemm_gathered(cudaStream_t st, const TpPeers &peers, void *out, const int8_t *wq, const void *scale, int M, int N,
                            int out_dtype, void *workspace, size_t workspace_bytes);

}  // namespace mynn
