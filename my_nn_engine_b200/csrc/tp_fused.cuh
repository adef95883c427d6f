// Internal interface of the fused tensor-parallel reduction (tp_fused.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace mynn {

constexpr int kTpMaxRanks = 8;  // ranks of one NVLink domain; sizes the flag and pointer arrays below

// Header of the block of device memory every rank shares with its peers (cudaIpc); the two f32 partial-sum buffers
// follow at the byte offsets TpPeers::part_off (identical on every rank).
struct TpLocal {
    uint32_t flags[kTpMaxRanks];  // flags[r] = last step number rank r has announced to this rank
    uint32_t epoch;     // step number of the last completed reduction on this rank
    uint32_t ticket;    // CTA arrival counter of the running reduction
    int status;         // 21 = a wait for a peer ran out of time
    uint32_t pad[5];
};
static_assert(sizeof(TpLocal) == 64, "TpLocal is one 64-byte header");

struct TpPeers {
    TpLocal *local;       // this rank's block
    TpLocal *remote[kTpMaxRanks];   // every rank's block as mapped into this process (remote[rank] == local)
    size_t part_off[2];   // byte offsets of the two partial-sum buffers inside a block
    int rank, world;
};

__host__ __device__ inline float *tp_part(TpLocal *blk, size_t off) { return (float *)((char *)blk + off); }

// sum over ranks of part[buf] -> x = round(x + round(sum)); if w != null: y = round(RMSNorm(x) * w) -> limbs + row scales
// in `workspace` (the DequantMatMul workspace).  rows <= 32.
int launch_tp_reduce_norm_limbs(cudaStream_t st, int dtype, const TpPeers &peers, int buf, void *workspace,
                                size_t workspace_bytes, void *x, const void *w, float eps, int rows, int D);

}  // namespace mynn
