// Internal interface between the decoder step and the communicator.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace mynn {
int comm_world();
int comm_rank();
// sum over ranks; dst may equal src; world == 1 degenerates to a copy
int comm_all_reduce(cudaStream_t st, void *dst, const void *src, size_t n, int dtype);
// dst [world][bytes_per_rank] <- every rank's src
int comm_all_gather(cudaStream_t st, void *dst, const void *src, size_t bytes_per_rank);
}  // namespace mynn
