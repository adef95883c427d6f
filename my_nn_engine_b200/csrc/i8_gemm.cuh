// Internal interface of the tcgen05 (kind::i8) weight-streaming DequantMatMul.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace mynn {
constexpr int kI8MaxRows = 32;  // activation rows per launch: 3 limbs x 32 rows = 96 accumulator columns
// Scratch layout: [0,256) status word, [256,512) activation row scales, then the int8 limb matrix.
size_t i8_gemm_workspace_bytes(int M, int K);
bool i8_gemm_supported(int M, int N, int K, const void *wq, int act_dtype, int out_dtype);
int i8_gemm_launch(cudaStream_t st, void *out, const void *act, const int8_t *wq, const void *scale, const void *resid,
                   int M, int N, int K, int act_dtype, int out_dtype, void *workspace, size_t workspace_bytes);
extern int g_i8_split_override;
}  // namespace mynn
