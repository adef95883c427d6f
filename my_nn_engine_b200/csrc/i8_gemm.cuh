// Internal interface of the tcgen05 (kind::i8) weight-streaming DequantMatMul.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace mynn {
constexpr int kI8MaxRows = 32;  // activation rows per launch: 3 limbs x 32 rows = 96 accumulator columns
// Scratch layout: [0,256) status word, [256,512) activation row scales, then the int8 limb matrix.
size_t i8_gemm_workspace_bytes(int M, int K);
int i8_gemm_limb_rows(int M);  // rows of the limb matrix for M activation rows (3 per row, padded to an MMA width)
bool i8_gemm_supported(int M, int N, int K, const void *wq, int act_dtype, int out_dtype);
int i8_gemm_launch(cudaStream_t st, void *out, const void *act, const int8_t *wq, const void *scale, const void *resid,
                   int M, int N, int K, int act_dtype, int out_dtype, void *workspace, size_t workspace_bytes);
// Lean kernel for at most 4 activation rows over a small weight matrix (gemv_lean.cu): same workspace contract and
// bit-identical results; i8_gemm_launch dispatches to it.
bool gemv_lean_supported(int M, int N, int K, const void *wq);
int gemv_lean_launch(cudaStream_t st, void *out, const void *act, const int8_t *wq, const void *scale, const void *resid, int M, int N,
                     int K, int act_dtype, int out_dtype, void *workspace, size_t workspace_bytes);
struct I8Tp;  // tp_fused.cuh
int i8_gemm_launch_tp(cudaStream_t st, void *out, const void *act, const int8_t *wq, const void *scale, const void *resid,
                      int M, int N, int K, int act_dtype, int out_dtype, void *workspace, size_t workspace_bytes, const I8Tp *tp,
                      const int8_t *limbs_ext, const float *ascale_ext);
// Fused producers: leave limbs + row scales in `workspace`; the following i8_gemm_launch is called with act == nullptr.
// rms_norm: y = round(RMSNorm(x) * w); with part != nullptr first sum_out = round(x + round(part)) is stored and
// normalised.  norm_out may be null.  swiglu: h = round(swish(gate) * up).
int launch_rms_norm_limbs(cudaStream_t st, int dtype, void *workspace, size_t workspace_bytes, void *norm_out, void *sum_out,
                          const void *x, const float *part, const void *w, float eps, int rows, int D);
int launch_swiglu_limbs(cudaStream_t st, int dtype, void *workspace, size_t workspace_bytes, const void *gate, const void *up,
                        int rows, int F, long long in_stride);
// TMA descriptor of a 2D int8 tensor [rows][cols] (row stride ld bytes), box = box_rows x 128 bytes, 128-byte swizzle.
int make_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);
bool tensor_map_api_available();

// Large-M (prefill) variant: activations as two int8 limbs per element, 128 x 128-token tiles, persistent CTAs.
// Scratch layout: [0,256) status word, then M row scales (rounded up to 256 bytes), then the [2M][K] limb matrix.
size_t i8_prefill_workspace_bytes(int M, int K);
bool i8_prefill_supported(int M, int N, int K, const void *wq, int act_dtype, int out_dtype);
int i8_prefill_launch(cudaStream_t st, void *out, const void *act, const int8_t *wq, const void *scale, const void *resid,
                      int M, int N, int K, int act_dtype, int out_dtype, void *workspace, size_t workspace_bytes);
// Fused producers for the prefill kernel (rows > 32): leave two limbs per element + row scales in `workspace`; the following
// i8_prefill_launch is called with act == nullptr.  prefill_fused_supported: 16-bit dtype, K % 16 == 0, 16-byte aligned inputs.
bool prefill_fused_supported(int dtype, int K, const void *a, const void *b);
int launch_rms_norm_limbs2(cudaStream_t st, int dtype, void *workspace, size_t workspace_bytes, const void *x, const void *w, float eps,
                           int rows, int D);
int launch_swiglu_limbs2(cudaStream_t st, int dtype, void *workspace, size_t workspace_bytes, const void *gate, const void *up, int rows,
                         int F, long long in_stride);
// QuantizedMatMul (int8 x int8, per-row or per-tensor lhs scale, per-channel rhs scale) on the same persistent kernel
// with one accumulator column per lhs row.  workspace: 256 bytes holding the status word.
bool i8_w8a8_supported(int M, int N, int K, const void *lhs, const void *rhs);
int i8_w8a8_launch(cudaStream_t st, void *out, const int8_t *lhs, const void *lhs_scale, int lhs_scale_per_row, const int8_t *rhs,
                   const void *rhs_scale, int M, int N, int K, int dtype, void *workspace, size_t workspace_bytes);
#ifdef MYNN_TUNING
extern unsigned long long *g_i8_timing;
extern int g_i8_stages_override, g_i8_timing_slots, g_i8_timing_next;
#endif
}  // namespace mynn
