/*
 * mynn_b200 — C ABI of the B200 (sm_100a) decode-path library.
 *
 * Drop-in boundary for the LLM decode hot path of kcvlex/my-nn-engine: the int8 weight-only
 * DequantMatMul and GQA decode attention over the KV cache, the small operators between them, the
 * tensor-parallel all-reduce, and a whole-step entry with the exact model_init / model /
 * model_destroy signatures the engine's CUDA session resolves from its generated library.
 *
 * Conventions
 *   - Every function returns 0 on success and a negative MYNN_E_* code otherwise; it never calls
 *     exit() and never traps the device (the engine's generated code exits the process on any CUDA
 *     error, src/codegen/cuda/cpp/common.cuh:7-43).  mynn_b200_last_error() gives the text.
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream).  Launchers only enqueue.
 *   - All tensor pointers are DEVICE pointers unless a parameter is documented as host memory.
 *   - dtype codes: MYNN_F32 / MYNN_BF16 / MYNN_F16.  bf16 and f32 are the engine's float storage types
 *     (src/tensor/types.rs:278-282); f16 is an extension with the same store points.
 *   - There is no CPU fallback: without a CUDA device every launcher returns MYNN_E_CUDA.
 *   - Thread safety: calls on distinct streams/states may run concurrently; a model state is
 *     single-caller, as the engine serialises runs with its CUDA_LOCK (src/session/cuda.rs:36-40).
 */
#ifndef MYNN_B200_H_
#define MYNN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { MYNN_F32 = 0, MYNN_BF16 = 1, MYNN_F16 = 2 };
enum { MYNN_OK = 0, MYNN_E_ARG = -1, MYNN_E_CUDA = -2, MYNN_E_UNSUPPORTED = -3, MYNN_E_COMM = -4, MYNN_E_STATE = -5 };
/* weight layouts of DequantMatMul: [N,K] with per-row scale (axis 0, what DequantGemmFusion produces)
 * or [K,N] with per-column scale (axis 1, the unfused DequantizeLinear -> MatMul graph). */
enum { MYNN_W_NK = 0, MYNN_W_KN = 1 };

const char *mynn_b200_last_error(void);
/* Process-wide options.  No counterpart in the engine (its generated code has no run-time switches); they exist so that the
 * bounded device-side waits and the kernel choices described below can be exercised by an integrator's tests.
 *   MYNN_OPT_WAIT_BUDGET_US   time limit of every bounded device-side wait (mbarrier waits of the tcgen05 kernels, the
 *                             cross-GPU flag wait of the fused tensor-parallel reduction), in microseconds; default
 *                             2,000,000.  Applies to the CURRENT device.  When a wait runs out the kernel records a status
 *                             code, finishes without the missing data and returns; the next *_check / model call reports it.
 *   MYNN_OPT_KSPLIT           force the cluster K split of the small-batch DequantMatMul kernels: 0 automatic, else 1, 2, 4
 *                             or 8.  The results do not depend on it (integer accumulation), which a test can verify.
 *   MYNN_OPT_PREFILL_ATTENTION  kernels for Sq > 1: 1 (default) tcgen05 with two heads per CTA where possible; 2 / 3 tcgen05
 *                             with one head per CTA, probabilities through shared / tensor memory; 0 the mma.sync tiled
 *                             kernel only; -1 the row-serial kernel only.
 *   MYNN_OPT_INJECT_STALL     test aid for the bounded waits, never set in production: 1 = the NEXT small-batch tcgen05
 *                             DequantMatMul launch leaves out its last TMA stage, so that its MMA thread's wait runs out
 *                             (status 2 in the workspace); 2 = the NEXT row-parallel product of a tensor-parallel step delivers
 *                             none of its partial sums, so that the reductions' waits run out (status 21 / MYNN_E_COMM).  Nothing faults or
 *                             hangs: the kernels return after the wait budget.
 *   MYNN_OPT_FUSE_ROPE        1 (default): in a decode step of the model entry points the attention kernel rotates q and the
 *                             new key itself and appends the new key / value rows to the cache (one launch less per layer);
 *                             0: RoPE + append run as a kernel of their own in front of it.  Read when a model's step is
 *                             recorded.  The rotated rows have the same bits either way; the softmax takes the new row in a tile of its own,
 *                             so outputs agree to rounding of the f32 sums, not to the bit.
 *   MYNN_OPT_DECODE_RING      1 (default): the 16-bit decode attention kernel takes its K / V tiles from per-warp rings in
 *                             shared memory that the TMA engine fills; 0: every thread loads its fragments from global
 *                             memory itself.  Same arithmetic on the same fragments: the outputs are bit-identical whenever
 *                             both forms use the same number of splits, which a test verifies.  Read at launch (a model
 *                             reads it when its step is recorded). */
enum {
    MYNN_OPT_WAIT_BUDGET_US = 1, MYNN_OPT_KSPLIT = 2, MYNN_OPT_PREFILL_ATTENTION = 3, MYNN_OPT_INJECT_STALL = 4,
    MYNN_OPT_FUSE_ROPE = 5, MYNN_OPT_DECODE_RING = 6
};
int mynn_b200_set_option(int option, long long value);

/* Library/ABI version and the SM architecture the kernels were compiled for (100 for sm_100a). */
int mynn_b200_abi_version(void);
int mynn_b200_compiled_arch(void);

/* ---------------------------------------------------------------------------------------------
 * DequantMatMul: out[m,n] = scale[n] * sum_k act[m,k] * wq[n,k]   (out in scale dtype)
 * Replaces: Operator::DequantMatMul (src/graph/operator.rs:240-244; operand slots LHS, RHS, SCALE, WORKSPACE at
 * :1109-1113) and its three CUDA kernels chosen in src/codegen/cuda.rs:1518-1652 (dequant_gemv.cuh:11-59,
 * dequant_matmul_wmma.cuh:87-192, dequant_matmul.cuh:13-51); argument order follows the generated launch
 * (out, act, wq, scale, M, N, K) with the operator's workspace slot last.
 * act [M,K] act_dtype; wq int8 [N,K] (MYNN_W_NK) or [K,N] (MYNN_W_KN); scale [N] and out [M,N] out_dtype.
 * Any M >= 0, N, K is accepted (M == 0 is a no-op).
 * workspace: device scratch of mynn_b200_dequant_matmul_workspace_bytes(M, N, K) bytes, 256-byte aligned and ZEROED
 * before its first use (its first word is a status flag, see mynn_b200_dequant_matmul_check).  With a workspace,
 * [N,K] problems of up to 32 rows with K % 16 == 0 run on the tcgen05 int8 tensor-core kernel (exact int32
 * accumulation of 23-bit fixed-point activations).  With workspace == NULL, or for other shapes, kernels that need no
 * scratch are used (mma.sync streaming kernel for K % 64 == 0, N % 16 == 0, M <= 32; a generic kernel otherwise).
 * Calls that share a workspace must be ordered on one stream. */
size_t mynn_b200_dequant_matmul_workspace_bytes(int M, int N, int K);
int mynn_b200_dequant_matmul(void *stream, void *out, const void *act, const int8_t *wq, const void *scale, int M,
                             int N, int K, int act_dtype, int out_dtype, int w_layout, void *workspace,
                             size_t workspace_bytes);

/* Same product followed by a fused epilogue used by the decoder step (no counterpart kernel in the engine,
 * which runs these as separate elementwise launches, src/codegen/cuda/kernel.rs:723-950):
 *   out = round(residual + round(product))      (two store points kept; out may alias residual)
 * wq must be [N,K]. */
int mynn_b200_dequant_matmul_residual(void *stream, void *out, const void *act, const int8_t *wq, const void *scale,
                                      const void *residual, int M, int N, int K, int dtype, void *workspace,
                                      size_t workspace_bytes);

/* DequantMatMul with the activations of the PREVIOUS mynn_b200_dequant_matmul call on the same workspace (same M, K
 * and activation tensor): the limb conversion is skipped.  For several weight matrices applied to one activation tensor
 * (q/k/v, gate/up when they are not stored adjacently).  Needs the tensor-core path: workspace, M <= 32, K % 16 == 0. */
int mynn_b200_dequant_matmul_same_act(void *stream, void *out, const int8_t *wq, const void *scale, int M, int N, int K,
                                      int act_dtype, int out_dtype, void *workspace, size_t workspace_bytes);

/* Synchronises the stream and reads the workspace status word: MYNN_E_CUDA if a bounded pipeline wait inside the
 * tcgen05 kernel expired (the outputs of that call are then invalid), MYNN_OK otherwise.  A reported expiry is cleared,
 * so the workspace can be used again. */
int mynn_b200_dequant_matmul_check(void *stream, const void *workspace);

/* ---------------------------------------------------------------------------------------------
 * Attention (decode and generic).  out = softmax(scale * Q K^T [causal]) V with GQA.
 * Replaces: Operator::Attention (src/graph/operator.rs:193-197), CUDA dispatch src/codegen/cuda.rs:1194-1403,
 * kernels attention_decode (cpp/attention.cuh:495-606) and attention / attention_tc (:50-489).
 * q [B,Hq,Sq,D], k/v [B,Hkv,cache_seq_len,D] contiguous, out [B,Hq,Sq,D], all `dtype`.
 * active_seq_kv: valid kv rows.  If active_seq_kv_dev != NULL the value is read on the device from that int32
 * (so a captured graph can be replayed as the sequence grows) and the host value is only an upper bound used
 * for grid sizing.  workspace: device scratch of at least mynn_b200_attention_workspace_bytes(); it may be
 * NULL when Sq > 1 or when the generic kernel is taken (D not 64/128, f32, or group size > 8). */
size_t mynn_b200_attention_workspace_bytes(int B, int Hq, int Hkv, int D, int cache_seq_len);
int mynn_b200_attention(void *stream, void *out, const void *q, const void *k, const void *v, float scale, int B,
                        int Hq, int Hkv, int Sq, int D, int cache_seq_len, int active_seq_kv,
                        const int32_t *active_seq_kv_dev, int is_causal, int dtype, void *workspace,
                        size_t workspace_bytes);
/* Attention with the additive MASK operand (slot ATTENTION_MASK, src/graph/operator.rs:1027; builder
 * crates/llm/src/builder.rs:466-515): qk = scale * (q . k) + mask before the softmax, then as mynn_b200_attention.
 * mask (`dtype`) is addressed as the engine's launch addresses it (src/codegen/cuda.rs:1297-1325):
 *   mask[(b * Hq + h) * mask_outer_stride + sq * mask_row_stride + kv_row],
 * mask_row_stride = last dim of the mask (0 if its second-to-last dim is 1), mask_outer_stride = product of its last two
 * dims (0 if all leading dims are 1).  Every shape runs on the row-serial kernel that follows the CPU recurrence
 * (src/codegen/cpu/translator.rs:4854-4881); the Llama decoder never passes a mask (crates/llm/src/decoder.rs:351-358). */
int mynn_b200_attention_masked(void *stream, void *out, const void *q, const void *k, const void *v, const void *mask,
                               long long mask_outer_stride, long long mask_row_stride, float scale, int B, int Hq, int Hkv,
                               int Sq, int D, int cache_seq_len, int active_seq_kv, const int32_t *active_seq_kv_dev,
                               int is_causal, int dtype);
/* Prefill chunks (Sq >= 64, D 64/128, 16-bit, 16-byte aligned tensors) run on a TMA-fed tcgen05 kernel whose pipeline
 * waits are bounded.  This call synchronises the stream and returns MYNN_E_CUDA if one of them expired in an earlier
 * attention call (the engine checks cudaGetLastError after its launches: src/codegen/cuda/cpp/common.cuh). */
int mynn_b200_attention_check(void *stream);

/* Decode attention (one query row per sequence) that takes no workspace and allocates nothing.  This entry point
 * has no counterpart in the engine.  It exists for callers that cannot hand over scratch memory and cannot allocate
 * any: the engine's Attention operator has no workspace operand and its planner fixes every device buffer when the
 * model is compiled, so code generated for that operator has nothing to pass and no allocator to call mid-step.
 * The split-KV partial results go to an array built into the library, mynn_b200_attention_decode_noalloc_max_bytes()
 * (4 MiB) of device memory that every GPU using the library holds until the process exits.
 *   - Same tensors and meaning as mynn_b200_attention with Sq = 1; bf16/f16, head_dim 64 or 128, at most 8 query heads
 *     per kv head, 16-byte aligned pointers; anything else, or a problem whose partial results exceed the array,
 *     returns MYNN_E_UNSUPPORTED with the sizes in the error text.
 *   - The first call on a device resolves the array's device address (once per device, that device current); issue
 *     that first call before starting any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents; its arrival counters are re-zeroed on
 *     the stream by each call.  Calls whose kernels may overlap on the GPU race on it: keep them ordered.
 *   - No cudaMalloc, cudaFree or other allocating routine is called. */
size_t mynn_b200_attention_decode_noalloc_max_bytes(void);
int mynn_b200_attention_decode_noalloc(void *stream, void *out, const void *q, const void *k, const void *v, float scale,
                                       int B, int Hq, int Hkv, int D, int cache_seq_len, int active_seq_kv,
                                       const int32_t *active_seq_kv_dev, int dtype);

/* KVCacheUpdate: cache[bh, offset+t, :] = new[bh, t, :] in place.
 * Replaces: kvcache_update (cpp/kvcache_update.cuh:6-26, dispatch src/codegen/cuda.rs:2176-2228).
 * Unlike the engine (no bounds check) rows that would land past cache_seq_len are rejected with MYNN_E_ARG when
 * the offset is given on the host, and skipped on the device when offset_dev is used. */
int mynn_b200_kv_cache_update(void *stream, void *cache, const void *new_kv, int BH, int cache_seq_len,
                              int new_seq_len, int D, int offset, const int32_t *offset_dev, int dtype);

/* QuantizingKVCacheUpdate (the engine's `quant_kv_cache` option): the new rows are quantized to int8 with one scale
 * per token, cache[bh, offset+t, :] = q, scale[bh, offset+t] = s, in place.
 *   s = max_d|x| * (1/127); inv = 127 / max (0 for an all-zero row); q = trunc(x * inv +- 0.5) clamped to [-128, 127]
 * which is the CPU backend's arithmetic (src/codegen/cpu/translator.rs:4090-4372), so the bytes are identical to it.
 * Replaces: quantizing_kvcache_update (cpp/quantizing_kvcache_update.cuh, dispatch src/codegen/cuda.rs:2116-2174).
 * cache int8 [BH, cache_seq_len, D]; scale [BH, cache_seq_len] and new_kv [BH, new_seq_len, D] in `dtype`.
 * Bounds are handled as in mynn_b200_kv_cache_update. */
int mynn_b200_quantizing_kv_cache_update(void *stream, int8_t *cache, void *scale, const void *new_kv, int BH,
                                         int cache_seq_len, int new_seq_len, int D, int offset,
                                         const int32_t *offset_dev, int dtype);

/* Attention over an int8 KV cache: as mynn_b200_attention, with k/v int8 [B, Hkv, cache_seq_len, D] and per-token
 * scales k_scale/v_scale [B, Hkv, cache_seq_len] in `dtype`; qk = (q . k_int) * k_scale * scale and the softmax weight
 * of a row is multiplied by its v_scale before it meets v_int (src/codegen/cpu/translator.rs:4440-5008; CUDA:
 * the QUANT template paths of cpp/attention.cuh:318-606).  The workspace rules are those of mynn_b200_attention. */
int mynn_b200_attention_q8(void *stream, void *out, const void *q, const int8_t *k, const int8_t *v, const void *k_scale,
                           const void *v_scale, float scale, int B, int Hq, int Hkv, int Sq, int D, int cache_seq_len,
                           int active_seq_kv, const int32_t *active_seq_kv_dev, int is_causal, int dtype, void *workspace,
                           size_t workspace_bytes);

/* DynamicQuantizeLinear (the engine's W8A8 path, src/graph/operator.rs:265-285): x [slices, inner] in `dtype` ->
 * y (int8 when symmetric, uint8 otherwise), y_scale (`dtype`) and y_zero_point (type of y); per_row = 1 gives one scale
 * per slice, per_row = 0 one scale for the whole tensor (outputs of 1 element).
 * Replaces: dynamic_quantize_linear_kernel (cpp/dynamic_quantize_linear.cuh:41-151) and, for the symmetric per-row form,
 * the CPU kernel mynn_dynquant_i8 (src/codegen/cpu/kernels/dynquant_i8.rs:13-37) whose rounding it reproduces. */
int mynn_b200_dynamic_quantize_linear(void *stream, void *y, void *y_scale, void *y_zero_point, const void *x,
                                      long long slices, long long inner, int symmetric, int per_row, int dtype);

/* QuantizedMatMul: out[m,n] = (sum_k lhs[m,k] * rhs[n,k] in int32) * lhs_scale[m or 0] * rhs_scale[n]; lhs int8 [M,K],
 * rhs int8 [N,K], scales and out in `dtype` (src/graph/operator.rs:243-263).
 * Replaces: quantized_gemv_int8 / quantized_matmul_int8 (cpp/quantized_gemv_int8.cuh, cpp/quantized_matmul_int8.cuh) and
 * mynn_qgemv_i8i8 (src/codegen/cpu/kernels/qgemv_i8i8.rs:38-80).
 * With a workspace (mynn_b200_quantized_matmul_workspace_bytes, 256-byte aligned, zeroed once; holds a status word that
 * mynn_b200_dequant_matmul_check reads), K % 16 == 0 and 16-byte aligned operands the product runs on the tcgen05 int8
 * tensor-core kernel; otherwise (workspace NULL included) on a plain kernel. */
size_t mynn_b200_quantized_matmul_workspace_bytes(int M, int N, int K);
int mynn_b200_quantized_matmul(void *stream, void *out, const int8_t *lhs, const void *lhs_scale, int lhs_scale_per_row,
                               const int8_t *rhs, const void *rhs_scale, int M, int N, int K, int dtype, void *workspace,
                               size_t workspace_bytes);

/* KVCacheUpdate with the ring operands of the streaming cache: cache[bh, phys(offset + t), :] = new[bh, t, :] with
 * phys(r) = r for r < ring_sink (or ring_window == 0), else ring_sink + (ring_start + r - ring_sink) % ring_window.
 * Replaces: kvcache_update with ring arguments (cpp/kvcache_update.cuh:6-26, ring_phys_index cpp/common.cuh:55-60). */
int mynn_b200_kv_cache_update_ring(void *stream, void *cache, const void *new_kv, int BH, int cache_seq_len, int new_seq_len,
                                   int D, int offset, int ring_sink, int ring_window, int ring_start, int dtype);

/* The engine's `rope_fused` over a cache: out[bh, s, :] = RoPE(cache[bh, s, :]) at table row kv_position[s] for the
 * slots s < active_seq_kv (the rest of `out` is left alone).  kv_position: device int64 [cache_seq_len].
 * Replaces: rope_fused applied to the K cache in streaming mode (crates/llm/src/decoder.rs:327-336, cpp/rope.cuh). */
int mynn_b200_rope_cache_rows(void *stream, void *out, const void *cache, const void *cos_table, const void *sin_table,
                              const int64_t *kv_position, int BH, int cache_seq_len, int D, int active_seq_kv, int dtype);

/* Attention whose K/V rows are addressed through the ring: logical row r of the 0..active_seq_kv-1 visited rows is read
 * from slot phys(r) (cpp/attention.cuh:546-600, the ring_sink/ring_window/ring_start operands of the Attention node).
 * Workspace as for mynn_b200_attention. */
int mynn_b200_attention_ring(void *stream, void *out, const void *q, const void *k, const void *v, float scale, int B,
                             int Hq, int Hkv, int Sq, int D, int cache_seq_len, int active_seq_kv, int is_causal,
                             int ring_sink, int ring_window, int ring_start, int dtype, void *workspace,
                             size_t workspace_bytes);

/* Attention with every streaming operand of the engine's Attention node (src/graph/operator.rs:1024-1042; builder
 * `attention_streaming`, crates/llm/src/builder.rs:526-568): k/v in `dtype` (kv_int8 = 0, scales NULL) or int8 with per-row
 * scales [B, Hkv, cache_seq_len] (kv_int8 = 1); the ring mapping of mynn_b200_attention_ring; and, when kv_position != NULL,
 * the in-kernel key rotation of the `(streaming, quant_kv_cache)` graph branch (crates/llm/src/decoder.rs:314-326): the key
 * of logical row r is multiplied by its scale and rotated in f32 at row kv_position[r] of the cos / sin tables
 * ([positions, D], `dtype`), as the engine's kernels do it (cpp/attention.cuh:546-600 for one query row, :319-489 for
 * several) -- kv_position (device int64) is indexed by the LOGICAL row.  Any Sq; with is_causal the bound of query row sq is
 * active_seq_kv - Sq + sq + 1 logical rows.  Row-serial arithmetic as in the engine (4 warps per query row). */
int mynn_b200_attention_streaming(void *stream, void *out, const void *q, const void *k, const void *v, const void *k_scale,
                                  const void *v_scale, float scale, int B, int Hq, int Hkv, int Sq, int D, int cache_seq_len,
                                  int active_seq_kv, const int32_t *active_seq_kv_dev, int is_causal, int ring_sink,
                                  int ring_window, int ring_start, const void *cos_table, const void *sin_table,
                                  const int64_t *kv_position, int dtype, int kv_int8);

/* RMSNorm over the last axis: y = x * rsqrt(mean(x^2) + eps) * w.  Replaces rms_norm (cpp/rms_norm.cuh:9-59). */
int mynn_b200_rms_norm(void *stream, void *out, const void *x, const void *weight, float eps, int rows, int D,
                       int dtype);
/* out = round(a + b); y = RMSNorm(out).  Two store points of the engine's schedule in one launch. */
int mynn_b200_add_rms_norm(void *stream, void *sum_out, void *norm_out, const void *a, const void *b,
                           const void *weight, float eps, int rows, int D, int dtype);

/* Half-split RoPE with per-token position gather.  x, out [outer, seq_len, D]; cos/sin tables [max_pos, D];
 * position int64 [seq_len] on the device.  Replaces rope (cpp/rope.cuh:19-46). */
int mynn_b200_rope(void *stream, void *out, const void *x, const void *cos_table, const void *sin_table,
                   const int64_t *position, int outer, int seq_len, int D, int dtype);

/* out = (gate / (1 + exp(-gate))) * up, f32 math.  Replaces the generated Swish*Mul elementwise group
 * (src/codegen/cuda/kernel.rs:763). */
int mynn_b200_swish_mul(void *stream, void *out, const void *gate, const void *up, int64_t n, int dtype);
/* out = a + b (residual add, a standalone kernel in the engine's schedule). */
int mynn_b200_add(void *stream, void *out, const void *a, const void *b, int64_t n, int dtype);

/* Gather(DequantizeLinear(table int8 [V,H], scale [V]), ids): out[i,:] = round(table[ids[i],:] * scale[ids[i]]).
 * Replaces dequantize_linear + gather_axis0_kernel (cpp/dequantize.cuh, cpp/gather.cuh), which dequantise the
 * whole table every step (crates/llm/src/decoder.rs:828-835); only the gathered rows are touched here. */
int mynn_b200_embed_gather_dequant(void *stream, void *out, const int8_t *table, const void *scale,
                                   const int64_t *ids, int n_ids, int H, int V, int dtype);

/* Greedy pick per row with the engine's tie rule (last index among equal maxima,
 * crates/llm/src/session.rs:683-690).  logits [rows, V]; out_idx int32 [rows] on the device. */
int mynn_b200_argmax_last(void *stream, int32_t *out_idx, const void *logits, int rows, int V, int dtype);

/* ---------------------------------------------------------------------------------------------
 * Tensor-parallel communicator.  Replaces trait Communicator {rank, world_size, all_reduce, barrier}
 * (crates/comm/src/lib.rs:32-38), the process-global slot of src/collective.rs:1-20 and the CPU helper
 * mynn_all_reduce(dst, src, num_elements, dtype) (src/codegen/cpu/kernels/all_reduce.rs:14-33).
 * One process per GPU.  unique_id is the 128-byte NCCL id created on rank 0 by mynn_b200_comm_unique_id and
 * distributed by the host (torch.distributed, a file, a socket ...). */
int mynn_b200_comm_unique_id(void *id_out_128_bytes);
int mynn_b200_comm_init(const void *unique_id_128_bytes, int rank, int world_size);
int mynn_b200_comm_rank(void);
int mynn_b200_comm_world_size(void);
int mynn_b200_all_reduce(void *stream, void *dst, const void *src, int64_t num_elements, int dtype);
int mynn_b200_comm_barrier(void *stream);
int mynn_b200_comm_destroy(void);

/* ---------------------------------------------------------------------------------------------
 * Whole decode step.  Replaces the generated library's entry points resolved by SessionCUDA
 * (src/session/cuda.rs:53-56,323-335; generated in src/codegen/cuda.rs:2727-2745):
 *     void *model_init(void **initializer, void **session_state);
 *     void  model(void *state, void **output, void **input);
 *     void  model_destroy(void *state);
 * The generated library is specialised per model at code-generation time; this one is specialised by a
 * configuration call made once before model_init.  Ownership is the engine's: the host owns weights
 * (initializer[i], device pointers) and KV buffers (session_state[i], device, zeroed by the host); the library
 * owns activations, streams and graphs.  input[i] / output[i] are HOST pointers in storage dtype.
 *
 * initializer order (a tensor-parallel rank passes its shard of each: rows of q/k/v/gate/up/lm_head, columns of o/down):
 *   0 embed int8 [V,H], 1 embed scale [V], then per layer l (base 2+16*l):
 *   +0 input_layernorm [H], +1..+2 q (wq, scale), +3..+4 k, +5..+6 v, +7..+8 o, +9 post_attention_layernorm,
 *   +10..+11 gate, +12..+13 up, +14..+15 down; then final norm [H], lm_head wq, lm_head scale, cos table, sin table
 *   ([max_seq_len, head_dim]).
 * session_state order: per layer K cache then V cache, each [batch, n_kv_heads/tp, max_seq_len, head_dim].
 * input: 0 input_ids int64 [batch,1]; 1 position_id int64 [1]; 2 past_len int64 []; 3 active_seq_kv int64 []
 *        (crates/llm/src/session.rs:508-537).
 * output: 0 logits [batch,1,vocab] storage dtype (output_mode 0) or int32 next-token ids [batch] (output_mode 1,
 *         on-device last-max argmax). */
typedef struct mynn_b200_model_config {
    int32_t n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, max_seq_len, batch;
    int32_t dtype;       /* MYNN_BF16 or MYNN_F16 */
    int32_t output_mode; /* 0 logits, 1 token ids */
    int32_t tp_rank, tp_world;
    int32_t use_graph;   /* capture the step in a CUDA graph and replay it */
    int32_t max_prefill; /* largest T accepted by mynn_b200_model_prefill (0 = decode only) */
    int32_t use_tensor_gemm; /* 1: DequantMatMul on the tcgen05 int8 kernel (needs scratch); 0: mma.sync streaming kernel */
    int32_t stream_sink;     /* streaming (sink + ring) KV cache, the engine's `streaming_kv` option: the first stream_sink */
    int32_t stream_window;   /* tokens stay, the last stream_window tokens live in a ring; 0 = off.  Steps then go through
                                mynn_b200_model_stream; sink + window <= max_seq_len.  With kv_int8 the keys are cached unrotated
                                as int8 and rotated inside the attention kernel (mynn_b200_attention_streaming) */
    int32_t kv_int8;         /* 1: the engine's `quant_kv_cache` option: int8 K/V caches with one scale per cached token;
                                session_state then holds FOUR buffers per layer: K int8, V int8, K scale, V scale */
    float rms_eps;
} mynn_b200_model_config;

int mynn_b200_model_configure(const mynn_b200_model_config *cfg);
void *model_init(void **initializer, void **session_state);
void model(void *state, void **output, void **input);
void model_destroy(void *state);
/* Status of the last model_init / model call (they return void to keep the engine's signatures). */
int mynn_b200_model_status(void);

/* One step of a model configured with stream_window > 0: appends the T tokens ids_host [batch, T] that sit at absolute
 * positions stream_pos .. stream_pos + T - 1 of the stream (T == 1: a decode step; T > 1: a prefill chunk, which must not
 * evict, i.e. stream_pos + T <= sink + window, and T <= max_prefill) and returns the last position's logits / token ids
 * in out_host as model() does.  The index math of the engine's streaming session (crates/llm/src/session.rs:539-635:
 * write slot, query position, active rows, ring start, per-slot key positions) is done inside. */
int mynn_b200_model_stream(void *state, const int64_t *ids_host, int T, long long stream_pos, void *out_host);
/* Device-resident variant of model(): ids and outputs stay on the device, no host synchronisation.
 * ids_dev int64 [batch]; past_len is advanced by the caller.  out_dev as output[0] of model(). */
int mynn_b200_model_step_device(void *state, void *stream, const int64_t *ids_dev, int past_len, void *out_dev);
/* Prefill of T tokens per sequence starting at cache row past_len: the engine's prefill graph
 * (crates/llm/src/session.rs:426-480) without its padding rows.  ids_host int64 [batch, T] (host memory); out_host
 * receives what model() would return for the last position.  T <= max_prefill. */
int mynn_b200_model_prefill(void *state, const int64_t *ids_host, int T, int past_len, void *out_host);
/* Fused tensor-parallel reduction over NVLink peer memory (tp_world > 1): each rank exports a 64-byte handle of its
 * shared block; the host gathers the handles in rank order (as it distributes the communicator id) and attaches them
 * before the first step.  The per-layer all-reduce of a decode step (at most 32 rows) then runs as the two fused
 * operators declared below (mynn_b200_tp_*).  Without attach, and for prefill chunks, the step calls ncclAllReduce
 * instead.  No counterpart in the engine, whose AllReduce operator has no CUDA lowering (src/codegen/cuda.rs:2577-2580). */
int mynn_b200_model_tp_export(void *state, void *handle_out_64_bytes);
int mynn_b200_model_tp_attach(void *state, const void *handles_world_x_64_bytes);

/* ---------------------------------------------------------------------------------------------
 * Fused tensor-parallel operators: the all-reduce behind a row-parallel DequantMatMul (o_proj, down_proj), merged with the
 * operators around it.  They replace the sequence DequantMatMul -> AllReduce(sum, f32, rank order:
 * crates/comm/src/uds.rs:106-116) -> Add -> RMSNorm of the engine's tensor-parallel graphs (crates/llm/src/decoder.rs:40-73)
 * and leave the activations of the DequantMatMul that follows ready in its workspace.
 *
 * A group is `world` blocks of device memory, one per rank, each of mynn_b200_tp_block_bytes() bytes, 256-byte aligned,
 * initialised once by its owner with mynn_b200_tp_block_init (before any rank's first push) and mapped into every rank's
 * process (cudaIpc*, or plain pointers when the ranks share a process); blocks[r] is rank r's block as THIS process
 * addresses it.
 *   push     row-parallel DequantMatMul of this rank's K shard: partial[m, :] = scale[:] * (act[m, :K] . wq[:, :K]^T) in f32,
 *            N = hidden, stored from the GEMM epilogue straight into EVERY rank's block (4-byte peer stores; a slot without a
 *            value holds a reserved NaN pattern, so the value itself says that it has arrived and no flag, fence or
 *            collective follows), buffer 0 or 1 in turn.
 *   reduce   on every rank: sum of the `world` partial rows in rank order (it waits, with a time limit, for values that have
 *            not arrived yet, and marks the slots empty again); x[m] = round(x[m] + round(sum)); y = round(RMSNorm(x[m]) *
 *            weight), left as the activation of the next DequantMatMul in `workspace` (call mynn_b200_dequant_matmul_same_act
 *            next; weight NULL: only x is updated).  x [M, hidden] in `dtype`; every rank computes the identical rows.
 * Both calls are made in this order, with the same M and buffer, on every rank; buffers alternate (0, 1, 0, ...); each rank
 * uses one stream.  The wait is bounded (MYNN_OPT_WAIT_BUDGET_US); mynn_b200_tp_check synchronises the stream and returns
 * MYNN_E_COMM, once, if it ran out.  After a rank that delivered nothing the ranks are in step again at the next reduction;
 * if a rank may have delivered late, re-initialise the blocks with all ranks idle before going on.  All ranks of a group may also live on
 * ONE GPU as long as their calls are issued in lock step (every push before any reduce): then no kernel ever waits for one
 * that has not finished.  workspace: as for mynn_b200_dequant_matmul (push: mynn_b200_dequant_matmul_workspace_bytes(M,
 * hidden, K); reduce: the workspace of the product that follows, mynn_b200_dequant_matmul_workspace_bytes(M, N, hidden)). */
typedef struct mynn_b200_tp_group {
    void *blocks[8];
    int32_t rank, world;
    int32_t max_rows; /* largest M of any call on this group (<= 32); fixes the block layout */
    int32_t hidden;
} mynn_b200_tp_group;
size_t mynn_b200_tp_block_bytes(int max_rows, int hidden, int world);
int mynn_b200_tp_block_init(void *stream, void *block, int max_rows, int hidden, int world);
int mynn_b200_tp_dequant_matmul_push(void *stream, const mynn_b200_tp_group *group, int buffer, const void *act,
                                     const int8_t *wq, const float *scale, int M, int K, int act_dtype, void *workspace,
                                     size_t workspace_bytes);
int mynn_b200_tp_reduce_norm(void *stream, const mynn_b200_tp_group *group, int buffer, void *x, const void *weight, float eps,
                             int M, int dtype, void *workspace, size_t workspace_bytes);
int mynn_b200_tp_check(void *stream, const mynn_b200_tp_group *group);

/* How many CTAs the 16-bit decode attention kernel lets share the kv rows of one (batch, kv head) pair, given an upper bound
 * of the rows and the number of CTAs of that kernel an SM holds (2 for the ring form at head_dim 128, else 4).  Pure host
 * arithmetic, exported so that an integrator can see what mynn_b200_attention_workspace_bytes is sized for. */
int mynn_b200_attention_decode_splits(int B, int Hkv, int rows_bound, int ctas_per_sm);

/* Kernels launched by this library since load (monotonic). */
int64_t mynn_b200_launch_count(void);

/* Pinned host allocations, as the engine's common.cu exports (src/codegen/cuda/cpp/common.cu:4-13). */
void *alloc_pinned(size_t bytes);
void free_pinned(void *p);

#ifdef __cplusplus
}
#endif
#endif /* MYNN_B200_H_ */
