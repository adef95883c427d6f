// Launchers shared between translation units that are not part of the public C ABI: the fused forms the
// decoder step uses on top of the operator-level entry points.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mynn {

// RoPE(q), RoPE(k) and the KV append of one step in a single launch.
// q/k/v: [B*S rows] with row strides (elements) q_stride/k_stride/v_stride, heads contiguous inside a row.
// positions int64 [S] (device) select the cos/sin rows; K and V rows go to cache row (*past_len_dev + s).
// q_out [B, Hq, S, D].  rotate_k = 0 appends K unrotated (streaming cache: keys are rotated when they are read).
int launch_rope_kv_append(cudaStream_t st, int dtype, void *q_out, void *k_cache, void *v_cache, const void *q,
                          const void *k, const void *v, long long q_stride, long long k_stride, long long v_stride,
                          const void *cos_t, const void *sin_t, const int64_t *positions, int B, int S, int Hq,
                          int Hkv, int D, int cache_seq, const int32_t *past_len_dev, int rotate_k = 1);

// out[bh, s, :] = RoPE(x[bh, s, :]) at position kv_position[s] for the slots s < active of a [BH, cache_seq, D] cache.
int launch_rope_cache_rows(cudaStream_t st, int dtype, void *out, const void *x, const void *cos_t, const void *sin_t,
                           const int64_t *kv_position, int BH, int cache_seq, int D, int active_host, const int32_t *active_dev);

// Attention with every streaming operand of the engine's Attention node (ring mapping, int8 cache with per-row scales, keys
// rotated inside the kernel at kv_position[logical row]); see streaming_kv.cu.
int launch_attention_streaming(cudaStream_t st, void *out, const void *q, const void *k, const void *v, const void *k_scale,
                               const void *v_scale, float scale, int B, int Hq, int Hkv, int Sq, int D, int cache_seq, int active,
                               const int32_t *active_dev, int causal, int rs, int rw, int r0, const void *cos_t, const void *sin_t,
                               const int64_t *kv_position, int dtype, int kv_int8, int out_bshd);

// The same step for an int8 KV cache: K (after RoPE and its store rounding) and V are quantized per token into
// k_cache/v_cache int8 [B, Hkv, cache_seq, D] with their scales [B, Hkv, cache_seq] in the storage dtype.
int launch_rope_kv_append_q8(cudaStream_t st, int dtype, void *q_out, void *k_cache, void *v_cache, void *k_scale,
                             void *v_scale, const void *q, const void *k, const void *v, long long q_stride,
                             long long k_stride, long long v_stride, const void *cos_t, const void *sin_t,
                             const int64_t *positions, int B, int S, int Hq, int Hkv, int D, int cache_seq,
                             const int32_t *past_len_dev, int rotate_k = 1);

// Attention over an int8 KV cache (per-token scales), with the output-layout choice of launch_attention.
int launch_attention_q8(cudaStream_t st, void *out, const void *q, const void *k, const void *v, const void *k_scale,
                        const void *v_scale, float scale, int B, int Hq, int Hkv, int Sq, int D, int cache_seq_len,
                        int active_seq_kv, const int32_t *active_seq_kv_dev, int is_causal, int dtype, void *workspace,
                        size_t workspace_bytes, int out_bshd);

// out[m, f] = swish(gate[m, f]) * up[m, f] with gate/up rows `in_stride` elements apart.
int launch_swiglu_strided(cudaStream_t st, int dtype, void *out, const void *gate, const void *up, int M, int F,
                          long long in_stride);

// sum = round(a + round(b_f32)); norm = RMSNorm(sum) (norm_out/weight may be null to skip the norm).
int launch_add_f32_rms_norm(cudaStream_t st, int dtype, void *sum_out, void *norm_out, const void *a, const float *b,
                            const void *weight, float eps, int rows, int D);

// Attention with a choice of output layout: out_bshd != 0 writes [B, Sq, Hq, D] instead of [B, Hq, Sq, D].
// limbs_out / ascale_out (decode fast path only, see attention_decode_fast_path): the output rows are also left as
// activation limbs [3 B][Hq * D] + row scales [B] for the DequantMatMul that follows; needs the workspace.
// fuse (decode fast path only): RoPE and the KV append happen inside the attention kernel.  q is then the UNROTATED projection
// output (row b at q + b * qkv_stride elements), k_new / v_new the new key / value rows with the same row stride; the new row
// is rotated at table row *pos, stored to cache row *row, and attended to as that row (active_seq_kv must be *row + 1).
struct AttentionFuse {
    const void *k_new, *v_new;
    long long qkv_stride;
    const void *cos_t, *sin_t;
    const int64_t *pos;
    const int32_t *row;
};
int launch_attention(cudaStream_t st, void *out, const void *q, const void *k, const void *v, float scale, int B,
                     int Hq, int Hkv, int Sq, int D, int cache_seq_len, int active_seq_kv,
                     const int32_t *active_seq_kv_dev, int is_causal, int dtype, void *workspace,
                     size_t workspace_bytes, int out_bshd, int8_t *limbs_out = nullptr, float *ascale_out = nullptr,
                     const AttentionFuse *fuse = nullptr, int *status_word = nullptr);
// status_word: where the ring form of the decode kernel records a timed-out wait (null: the library's own word)
int attention_decode_take_status(int *status);
int attention_decode_q8_take_status(int *status);
bool attention_decode_fast_path(int Sq, int D, int Hq, int Hkv, int dtype, const void *q, const void *k, const void *v);

// Tiled tensor-core attention for several query rows (prefill chunks); see attention_prefill.cu.
bool attention_prefill_supported(int Sq, int D, int dtype, const void *q, const void *k, const void *v, const void *out);
int launch_attention_prefill(cudaStream_t st, void *out, const void *q, const void *k, const void *v, float scale, int B, int Hq,
                             int Hkv, int Sq, int D, int cache_seq_len, int active_seq_kv, const int32_t *active_seq_kv_dev,
                             int is_causal, int dtype, int out_bshd);
// 16-bit copy of the live rows of an int8 KV cache (value * per-row scale, rounded once); see kv_int8.cu.
int launch_dequant_kv_rows(cudaStream_t st, int dtype, void *out, const void *cache, const void *scale, int BH, int cache_seq, int D,
                           int active_host, const int32_t *active_dev);
// The same on tcgen05 / tensor memory (128 query rows per CTA, TMA-fed); see attention_prefill_tc.cu.
bool attention_prefill_tc_supported(int B, int Hq, int Hkv, int Sq, int D, int cache_seq_len, int dtype, const void *q, const void *k,
                                    const void *v, const void *out);
int launch_attention_prefill_tc(cudaStream_t st, void *out, const void *q, const void *k, const void *v, float scale, int B, int Hq,
                                int Hkv, int Sq, int D, int cache_seq_len, int active_seq_kv, const int32_t *active_seq_kv_dev,
                                int is_causal, int dtype, int out_bshd);

// Reads and clears the status word of the tcgen05 prefill attention kernels (call with the stream idle); non-zero = a bounded
// wait expired in an earlier launch.
int attention_prefill_tc_take_status(int *status);

// Per-row (max value, last index of the maximum) of a logits shard, and the merge over tensor-parallel shards.
int launch_argmax_pairs(cudaStream_t st, int dtype, float *pairs /*[rows][2]*/, const void *logits, int rows, int V,
                        int index_offset);
int launch_argmax_merge(cudaStream_t st, int32_t *out_idx, const float *pairs /*[world][rows][2]*/, int rows, int world);

int launch_argmax_two_stage(cudaStream_t st, int dtype, int32_t *out_idx, float *pairs /*[chunks][rows][2]*/, const void *logits,
                            int rows, int V, int chunks);

// ids[i] = tok[i]: feeds the greedy tokens back as the next step's input ids without leaving the device.
int launch_tok_feedback(cudaStream_t st, int64_t *ids, const int32_t *tok, int n);

}  // namespace mynn
