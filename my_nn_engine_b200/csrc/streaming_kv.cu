// Streaming (sink + ring) KV cache: the long-context mode of the engine (`streaming_kv` build option).
//
// Layout: the first `sink` tokens keep their slots; later tokens live in a ring of `window` slots.  Keys are cached
// UNROTATED: the RoPE position of a cached key is its recency rank, which changes every time a token is evicted, so the
// keys are rotated when they are read (crates/llm/src/decoder.rs:280-360: `rope_fused` over the cache with the per-slot
// table `kv_position`, then attention with the ring operands).
//
// This file holds the two pieces that differ from the plain cache: the append through `ring_phys_index`
// (src/codegen/cuda/cpp/common.cuh:55-60, kvcache_update.cuh:6-26) and the rotation of the live cache rows into a
// scratch copy that the attention kernels then read (the ring walk itself is in attention.cu).
#include <type_traits>

#include "common.cuh"
#include "ops_internal.cuh"

namespace mynn {

__device__ __forceinline__ int ring_phys_index(int rank, int ring_sink, int ring_window, int ring_start) {
    if (ring_window == 0 || rank < ring_sink) return rank;
    return ring_sink + (ring_start + (rank - ring_sink)) % ring_window;
}

// grid (ceil(new_seq * D / 256), BH); U = storage word of one element
template <typename U>
__global__ void kv_update_ring_kernel(U *cache, const U *new_kv, int cache_seq, int new_seq, int D, int offset, int ring_sink,
                                      int ring_window, int ring_start) {
    const int bh = blockIdx.y;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)new_seq * D; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / D), d = (int)(i - (long long)t * D);
        const int phys = ring_phys_index(offset + t, ring_sink, ring_window, ring_start);
        if (phys >= 0 && phys < cache_seq) cache[((size_t)bh * cache_seq + phys) * D + d] = new_kv[((size_t)bh * new_seq + t) * D + d];
    }
}

// out[bh, s, :] = RoPE(x[bh, s, :]) at position kv_position[s] for the live slots s < active; 8 (low, high) pairs per
// thread with 128-bit accesses.  grid (ceil(active_bound * D / 16 / 256), BH).
template <typename T>
__global__ void rope_cache_rows_kernel(T *out, const T *x, const T *cos_t, const T *sin_t, const int64_t *kv_position,
                                       int cache_seq, int D, int active_host, const int32_t *active_dev) {
    pdl_trigger();
    pdl_wait();
    const int active = min(active_dev ? *active_dev : active_host, cache_seq);
    const int half = D >> 1, groups = half >> 3;  // groups of 8 pairs per row
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)active * groups) return;
    const int s = (int)(idx / groups), j0 = 8 * (int)(idx - (long long)s * groups);
    const size_t ro = ((size_t)blockIdx.y * cache_seq + s) * D, to = (size_t)kv_position[s] * D;
    T xl[8], xh[8], cl[8], ch[8], sl[8], sh[8], ol[8], oh[8];
    *reinterpret_cast<uint4 *>(xl) = *reinterpret_cast<const uint4 *>(x + ro + j0);
    *reinterpret_cast<uint4 *>(xh) = *reinterpret_cast<const uint4 *>(x + ro + j0 + half);
    *reinterpret_cast<uint4 *>(cl) = *reinterpret_cast<const uint4 *>(cos_t + to + j0);
    *reinterpret_cast<uint4 *>(ch) = *reinterpret_cast<const uint4 *>(cos_t + to + j0 + half);
    *reinterpret_cast<uint4 *>(sl) = *reinterpret_cast<const uint4 *>(sin_t + to + j0);
    *reinterpret_cast<uint4 *>(sh) = *reinterpret_cast<const uint4 *>(sin_t + to + j0 + half);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float a = to_f32<T>(xl[i]), b = to_f32<T>(xh[i]);
        ol[i] = from_f32<T>(a * to_f32<T>(cl[i]) - b * to_f32<T>(sl[i]));
        oh[i] = from_f32<T>(b * to_f32<T>(ch[i]) + a * to_f32<T>(sh[i]));
    }
    *reinterpret_cast<uint4 *>(out + ro + j0) = *reinterpret_cast<const uint4 *>(ol);
    *reinterpret_cast<uint4 *>(out + ro + j0 + half) = *reinterpret_cast<const uint4 *>(oh);
}

// generic form (any even D, f32): one thread per pair
template <typename T>
__global__ void rope_cache_rows_plain_kernel(T *out, const T *x, const T *cos_t, const T *sin_t, const int64_t *kv_position,
                                             int cache_seq, int D, int active_host, const int32_t *active_dev) {
    const int active = min(active_dev ? *active_dev : active_host, cache_seq);
    const int half = D >> 1;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)active * half) return;
    const int s = (int)(idx / half), j = (int)(idx - (long long)s * half);
    const size_t ro = ((size_t)blockIdx.y * cache_seq + s) * D, to = (size_t)kv_position[s] * D;
    const float a = to_f32<T>(x[ro + j]), b = to_f32<T>(x[ro + j + half]);
    out[ro + j] = from_f32<T>(rope_low(a, b, to_f32<T>(cos_t[to + j]), to_f32<T>(sin_t[to + j])));
    out[ro + j + half] = from_f32<T>(rope_high(a, b, to_f32<T>(cos_t[to + j + half]), to_f32<T>(sin_t[to + j + half])));
}

int launch_rope_cache_rows(cudaStream_t st, int dtype, void *out, const void *x, const void *cos_t, const void *sin_t,
                           const int64_t *kv_position, int BH, int cache_seq, int D, int active_host, const int32_t *active_dev) {
    if (BH == 0 || cache_seq == 0) return MYNN_OK;
    const int bound = active_dev ? cache_seq : (active_host < cache_seq ? active_host : cache_seq);
    if (bound <= 0) return MYNN_OK;
    const bool vec = dtype != MYNN_F32 && D % 16 == 0 && ((((uintptr_t)out | (uintptr_t)x | (uintptr_t)cos_t | (uintptr_t)sin_t) % 16) == 0);
    MYNN_DISPATCH_DTYPE(dtype, T, {
        if (vec) {
            const long long n = (long long)bound * (D / 16);
            MYNN_CUDA_OK(launch_pdl(rope_cache_rows_kernel<T>, dim3((unsigned)((n + 255) / 256), BH), dim3(256), 0, st, (T *)out, (const T *)x,
                                    (const T *)cos_t, (const T *)sin_t, kv_position, cache_seq, D, active_host, active_dev));
        } else {
            const long long n = (long long)bound * (D / 2);
            rope_cache_rows_plain_kernel<T><<<dim3((unsigned)((n + 255) / 256), BH), 256, 0, st>>>((T *)out, (const T *)x, (const T *)cos_t,
                                                                                                (const T *)sin_t, kv_position, cache_seq, D,
                                                                                                active_host, active_dev);
        }
    });
    MYNN_LAUNCH_OK("rope_cache_rows_kernel");
    return MYNN_OK;
}

// Attention with ALL the streaming operands of the engine's Attention node (src/graph/operator.rs:1024-1042): an int8 or
// 16/32-bit cache, per-row k/v scales, the ring mapping, and the cos / sin / kv_position operands that make the kernel rotate
// every key on the fly: the `(streaming, quant_kv_cache)` branch of the decoder graph (crates/llm/src/decoder.rs:314-326).
// The arithmetic follows the engine's kernels row by row (src/codegen/cuda/cpp/attention.cuh:495-606 and :319-489): the key of
// logical row r is read from slot ring_phys_index(r), multiplied by its k_scale, rotated in f32 at table row kv_position[r]
// (indexed by the LOGICAL row, as the engine's kernel does; never rounded), dotted with q; the softmax weight is multiplied by
// v_scale before it meets v.  One CTA of 4 warps per query row (b, h, sq): the warps take kv rows in turn, each with its own
// running maximum and sum, and are merged through shared memory.  D <= 32 * MAXE.
constexpr int kStreamWarps = 4;

template <typename T, typename TKV, int MAXE>
__global__ void __launch_bounds__(kStreamWarps * 32)
attention_streaming_kernel(T *out, const T *q, const TKV *k, const TKV *v, const T *k_scale, const T *v_scale, float scale, int Hq,
                           int Hkv, int Sq, int D, int cache_seq, int active_host, const int32_t *active_dev, int is_causal,
                           int ring_sink, int ring_window, int ring_start, const T *cos_t, const T *sin_t,
                           const long long *kv_position, int out_bshd) {
    __shared__ float sm_o[kStreamWarps][32 * MAXE];
    __shared__ float sm_m[kStreamWarps], sm_s[kStreamWarps];
    pdl_trigger();
    pdl_wait();
    const long long row = blockIdx.x;  // (b * Hq + h) * Sq + sq
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sq = (int)(row % Sq);
    const long long bh = row / Sq;
    const int h = (int)(bh % Hq), b = (int)(bh / Hq);
    const int kvh = h / (Hq / Hkv), half = D >> 1;
    const int active = min(active_dev ? *active_dev : active_host, cache_seq);
    int bound = active;
    if (is_causal) bound = min(bound, active - Sq + sq + 1);
    const T *qp = q + (size_t)row * D;
    const size_t kv_base = (size_t)(b * Hkv + kvh) * cache_seq;
    constexpr bool QUANT = !std::is_same<T, TKV>::value;
    float qr[MAXE], o[MAXE];
#pragma unroll
    for (int e = 0; e < MAXE; e++) {
        const int d = lane + 32 * e;
        qr[e] = d < D ? to_f32<T>(qp[d]) : 0.f;
        o[e] = 0.f;
    }
    float m = -INFINITY, ssum = 0.f;
    for (int lr = warp; lr < bound; lr += kStreamWarps) {
        const int phys = ring_phys_index(lr, ring_sink, ring_window, ring_start);
        const TKV *kp = k + (kv_base + phys) * D, *vp = v + (kv_base + phys) * D;
        const float ks = QUANT ? to_f32<T>(k_scale[kv_base + phys]) : 1.0f;
        const float vs = QUANT ? to_f32<T>(v_scale[kv_base + phys]) : 1.0f;
        const long long pos = kv_position ? kv_position[lr] : 0;
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < MAXE; e++) {
            const int d = lane + 32 * e;
            if (d < D) {
                float kv_ = (float)kp[d] * ks;
                if (kv_position) {
                    const int pair = d < half ? d + half : d - half;
                    const float kpair = (float)kp[pair] * ks;
                    const float c = to_f32<T>(cos_t[(size_t)pos * D + d]), s_ = to_f32<T>(sin_t[(size_t)pos * D + d]);
                    kv_ = kv_ * c + (d < half ? -kpair : kpair) * s_;
                }
                dot += qr[e] * kv_;
            }
        }
        const float qk = warp_sum(dot) * scale;
        const float m_new = fmaxf(m, qk);
        const float coeff = expf(m - m_new);
        float score = expf(qk - m_new);
        ssum = ssum * coeff + score;
        if (QUANT) score *= vs;
#pragma unroll
        for (int e = 0; e < MAXE; e++) {
            const int d = lane + 32 * e;
            if (d < D) o[e] = o[e] * coeff + score * (float)vp[d];
        }
        m = m_new;
    }
#pragma unroll
    for (int e = 0; e < MAXE; e++) sm_o[warp][lane + 32 * e] = o[e];
    if (lane == 0) {
        sm_m[warp] = m;
        sm_s[warp] = ssum;
    }
    __syncthreads();
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < kStreamWarps; w++) mx = fmaxf(mx, sm_m[w]);
    for (int d = threadIdx.x; d < D; d += kStreamWarps * 32) {
        float L = 0.f, O = 0.f;
        for (int w = 0; w < kStreamWarps; w++)
            if (sm_m[w] > -INFINITY) {
                const float f = expf(sm_m[w] - mx);
                L += sm_s[w] * f;
                O += sm_o[w][d] * f;
            }
        const size_t orow = out_bshd ? ((size_t)b * Sq + sq) * Hq + h : (size_t)row;  // [B, Sq, Hq, D] rows for a following o_proj
        out[orow * D + d] = from_f32<T>(O / L);
    }
}

template <typename T, typename TKV>
static int launch_streaming_typed(cudaStream_t st, void *out, const void *q, const void *k, const void *v, const void *k_scale,
                                  const void *v_scale, float scale, int B, int Hq, int Hkv, int Sq, int D, int cache_seq, int active,
                                  const int32_t *active_dev, int causal, int rs, int rw, int r0, const void *cos_t, const void *sin_t,
                                  const int64_t *kv_position, int out_bshd) {
    const unsigned blocks = (unsigned)((long long)B * Hq * Sq);
#define GEN(MAXE)                                                                                                                       \
    MYNN_CUDA_OK(launch_pdl(attention_streaming_kernel<T, TKV, MAXE>, dim3(blocks), dim3(kStreamWarps * 32), 0, st, (T *)out, (const T *)q, \
                            (const TKV *)k, (const TKV *)v, (const T *)k_scale, (const T *)v_scale, scale, Hq, Hkv, Sq, D, cache_seq, active, \
                            active_dev, causal, rs, rw, r0, (const T *)cos_t, (const T *)sin_t, (const long long *)kv_position, out_bshd))
    if (D <= 32) GEN(1);
    else if (D <= 64) GEN(2);
    else if (D <= 128) GEN(4);
    else if (D <= 256) GEN(8);
    else return fail(MYNN_E_UNSUPPORTED, "attention_streaming: head dim %d > 256", D);
#undef GEN
    MYNN_LAUNCH_OK("attention_streaming_kernel");
    return MYNN_OK;
}

int launch_attention_streaming(cudaStream_t st, void *out, const void *q, const void *k, const void *v, const void *k_scale,
                               const void *v_scale, float scale, int B, int Hq, int Hkv, int Sq, int D, int cache_seq, int active,
                               const int32_t *active_dev, int causal, int rs, int rw, int r0, const void *cos_t, const void *sin_t,
                               const int64_t *kv_position, int dtype, int kv_int8, int out_bshd) {
#define GO(T)                                                                                                                          \
    return kv_int8 ? launch_streaming_typed<T, int8_t>(st, out, q, k, v, k_scale, v_scale, scale, B, Hq, Hkv, Sq, D, cache_seq, active, \
                                                       active_dev, causal, rs, rw, r0, cos_t, sin_t, kv_position, out_bshd)            \
                   : launch_streaming_typed<T, T>(st, out, q, k, v, k_scale, v_scale, scale, B, Hq, Hkv, Sq, D, cache_seq, active,      \
                                                  active_dev, causal, rs, rw, r0, cos_t, sin_t, kv_position, out_bshd)
    if (dtype == MYNN_F32) GO(float);
    if (dtype == MYNN_BF16) GO(__nv_bfloat16);
    GO(__half);
#undef GO
}

}  // namespace mynn

using namespace mynn;

extern "C" int mynn_b200_kv_cache_update_ring(void *stream, void *cache, const void *new_kv, int BH, int cache_seq_len,
                                              int new_seq_len, int D, int offset, int ring_sink, int ring_window,
                                              int ring_start, int dtype) {
    if (BH < 0 || cache_seq_len < 0 || new_seq_len < 0 || D <= 0 || offset < 0) return fail(MYNN_E_ARG, "kv_cache_update_ring: bad shape");
    if (!dtype_ok(dtype)) return fail(MYNN_E_ARG, "kv_cache_update_ring: bad dtype %d", dtype);
    if (ring_sink < 0 || ring_window < 0 || ring_start < 0 || (ring_window > 0 && ring_start >= ring_window) ||
        ring_sink + ring_window > cache_seq_len)
        return fail(MYNN_E_ARG, "kv_cache_update_ring: bad ring (sink %d, window %d, start %d, cache %d)", ring_sink, ring_window, ring_start, cache_seq_len);
    if (ring_window == 0 && offset + new_seq_len > cache_seq_len)
        return fail(MYNN_E_ARG, "kv_cache_update_ring: rows [%d, %d) fall outside the cache of %d rows", offset, offset + new_seq_len, cache_seq_len);
    if (BH == 0 || new_seq_len == 0) return MYNN_OK;
    if (!cache || !new_kv) return fail(MYNN_E_ARG, "kv_cache_update_ring: null pointer");
    const long long n = (long long)new_seq_len * D;
    dim3 grid((unsigned)std::min<long long>((n + 255) / 256, 1024), BH);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == MYNN_F32)
        kv_update_ring_kernel<uint32_t><<<grid, 256, 0, st>>>((uint32_t *)cache, (const uint32_t *)new_kv, cache_seq_len, new_seq_len, D, offset, ring_sink, ring_window, ring_start);
    else
        kv_update_ring_kernel<uint16_t><<<grid, 256, 0, st>>>((uint16_t *)cache, (const uint16_t *)new_kv, cache_seq_len, new_seq_len, D, offset, ring_sink, ring_window, ring_start);
    MYNN_LAUNCH_OK("kv_update_ring_kernel");
    return MYNN_OK;
}

extern "C" int mynn_b200_rope_cache_rows(void *stream, void *out, const void *cache, const void *cos_table, const void *sin_table,
                                         const int64_t *kv_position, int BH, int cache_seq_len, int D, int active_seq_kv, int dtype) {
    if (BH < 0 || cache_seq_len < 0 || D <= 0 || (D & 1) || active_seq_kv < 0) return fail(MYNN_E_ARG, "rope_cache_rows: bad shape");
    if (!dtype_ok(dtype)) return fail(MYNN_E_ARG, "rope_cache_rows: bad dtype %d", dtype);
    if (BH == 0 || cache_seq_len == 0 || active_seq_kv == 0) return MYNN_OK;
    if (!out || !cache || !cos_table || !sin_table || !kv_position) return fail(MYNN_E_ARG, "rope_cache_rows: null pointer");
    return launch_rope_cache_rows((cudaStream_t)stream, dtype, out, cache, cos_table, sin_table, kv_position, BH, cache_seq_len, D,
                                  active_seq_kv, nullptr);
}

extern "C" int mynn_b200_attention_streaming(void *stream, void *out, const void *q, const void *k, const void *v, const void *k_scale,
                                             const void *v_scale, float scale, int B, int Hq, int Hkv, int Sq, int D, int cache_seq_len,
                                             int active_seq_kv, const int32_t *active_seq_kv_dev, int is_causal, int ring_sink,
                                             int ring_window, int ring_start, const void *cos_table, const void *sin_table,
                                             const int64_t *kv_position, int dtype, int kv_int8) {
    if (B < 0 || Hq <= 0 || Hkv <= 0 || Sq < 0 || D <= 0 || (D & 1) || cache_seq_len < 0 || active_seq_kv < 0 || Hq % Hkv)
        return fail(MYNN_E_ARG, "attention_streaming: bad shape");
    if (!dtype_ok(dtype)) return fail(MYNN_E_ARG, "attention_streaming: bad dtype %d", dtype);
    if (ring_sink < 0 || ring_window < 0 || ring_start < 0 || (ring_window > 0 && ring_start >= ring_window) ||
        ring_sink + ring_window > cache_seq_len)
        return fail(MYNN_E_ARG, "attention_streaming: bad ring (sink %d, window %d, start %d, cache %d)", ring_sink, ring_window, ring_start, cache_seq_len);
    if (ring_window > 0 && active_seq_kv > ring_sink + ring_window)
        return fail(MYNN_E_ARG, "attention_streaming: %d active rows exceed sink + window = %d", active_seq_kv, ring_sink + ring_window);
    if (B == 0 || Sq == 0) return MYNN_OK;
    if (!out || !q || !k || !v) return fail(MYNN_E_ARG, "attention_streaming: null pointer");
    if (kv_int8 && (!k_scale || !v_scale)) return fail(MYNN_E_ARG, "attention_streaming: an int8 cache needs k_scale and v_scale");
    if (kv_position && (!cos_table || !sin_table)) return fail(MYNN_E_ARG, "attention_streaming: kv_position needs the cos and sin tables");
    return launch_attention_streaming((cudaStream_t)stream, out, q, k, v, k_scale, v_scale, scale, B, Hq, Hkv, Sq, D, cache_seq_len,
                                      active_seq_kv, active_seq_kv_dev, is_causal, ring_sink, ring_window, ring_start, cos_table, sin_table,
                                      kv_position, dtype, kv_int8, 0);
}
