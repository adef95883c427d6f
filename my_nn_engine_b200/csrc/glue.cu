// Small operators between the two heavy kernels of a decoder layer: RMSNorm (optionally fused with the
// preceding residual add), RoPE, Swish*Mul, residual add, KV-cache append, embedding gather+dequant and the
// greedy argmax.  All math is f32 with one rounding to the storage dtype per output, matching the store
// points of the engine's schedule (one store per kernel, f32 inside a kernel).
#include <algorithm>

#include "common.cuh"
#include "ops_internal.cuh"

namespace mynn {

// ---- RMSNorm -------------------------------------------------------------------------------------------
// One CTA per row.  With ADD: s = round(a + b) is written to sum_out and normalised.
// VEC: 16-bit tensors read and written 8 elements at a time (D a multiple of 8, 16-byte aligned rows).
template <typename T, bool ADD, bool VEC>
__global__ void __launch_bounds__(256)
rms_norm_kernel(T *sum_out, T *norm_out, const T *a, const T *b, const T *w, float eps, int D) {
    extern __shared__ __align__(16) float row[];
    __shared__ float warp_part[8];
    __shared__ float inv_s;
    const size_t base = (size_t)blockIdx.x * D;
    float ss = 0.f;
    if constexpr (VEC) {
        for (int i = 8 * threadIdx.x; i < D; i += 8 * blockDim.x) {
            T av[8], bv[8], sv[8];
            *reinterpret_cast<uint4 *>(av) = *reinterpret_cast<const uint4 *>(a + base + i);
            if constexpr (ADD) *reinterpret_cast<uint4 *>(bv) = *reinterpret_cast<const uint4 *>(b + base + i);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                float v = to_f32<T>(av[j]);
                if constexpr (ADD) {
                    sv[j] = from_f32<T>(v + to_f32<T>(bv[j]));
                    v = to_f32<T>(sv[j]);
                }
                row[i + j] = v;
                ss += v * v;
            }
            if constexpr (ADD) *reinterpret_cast<uint4 *>(sum_out + base + i) = *reinterpret_cast<const uint4 *>(sv);
        }
    } else {
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            float v = to_f32<T>(a[base + i]);
            if constexpr (ADD) {
                v = round_store<T>(v + to_f32<T>(b[base + i]));
                sum_out[base + i] = from_f32<T>(v);
            }
            row[i] = v;
            ss += v * v;
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int i = 0; i < (int)(blockDim.x >> 5); i++) tot += warp_part[i];
        inv_s = 1.0f / sqrtf(tot / (float)D + eps);
    }
    __syncthreads();
    const float inv = inv_s;
    if constexpr (VEC) {
        for (int i = 8 * threadIdx.x; i < D; i += 8 * blockDim.x) {
            T wv[8], ov[8];
            *reinterpret_cast<uint4 *>(wv) = *reinterpret_cast<const uint4 *>(w + i);
#pragma unroll
            for (int j = 0; j < 8; j++) ov[j] = from_f32<T>(row[i + j] * inv * to_f32<T>(wv[j]));
            *reinterpret_cast<uint4 *>(norm_out + base + i) = *reinterpret_cast<const uint4 *>(ov);
        }
    } else {
        for (int i = threadIdx.x; i < D; i += blockDim.x)
            norm_out[base + i] = from_f32<T>(row[i] * inv * to_f32<T>(w[i]));
    }
}

template <typename T, bool ADD>
static int launch_rms_norm(cudaStream_t st, T *sum_out, T *norm_out, const T *a, const T *b, const T *w, float eps, int rows, int D) {
    const bool vec = sizeof(T) == 2 && D % 8 == 0 &&
                     (((uintptr_t)sum_out | (uintptr_t)norm_out | (uintptr_t)a | (uintptr_t)b | (uintptr_t)w) % 16) == 0;
    auto kern = vec ? rms_norm_kernel<T, ADD, sizeof(T) == 2> : rms_norm_kernel<T, ADD, false>;
    if ((size_t)D * 4 > 48 * 1024) MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, D * 4));
    kern<<<rows, 256, (size_t)D * 4, st>>>(sum_out, norm_out, a, b, w, eps, D);
    return MYNN_OK;
}

// ---- RoPE ------------------------------------------------------------------------------------------------
// x [outer, S, D]; out = x*cos[pos] + concat(-x_high, x_low)*sin[pos]; one thread per (row, j < D/2).
template <typename T>
__global__ void rope_kernel(T *out, const T *x, const T *cos_t, const T *sin_t, const int64_t *position, int rows,
                            int S, int D) {
    const int half = D >> 1;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)rows * half) return;
    const int row = (int)(idx / half), j = (int)(idx - (long long)row * half);
    const long long pos = position[row % S];
    const size_t ro = (size_t)row * D, to = (size_t)pos * D;
    const float xl = to_f32<T>(x[ro + j]), xh = to_f32<T>(x[ro + j + half]);
    out[ro + j] = from_f32<T>(rope_low(xl, xh, to_f32<T>(cos_t[to + j]), to_f32<T>(sin_t[to + j])));
    out[ro + j + half] = from_f32<T>(rope_high(xl, xh, to_f32<T>(cos_t[to + j + half]), to_f32<T>(sin_t[to + j + half])));
}

// ---- elementwise --------------------------------------------------------------------------------------
template <typename T>
__global__ void swish_mul_kernel(T *out, const T *gate, const T *up, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = to_f32<T>(gate[i]);
    out[i] = from_f32<T>((g / (1.0f + expf(-g))) * to_f32<T>(up[i]));
}

// 8 elements per thread with 128-bit accesses (16-bit tensors, 16-byte aligned, n a multiple of 8); out may alias a or b
template <typename T>
__global__ void __launch_bounds__(256) add_vec_kernel(T *out, const T *a, const T *b, long long n8) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    T av[8], bv[8], ov[8];
    *reinterpret_cast<uint4 *>(av) = reinterpret_cast<const uint4 *>(a)[i];
    *reinterpret_cast<uint4 *>(bv) = reinterpret_cast<const uint4 *>(b)[i];
#pragma unroll
    for (int j = 0; j < 8; j++) ov[j] = from_f32<T>(to_f32<T>(av[j]) + to_f32<T>(bv[j]));
    reinterpret_cast<uint4 *>(out)[i] = *reinterpret_cast<const uint4 *>(ov);
}

template <typename T>
__global__ void add_kernel(T *out, const T *a, const T *b, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    out[i] = from_f32<T>(to_f32<T>(a[i]) + to_f32<T>(b[i]));
}

// ---- KV append ------------------------------------------------------------------------------------------
// cache [BH, cache_seq, D], new [BH, new_seq, D]; 16-bit or 32-bit elements copied as raw words.
template <typename W>
__global__ void kv_update_kernel(W *cache, const W *newkv, int cache_seq, int new_seq, int D, int offset_host,
                                 const int32_t *offset_dev) {
    const int offset = offset_dev ? *offset_dev : offset_host;
    const int bh = blockIdx.y;
    const long long n = (long long)new_seq * D;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / D), d = (int)(i - (long long)t * D);
        const int row = offset + t;
        if (row < 0 || row >= cache_seq) continue;  // never write outside the cache
        cache[((size_t)bh * cache_seq + row) * D + d] = newkv[((size_t)bh * new_seq + t) * D + d];
    }
}

// ---- embedding ------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(T *out, const int8_t *table, const T *scale, const int64_t *ids, int H, int V) {
    const long long id = ids[blockIdx.x];
    if (id < 0 || id >= V) {  // out-of-vocabulary id: emit zeros instead of reading out of bounds
        for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)blockIdx.x * H + i] = from_f32<T>(0.f);
        return;
    }
    const float s = to_f32<T>(scale[id]);
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        out[(size_t)blockIdx.x * H + i] = from_f32<T>((float)table[(size_t)id * H + i] * s);
}

// ---- argmax, last maximum wins ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(1024) argmax_last_kernel(int32_t *out_idx, const T *logits, int V) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const T *row = logits + (size_t)blockIdx.x * V;
    float best = -INFINITY;
    int besti = -1;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = to_f32<T>(row[i]);
        if (v >= best || besti < 0) {  // ascending i per thread, so >= keeps the last maximum
            best = v;
            besti = i;
        }
    }
    auto better = [](float v, int i, float bv_, int bi_) { return bi_ < 0 || (i >= 0 && (v > bv_ || (v == bv_ && i > bi_))); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
        if (better(ov, oi, best, besti)) {
            best = ov;
            besti = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        bv[threadIdx.x >> 5] = best;
        bi[threadIdx.x >> 5] = besti;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = blockDim.x >> 5;
        best = threadIdx.x < nw ? bv[threadIdx.x] : -INFINITY;
        besti = threadIdx.x < nw ? bi[threadIdx.x] : -1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
            if (better(ov, oi, best, besti)) {
                best = ov;
                besti = oi;
            }
        }
        if (threadIdx.x == 0) out_idx[blockIdx.x] = besti;
    }
}


// ---- fused RoPE + KV append ------------------------------------------------------------------------------
// grid (token row b*S+s, head slot): slots [0,Hq) rotate q, [Hq,Hq+Hkv) rotate k into the cache, the rest copy v into
// the cache.  One thread per (low, high) element pair.
template <typename T>
__global__ void rope_kv_append_kernel(T *q_out, T *k_cache, T *v_cache, const T *q, const T *k, const T *v,
                                      long long q_stride, long long k_stride, long long v_stride, const T *cos_t,
                                      const T *sin_t, const int64_t *positions, int S, int Hq, int Hkv, int D,
                                      int cache_seq, const int32_t *past_len_dev, int rotate_k) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x, b = row / S, s = row - b * S;
    const int slot = blockIdx.y;
    const int half = D >> 1;
    const int cache_row = *past_len_dev + s;
    const bool in_cache = cache_row >= 0 && cache_row < cache_seq;
    if (slot >= Hq && slot < Hq + Hkv && !rotate_k) {  // streaming cache: keys are stored as the projection left them
        if (!in_cache) return;
        const int h = slot - Hq;
        const T *src = k + (size_t)row * k_stride + (size_t)h * D;
        T *dst = k_cache + (((size_t)b * Hkv + h) * cache_seq + cache_row) * D;
        for (int j = threadIdx.x; j < D; j += blockDim.x) dst[j] = src[j];
    } else if (slot < Hq + Hkv) {
        const long long pos = positions[s];
        const T *cr = cos_t + (size_t)pos * D, *sr = sin_t + (size_t)pos * D;
        const bool is_q = slot < Hq;
        const int h = is_q ? slot : slot - Hq;
        if (!is_q && !in_cache) return;
        const T *src = is_q ? q + (size_t)row * q_stride + (size_t)h * D : k + (size_t)row * k_stride + (size_t)h * D;
        T *dst = is_q ? q_out + (((size_t)b * Hq + h) * S + s) * D : k_cache + (((size_t)b * Hkv + h) * cache_seq + cache_row) * D;
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            const float xl = to_f32<T>(src[j]), xh = to_f32<T>(src[j + half]);
            dst[j] = from_f32<T>(rope_low(xl, xh, to_f32<T>(cr[j]), to_f32<T>(sr[j])));
            dst[j + half] = from_f32<T>(rope_high(xl, xh, to_f32<T>(cr[j + half]), to_f32<T>(sr[j + half])));
        }
    } else {
        if (!in_cache) return;
        const int h = slot - Hq - Hkv;
        const T *src = v + (size_t)row * v_stride + (size_t)h * D;
        T *dst = v_cache + (((size_t)b * Hkv + h) * cache_seq + cache_row) * D;
        for (int j = threadIdx.x; j < D; j += blockDim.x) dst[j] = src[j];
    }
}

// The same with 128-bit accesses for 16-bit tensors (D a multiple of 16, everything 16-byte aligned): one thread per
// (token row, head slot, group of 8 (low, high) pairs); a v slot copies 16 elements per thread.
template <typename T>
__global__ void __launch_bounds__(256)
rope_kv_append_vec_kernel(T *q_out, T *k_cache, T *v_cache, const T *q, const T *k, const T *v, long long q_stride,
                          long long k_stride, long long v_stride, const T *cos_t, const T *sin_t, const int64_t *positions,
                          long long units, int S, int Hq, int Hkv, int D, int cache_seq, const int32_t *past_len_dev, int rotate_k) {
    pdl_trigger();
    pdl_wait();
    const long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= units) return;
    const int half = D >> 1, groups = half >> 3, slots = Hq + 2 * Hkv;
    const int g = (int)(u % groups), slot = (int)((u / groups) % slots);
    const int row = (int)(u / ((long long)groups * slots)), b = row / S, s = row - b * S;
    const int j0 = 8 * g;
    const int cache_row = *past_len_dev + s;
    const bool in_cache = cache_row >= 0 && cache_row < cache_seq;
    const bool is_q = slot < Hq, is_k = !is_q && slot < Hq + Hkv;
    if (!is_q && !in_cache) return;
    const int h = is_q ? slot : (is_k ? slot - Hq : slot - Hq - Hkv);
    const T *src = is_q ? q + (size_t)row * q_stride + (size_t)h * D
                        : (is_k ? k + (size_t)row * k_stride + (size_t)h * D : v + (size_t)row * v_stride + (size_t)h * D);
    T *dst = is_q ? q_out + (((size_t)b * Hq + h) * S + s) * D
                  : (is_k ? k_cache : v_cache) + (((size_t)b * Hkv + h) * cache_seq + cache_row) * D;
    const uint4 lo = *reinterpret_cast<const uint4 *>(src + j0), hi = *reinterpret_cast<const uint4 *>(src + j0 + half);
    if (!is_q && !(is_k && rotate_k)) {  // v, or a key of the streaming cache (stored as the projection left it)
        *reinterpret_cast<uint4 *>(dst + j0) = lo;
        *reinterpret_cast<uint4 *>(dst + j0 + half) = hi;
        return;
    }
    const size_t to = (size_t)positions[s] * D;
    T xl[8], xh[8], cl[8], ch[8], sl[8], sh[8], ol[8], oh[8];
    *reinterpret_cast<uint4 *>(xl) = lo;
    *reinterpret_cast<uint4 *>(xh) = hi;
    *reinterpret_cast<uint4 *>(cl) = *reinterpret_cast<const uint4 *>(cos_t + to + j0);
    *reinterpret_cast<uint4 *>(ch) = *reinterpret_cast<const uint4 *>(cos_t + to + j0 + half);
    *reinterpret_cast<uint4 *>(sl) = *reinterpret_cast<const uint4 *>(sin_t + to + j0);
    *reinterpret_cast<uint4 *>(sh) = *reinterpret_cast<const uint4 *>(sin_t + to + j0 + half);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float a = to_f32<T>(xl[i]), c = to_f32<T>(xh[i]);
        ol[i] = from_f32<T>(rope_low(a, c, to_f32<T>(cl[i]), to_f32<T>(sl[i])));
        oh[i] = from_f32<T>(rope_high(a, c, to_f32<T>(ch[i]), to_f32<T>(sh[i])));
    }
    *reinterpret_cast<uint4 *>(dst + j0) = *reinterpret_cast<const uint4 *>(ol);
    *reinterpret_cast<uint4 *>(dst + j0 + half) = *reinterpret_cast<const uint4 *>(oh);
}

int launch_rope_kv_append(cudaStream_t st, int dtype, void *q_out, void *k_cache, void *v_cache, const void *q,
                          const void *k, const void *v, long long q_stride, long long k_stride, long long v_stride,
                          const void *cos_t, const void *sin_t, const int64_t *positions, int B, int S, int Hq,
                          int Hkv, int D, int cache_seq, const int32_t *past_len_dev, int rotate_k) {
    if (B * S == 0) return MYNN_OK;
    const bool vec = dtype != MYNN_F32 && D % 16 == 0 && q_stride % 8 == 0 && k_stride % 8 == 0 && v_stride % 8 == 0 &&
                     (((uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)q | (uintptr_t)k | (uintptr_t)v |
                       (uintptr_t)cos_t | (uintptr_t)sin_t) % 16) == 0;
    if (vec) {
        const long long units = (long long)B * S * (Hq + 2 * Hkv) * (D / 16);
        const unsigned blocks = (unsigned)((units + 255) / 256);
        if (dtype == MYNN_BF16) {
            using T = __nv_bfloat16;
            MYNN_CUDA_OK(launch_pdl(rope_kv_append_vec_kernel<T>, dim3(blocks), dim3(256), 0, st, (T *)q_out, (T *)k_cache, (T *)v_cache,
                                    (const T *)q, (const T *)k, (const T *)v, q_stride, k_stride, v_stride, (const T *)cos_t,
                                    (const T *)sin_t, positions, units, S, Hq, Hkv, D, cache_seq, past_len_dev, rotate_k));
        } else {
            using T = __half;
            MYNN_CUDA_OK(launch_pdl(rope_kv_append_vec_kernel<T>, dim3(blocks), dim3(256), 0, st, (T *)q_out, (T *)k_cache, (T *)v_cache,
                                    (const T *)q, (const T *)k, (const T *)v, q_stride, k_stride, v_stride, (const T *)cos_t,
                                    (const T *)sin_t, positions, units, S, Hq, Hkv, D, cache_seq, past_len_dev, rotate_k));
        }
        MYNN_LAUNCH_OK("rope_kv_append_vec_kernel");
        return MYNN_OK;
    }
    const int threads = D / 2 >= 64 ? 64 : 32;
    MYNN_DISPATCH_DTYPE(dtype, T, {
        MYNN_CUDA_OK(launch_pdl(rope_kv_append_kernel<T>, dim3(B * S, Hq + 2 * Hkv), dim3(threads), 0, st, (T *)q_out, (T *)k_cache,
                                (T *)v_cache, (const T *)q, (const T *)k, (const T *)v, q_stride, k_stride, v_stride,
                                (const T *)cos_t, (const T *)sin_t, positions, S, Hq, Hkv, D, cache_seq, past_len_dev, rotate_k));
    });
    MYNN_LAUNCH_OK("rope_kv_append_kernel");
    return MYNN_OK;
}

template <typename T>
__global__ void swiglu_strided_kernel(T *out, const T *gate, const T *up, int F, long long in_stride) {
    const int m = blockIdx.y;
    const int f = blockIdx.x * blockDim.x + threadIdx.x;
    if (f >= F) return;
    const float g = to_f32<T>(gate[(size_t)m * in_stride + f]);
    out[(size_t)m * F + f] = from_f32<T>((g / (1.0f + expf(-g))) * to_f32<T>(up[(size_t)m * in_stride + f]));
}

// 8 elements per thread with 128-bit accesses (16-bit tensors, F and the row stride multiples of 8, 16-byte aligned)
template <typename T>
__global__ void __launch_bounds__(256) swiglu_strided_vec_kernel(T *out, const T *gate, const T *up, int F, long long in_stride) {
    const int m = blockIdx.y;
    const int f = 8 * (blockIdx.x * blockDim.x + threadIdx.x);
    if (f >= F) return;
    T g[8], u[8], o[8];
    *reinterpret_cast<uint4 *>(g) = *reinterpret_cast<const uint4 *>(gate + (size_t)m * in_stride + f);
    *reinterpret_cast<uint4 *>(u) = *reinterpret_cast<const uint4 *>(up + (size_t)m * in_stride + f);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float x = to_f32<T>(g[i]);
        o[i] = from_f32<T>((x / (1.0f + expf(-x))) * to_f32<T>(u[i]));
    }
    *reinterpret_cast<uint4 *>(out + (size_t)m * F + f) = *reinterpret_cast<const uint4 *>(o);
}

int launch_swiglu_strided(cudaStream_t st, int dtype, void *out, const void *gate, const void *up, int M, int F,
                          long long in_stride) {
    if (M * F == 0) return MYNN_OK;
    if (dtype != MYNN_F32 && F % 8 == 0 && in_stride % 8 == 0 && (((uintptr_t)out | (uintptr_t)gate | (uintptr_t)up) % 16) == 0 && M <= 65535) {
        const dim3 grid((F / 8 + 255) / 256, M);
        if (dtype == MYNN_BF16)
            swiglu_strided_vec_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((__nv_bfloat16 *)out, (const __nv_bfloat16 *)gate, (const __nv_bfloat16 *)up, F, in_stride);
        else
            swiglu_strided_vec_kernel<__half><<<grid, 256, 0, st>>>((__half *)out, (const __half *)gate, (const __half *)up, F, in_stride);
        MYNN_LAUNCH_OK("swiglu_strided_vec_kernel");
        return MYNN_OK;
    }
    MYNN_DISPATCH_DTYPE(dtype, T, {
        swiglu_strided_kernel<T><<<dim3((F + 255) / 256, M), 256, 0, st>>>((T *)out, (const T *)gate, (const T *)up, F, in_stride);
    });
    MYNN_LAUNCH_OK("swiglu_strided_kernel");
    return MYNN_OK;
}

// sum = round(a + round(b)), b in f32 (an all-reduced partial product); optional RMSNorm of the sum.
template <typename T>
__global__ void __launch_bounds__(256)
add_f32_rms_norm_kernel(T *sum_out, T *norm_out, const T *a, const float *b, const T *w, float eps, int D) {
    extern __shared__ float row[];
    __shared__ float warp_part[8];
    __shared__ float inv_s;
    const size_t base = (size_t)blockIdx.x * D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float v = round_store<T>(to_f32<T>(a[base + i]) + round_store<T>(b[base + i]));
        sum_out[base + i] = from_f32<T>(v);
        row[i] = v;
        ss += v * v;
    }
    if (norm_out == nullptr) return;
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int i = 0; i < (int)(blockDim.x >> 5); i++) tot += warp_part[i];
        inv_s = 1.0f / sqrtf(tot / (float)D + eps);
    }
    __syncthreads();
    const float inv = inv_s;
    for (int i = threadIdx.x; i < D; i += blockDim.x)
        norm_out[base + i] = from_f32<T>(row[i] * inv * to_f32<T>(w[i]));
}

int launch_add_f32_rms_norm(cudaStream_t st, int dtype, void *sum_out, void *norm_out, const void *a, const float *b,
                            const void *weight, float eps, int rows, int D) {
    if (rows == 0) return MYNN_OK;
    if ((size_t)D * 4 > 48 * 1024) return fail(MYNN_E_UNSUPPORTED, "add_f32_rms_norm: D=%d too large", D);
    MYNN_DISPATCH_DTYPE(dtype, T, {
        add_f32_rms_norm_kernel<T><<<rows, 256, (size_t)D * 4, st>>>((T *)sum_out, (T *)norm_out, (const T *)a, b, (const T *)weight, eps, D);
    });
    MYNN_LAUNCH_OK("add_f32_rms_norm_kernel");
    return MYNN_OK;
}

// (max, last index of max) per row of a logits shard; index_offset makes the index global.
template <typename T>
__global__ void __launch_bounds__(1024) argmax_pairs_kernel(float *pairs, const T *logits, int V, int index_offset) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const T *row = logits + (size_t)blockIdx.x * V;
    float best = -INFINITY;
    int besti = -1;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = to_f32<T>(row[i]);
        if (v >= best || besti < 0) {
            best = v;
            besti = i;
        }
    }
    auto better = [](float v, int i, float bv_, int bi_) { return bi_ < 0 || (i >= 0 && (v > bv_ || (v == bv_ && i > bi_))); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
        if (better(ov, oi, best, besti)) { best = ov; besti = oi; }
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = besti; }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = blockDim.x >> 5;
        best = threadIdx.x < nw ? bv[threadIdx.x] : -INFINITY;
        besti = threadIdx.x < nw ? bi[threadIdx.x] : -1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
            if (better(ov, oi, best, besti)) { best = ov; besti = oi; }
        }
        if (threadIdx.x == 0) {
            pairs[2 * blockIdx.x] = best;
            pairs[2 * blockIdx.x + 1] = __int_as_float(besti + index_offset);
        }
    }
}

__global__ void argmax_merge_kernel(int32_t *out_idx, const float *pairs, int rows, int world) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    float best = -INFINITY;
    int besti = -1;
    for (int w = 0; w < world; w++) {  // shards hold ascending index ranges: >= keeps the last maximum
        const float v = pairs[((size_t)w * rows + r) * 2];
        const int i = __float_as_int(pairs[((size_t)w * rows + r) * 2 + 1]);
        if (besti < 0 || v >= best) { best = v; besti = i; }
    }
    out_idx[r] = besti;
}

int launch_argmax_pairs(cudaStream_t st, int dtype, float *pairs, const void *logits, int rows, int V, int index_offset) {
    if (rows == 0) return MYNN_OK;
    MYNN_DISPATCH_DTYPE(dtype, T, {
        argmax_pairs_kernel<T><<<rows, 1024, 0, st>>>(pairs, (const T *)logits, V, index_offset);
    });
    MYNN_LAUNCH_OK("argmax_pairs_kernel");
    return MYNN_OK;
}

// Two-stage greedy pick for long rows: `chunks` CTAs per row each find (max, last index) of a slice, then the slices
// are merged in ascending order (>= keeps the last maximum).  pairs: scratch of chunks * rows * 2 floats.
template <typename T>
__global__ void __launch_bounds__(1024) argmax_chunk_kernel(float *pairs, const T *logits, int rows, int V, int chunks) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const int r = blockIdx.x / chunks, c = blockIdx.x - r * chunks;
    const int per = (V + chunks - 1) / chunks;
    const int beg = c * per, end = min(V, beg + per);
    const T *row = logits + (size_t)r * V;
    float best = -INFINITY;
    int besti = -1;
    for (int i = beg + threadIdx.x; i < end; i += blockDim.x) {
        const float v = to_f32<T>(row[i]);
        if (v >= best || besti < 0) {
            best = v;
            besti = i;
        }
    }
    auto better = [](float v, int i, float bv_, int bi_) { return bi_ < 0 || (i >= 0 && (v > bv_ || (v == bv_ && i > bi_))); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
        if (better(ov, oi, best, besti)) { best = ov; besti = oi; }
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = besti; }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = blockDim.x >> 5;
        best = threadIdx.x < nw ? bv[threadIdx.x] : -INFINITY;
        besti = threadIdx.x < nw ? bi[threadIdx.x] : -1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
            if (better(ov, oi, best, besti)) { best = ov; besti = oi; }
        }
        if (threadIdx.x == 0) {
            pairs[((size_t)c * rows + r) * 2] = best;
            pairs[((size_t)c * rows + r) * 2 + 1] = __int_as_float(besti);
        }
    }
}

int launch_argmax_two_stage(cudaStream_t st, int dtype, int32_t *out_idx, float *pairs, const void *logits, int rows, int V,
                            int chunks) {
    if (rows == 0) return MYNN_OK;
    MYNN_DISPATCH_DTYPE(dtype, T, {
        argmax_chunk_kernel<T><<<rows * chunks, 512, 0, st>>>(pairs, (const T *)logits, rows, V, chunks);
    });
    MYNN_LAUNCH_OK("argmax_chunk_kernel");
    return launch_argmax_merge(st, out_idx, pairs, rows, chunks);
}

int launch_argmax_merge(cudaStream_t st, int32_t *out_idx, const float *pairs, int rows, int world) {
    if (rows == 0) return MYNN_OK;
    argmax_merge_kernel<<<(rows + 127) / 128, 128, 0, st>>>(out_idx, pairs, rows, world);
    MYNN_LAUNCH_OK("argmax_merge_kernel");
    return MYNN_OK;
}

__global__ void tok_feedback_kernel(int64_t *ids, const int32_t *tok, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) ids[i] = tok[i];
}

int launch_tok_feedback(cudaStream_t st, int64_t *ids, const int32_t *tok, int n) {
    if (n == 0) return MYNN_OK;
    tok_feedback_kernel<<<(n + 127) / 128, 128, 0, st>>>(ids, tok, n);
    MYNN_LAUNCH_OK("tok_feedback_kernel");
    return MYNN_OK;
}

}  // namespace mynn

using namespace mynn;

extern "C" int mynn_b200_rms_norm(void *stream, void *out, const void *x, const void *weight, float eps, int rows,
                                  int D, int dtype) {
    if (rows < 0 || D <= 0) return fail(MYNN_E_ARG, "rms_norm: bad shape rows=%d D=%d", rows, D);
    if (rows == 0) return MYNN_OK;
    if (!out || !x || !weight) return fail(MYNN_E_ARG, "rms_norm: null pointer");
    if ((size_t)D * 4 > 200 * 1024) return fail(MYNN_E_UNSUPPORTED, "rms_norm: D=%d exceeds the shared-memory row buffer", D);
    MYNN_DISPATCH_DTYPE(dtype, T, {
        if (int rc = launch_rms_norm<T, false>((cudaStream_t)stream, nullptr, (T *)out, (const T *)x, nullptr, (const T *)weight, eps, rows, D)) return rc;
    });
    MYNN_LAUNCH_OK("rms_norm_kernel");
    return MYNN_OK;
}

extern "C" int mynn_b200_add_rms_norm(void *stream, void *sum_out, void *norm_out, const void *a, const void *b,
                                      const void *weight, float eps, int rows, int D, int dtype) {
    if (rows < 0 || D <= 0) return fail(MYNN_E_ARG, "add_rms_norm: bad shape rows=%d D=%d", rows, D);
    if (rows == 0) return MYNN_OK;
    if (!sum_out || !norm_out || !a || !b || !weight) return fail(MYNN_E_ARG, "add_rms_norm: null pointer");
    if ((size_t)D * 4 > 200 * 1024) return fail(MYNN_E_UNSUPPORTED, "add_rms_norm: D=%d too large", D);
    MYNN_DISPATCH_DTYPE(dtype, T, {
        if (int rc = launch_rms_norm<T, true>((cudaStream_t)stream, (T *)sum_out, (T *)norm_out, (const T *)a, (const T *)b, (const T *)weight, eps, rows, D)) return rc;
    });
    MYNN_LAUNCH_OK("add_rms_norm_kernel");
    return MYNN_OK;
}

extern "C" int mynn_b200_rope(void *stream, void *out, const void *x, const void *cos_table, const void *sin_table,
                              const int64_t *position, int outer, int seq_len, int D, int dtype) {
    if (outer < 0 || seq_len < 0 || D <= 0 || (D & 1)) return fail(MYNN_E_ARG, "rope: bad shape outer=%d S=%d D=%d", outer, seq_len, D);
    const long long rows = (long long)outer * seq_len;
    if (rows == 0) return MYNN_OK;
    if (!out || !x || !cos_table || !sin_table || !position) return fail(MYNN_E_ARG, "rope: null pointer");
    const long long n = rows * (D / 2);
    MYNN_DISPATCH_DTYPE(dtype, T, {
        rope_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>((T *)out, (const T *)x, (const T *)cos_table, (const T *)sin_table, position, (int)rows, seq_len, D);
    });
    MYNN_LAUNCH_OK("rope_kernel");
    return MYNN_OK;
}

extern "C" int mynn_b200_swish_mul(void *stream, void *out, const void *gate, const void *up, int64_t n, int dtype) {
    if (n < 0) return fail(MYNN_E_ARG, "swish_mul: negative size");
    if (n == 0) return MYNN_OK;
    if (!out || !gate || !up) return fail(MYNN_E_ARG, "swish_mul: null pointer");
    MYNN_DISPATCH_DTYPE(dtype, T, {
        swish_mul_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>((T *)out, (const T *)gate, (const T *)up, n);
    });
    MYNN_LAUNCH_OK("swish_mul_kernel");
    return MYNN_OK;
}

extern "C" int mynn_b200_add(void *stream, void *out, const void *a, const void *b, int64_t n, int dtype) {
    if (n < 0) return fail(MYNN_E_ARG, "add: negative size");
    if (n == 0) return MYNN_OK;
    if (!out || !a || !b) return fail(MYNN_E_ARG, "add: null pointer");
    if (dtype != MYNN_F32 && n % 8 == 0 && (((uintptr_t)out | (uintptr_t)a | (uintptr_t)b) % 16) == 0) {
        const long long n8 = n / 8;
        const unsigned blocks = (unsigned)((n8 + 255) / 256);
        if (dtype == MYNN_BF16)
            add_vec_kernel<__nv_bfloat16><<<blocks, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16 *)out, (const __nv_bfloat16 *)a, (const __nv_bfloat16 *)b, n8);
        else
            add_vec_kernel<__half><<<blocks, 256, 0, (cudaStream_t)stream>>>((__half *)out, (const __half *)a, (const __half *)b, n8);
        MYNN_LAUNCH_OK("add_vec_kernel");
        return MYNN_OK;
    }
    MYNN_DISPATCH_DTYPE(dtype, T, {
        add_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>((T *)out, (const T *)a, (const T *)b, n);
    });
    MYNN_LAUNCH_OK("add_kernel");
    return MYNN_OK;
}

extern "C" int mynn_b200_kv_cache_update(void *stream, void *cache, const void *new_kv, int BH, int cache_seq_len,
                                         int new_seq_len, int D, int offset, const int32_t *offset_dev, int dtype) {
    if (BH < 0 || cache_seq_len < 0 || new_seq_len < 0 || D <= 0) return fail(MYNN_E_ARG, "kv_cache_update: bad shape");
    if (!dtype_ok(dtype)) return fail(MYNN_E_ARG, "kv_cache_update: bad dtype %d", dtype);
    if (BH == 0 || new_seq_len == 0) return MYNN_OK;
    if (!cache || !new_kv) return fail(MYNN_E_ARG, "kv_cache_update: null pointer");
    if (!offset_dev && (offset < 0 || offset + new_seq_len > cache_seq_len))
        return fail(MYNN_E_ARG, "kv_cache_update: rows [%d, %d) fall outside the cache of %d rows", offset, offset + new_seq_len, cache_seq_len);
    const long long n = (long long)new_seq_len * D;
    dim3 grid((unsigned)std::min<long long>((n + 255) / 256, 1024), BH);
    if (dtype == MYNN_F32)
        kv_update_kernel<uint32_t><<<grid, 256, 0, (cudaStream_t)stream>>>((uint32_t *)cache, (const uint32_t *)new_kv, cache_seq_len, new_seq_len, D, offset, offset_dev);
    else
        kv_update_kernel<uint16_t><<<grid, 256, 0, (cudaStream_t)stream>>>((uint16_t *)cache, (const uint16_t *)new_kv, cache_seq_len, new_seq_len, D, offset, offset_dev);
    MYNN_LAUNCH_OK("kv_update_kernel");
    return MYNN_OK;
}

extern "C" int mynn_b200_embed_gather_dequant(void *stream, void *out, const int8_t *table, const void *scale,
                                              const int64_t *ids, int n_ids, int H, int V, int dtype) {
    if (n_ids < 0 || H <= 0 || V <= 0) return fail(MYNN_E_ARG, "embed_gather_dequant: bad shape");
    if (n_ids == 0) return MYNN_OK;
    if (!out || !table || !scale || !ids) return fail(MYNN_E_ARG, "embed_gather_dequant: null pointer");
    MYNN_DISPATCH_DTYPE(dtype, T, {
        embed_kernel<T><<<n_ids, 256, 0, (cudaStream_t)stream>>>((T *)out, table, (const T *)scale, ids, H, V);
    });
    MYNN_LAUNCH_OK("embed_kernel");
    return MYNN_OK;
}

extern "C" int mynn_b200_argmax_last(void *stream, int32_t *out_idx, const void *logits, int rows, int V, int dtype) {
    if (rows < 0 || V <= 0) return fail(MYNN_E_ARG, "argmax_last: bad shape rows=%d V=%d", rows, V);
    if (rows == 0) return MYNN_OK;
    if (!out_idx || !logits) return fail(MYNN_E_ARG, "argmax_last: null pointer");
    MYNN_DISPATCH_DTYPE(dtype, T, {
        argmax_last_kernel<T><<<rows, 1024, 0, (cudaStream_t)stream>>>(out_idx, (const T *)logits, V);
    });
    MYNN_LAUNCH_OK("argmax_last_kernel");
    return MYNN_OK;
}
