// INT8 KV cache for sm_100a: the quantizing append and attention over the quantized cache.
//
// The engine's option `quant_kv_cache` stores K and V as int8 [B, H, MAX_SEQ, D] with ONE scale per cached token
// [B, H, MAX_SEQ] (QuantizingKVCacheUpdate, src/codegen/cpu/translator.rs:4090-4372,
// src/codegen/cuda/cpp/quantizing_kvcache_update.cuh) and folds the scales into attention as qk * k_scale and
// e * v_scale (src/codegen/cpu/translator.rs:4440-5008).  The cache bytes, which bound decode attention, halve.
//
// Decode kernel: same structure as the 16-bit kernel (one CTA per (split, kv head, batch), 4 warps taking 16-row tiles,
// O^T = V^T P^T on mma.m16n8k16, online softmax in f32), with these differences:
//   * QK^T runs on the int8 path (mma.m16n8k32.s8): a lane's 16 K bytes are 16 head-dim values and go to the tensor
//     core as they are, against the query row as two signed 8-bit limbs kept in shared memory, with the head-dim
//     index of Q permuted to match;
//   * V bytes of two kv rows are interleaved by a byte permute BEFORE the conversion, so that one conversion yields the
//     (row 2t, row 2t+1) pairs of two head-dim values, i.e. two A-fragment registers;
//   * k_scale multiplies S per kv row after the MMA, v_scale multiplies P per kv row before it, so the tensor cores
//     only ever see exact small integers on the cache side.
#include "attention_internal.cuh"
#include "i8_cvt.cuh"
#include "i8_gemm.cuh"
#include "ops_internal.cuh"
#include "tcgen05.cuh"

namespace mynn {

// ---- quantizing append -----------------------------------------------------------------------------------------------
// s = max|x| * (1/127); inv = 127 / max (0 for an all-zero row); q = trunc(x * inv +- 0.5) clamped to [-128, 127].
// The products are kept as separate roundings (no fused multiply-add) so that the bytes equal the CPU backend's.
__device__ __forceinline__ int8_t quantize_kv_value(float v, float inv) {
    const float sc = __fmul_rn(v, inv);
    const int q = (int)__fadd_rn(sc, sc >= 0.f ? 0.5f : -0.5f);
    return (int8_t)max(-128, min(127, q));
}

// one warp per new row (bh, t)
template <typename T>
__global__ void quant_kv_update_kernel(int8_t *cache, T *scale, const T *new_kv, long long rows, int cache_seq,
                                       int new_seq, int D, int offset_host, const int32_t *offset_dev) {
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= rows) return;
    const int t = (int)(wid % new_seq);
    const long long bh = wid / new_seq;
    const int dst_row = (offset_dev ? *offset_dev : offset_host) + t;
    if (dst_row < 0 || dst_row >= cache_seq) return;
    const T *src = new_kv + (size_t)wid * D;
    float mx = 0.f;
    for (int d = lane; d < D; d += 32) mx = fmaxf(mx, fabsf(to_f32<T>(src[d])));
    mx = warp_max(mx);
    const float inv = mx == 0.f ? 0.f : __fdiv_rn(127.0f, mx);
    int8_t *dst = cache + ((size_t)bh * cache_seq + dst_row) * D;
    for (int d = lane; d < D; d += 32) dst[d] = quantize_kv_value(to_f32<T>(src[d]), inv);
    if (lane == 0) scale[(size_t)bh * cache_seq + dst_row] = from_f32<T>(__fmul_rn(mx, 1.0f / 127.0f));
}

// ---- fused RoPE + quantizing append of one decoder step ------------------------------------------------------------
// grid (token row b*S+s, head slot): slots [0,Hq) rotate q, [Hq,Hq+Hkv) rotate k, round it to the storage dtype (the
// Rope operator's store) and quantize it into the cache, the rest quantize v into the cache.  blockDim = 64.
template <typename T>
__global__ void __launch_bounds__(64)
rope_kv_append_q8_kernel(T *q_out, int8_t *k_cache, int8_t *v_cache, T *k_scale, T *v_scale, const T *q, const T *k,
                         const T *v, long long q_stride, long long k_stride, long long v_stride, const T *cos_t,
                         const T *sin_t, const int64_t *positions, int S, int Hq, int Hkv, int D, int cache_seq,
                         const int32_t *past_len_dev, int slot0, int rotate_k) {
    extern __shared__ float rowv[];  // D rotated / copied values
    __shared__ float wmax[2];
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x, b = row / S, s = row - b * S;
    const int slot = blockIdx.y + slot0;  // slot0 = Hq: the q heads are rotated by another launch
    const int half = D >> 1;
    const int cache_row = *past_len_dev + s;
    const bool in_cache = cache_row >= 0 && cache_row < cache_seq;
    if (slot < Hq) {
        const long long pos = positions[s];
        const T *cr = cos_t + (size_t)pos * D, *sr = sin_t + (size_t)pos * D;
        const T *src = q + (size_t)row * q_stride + (size_t)slot * D;
        T *dst = q_out + (((size_t)b * Hq + slot) * S + s) * D;
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            const float xl = to_f32<T>(src[j]), xh = to_f32<T>(src[j + half]);
            dst[j] = from_f32<T>(rope_low(xl, xh, to_f32<T>(cr[j]), to_f32<T>(sr[j])));
            dst[j + half] = from_f32<T>(rope_high(xl, xh, to_f32<T>(cr[j + half]), to_f32<T>(sr[j + half])));
        }
        return;
    }
    if (!in_cache) return;  // uniform over the block
    const bool is_k = slot < Hq + Hkv;
    const int h = is_k ? slot - Hq : slot - Hq - Hkv;
    float mx = 0.f;
    if (is_k && rotate_k) {
        const long long pos = positions[s];
        const T *cr = cos_t + (size_t)pos * D, *sr = sin_t + (size_t)pos * D;
        const T *src = k + (size_t)row * k_stride + (size_t)h * D;
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            const float xl = to_f32<T>(src[j]), xh = to_f32<T>(src[j + half]);
            const float lo = round_store<T>(rope_low(xl, xh, to_f32<T>(cr[j]), to_f32<T>(sr[j])));
            const float hi = round_store<T>(rope_high(xl, xh, to_f32<T>(cr[j + half]), to_f32<T>(sr[j + half])));
            rowv[j] = lo;
            rowv[j + half] = hi;
            mx = fmaxf(mx, fmaxf(fabsf(lo), fabsf(hi)));
        }
    } else {  // V, or K of a streaming cache (cached as the projection left it, rotated when it is read)
        const T *src = is_k ? k + (size_t)row * k_stride + (size_t)h * D : v + (size_t)row * v_stride + (size_t)h * D;
        for (int j = threadIdx.x; j < D; j += blockDim.x) {
            const float x = to_f32<T>(src[j]);
            rowv[j] = x;
            mx = fmaxf(mx, fabsf(x));
        }
    }
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = fmaxf(wmax[0], wmax[1]);
    const float inv = mx == 0.f ? 0.f : __fdiv_rn(127.0f, mx);
    const size_t crow = ((size_t)b * Hkv + h) * cache_seq + cache_row;
    int8_t *dst = (is_k ? k_cache : v_cache) + crow * D;
    for (int j = threadIdx.x; j < D; j += blockDim.x) dst[j] = quantize_kv_value(rowv[j], inv);
    if (threadIdx.x == 0) (is_k ? k_scale : v_scale)[crow] = from_f32<T>(__fmul_rn(mx, 1.0f / 127.0f));
}

int launch_rope_kv_append_q8(cudaStream_t st, int dtype, void *q_out, void *k_cache, void *v_cache, void *k_scale,
                             void *v_scale, const void *q, const void *k, const void *v, long long q_stride,
                             long long k_stride, long long v_stride, const void *cos_t, const void *sin_t,
                             const int64_t *positions, int B, int S, int Hq, int Hkv, int D, int cache_seq,
                             const int32_t *past_len_dev, int rotate_k) {
    if (B * S == 0) return MYNN_OK;
    if (D > 4096) return fail(MYNN_E_UNSUPPORTED, "rope_kv_append_q8: head dim %d too large", D);
    // prefill chunks: the q heads (most of the slots) go through the 128-bit RoPE kernel, this one keeps the k / v slots
    int slot0 = 0;
    if (S > 1 && dtype != MYNN_F32 && D % 16 == 0) {
        if (int rc = launch_rope_kv_append(st, dtype, q_out, q_out, q_out, q, q, q, q_stride, q_stride, q_stride, cos_t, sin_t, positions,
                                           B, S, Hq, 0, D, cache_seq, past_len_dev, 1))
            return rc;
        slot0 = Hq;
    }
    MYNN_DISPATCH_DTYPE(dtype, T, {
        MYNN_CUDA_OK(launch_pdl(rope_kv_append_q8_kernel<T>, dim3(B * S, Hq + 2 * Hkv - slot0), dim3(64), (size_t)D * 4, st, (T *)q_out,
                                (int8_t *)k_cache, (int8_t *)v_cache, (T *)k_scale, (T *)v_scale, (const T *)q, (const T *)k,
                                (const T *)v, q_stride, k_stride, v_stride, (const T *)cos_t, (const T *)sin_t, positions, S,
                                Hq, Hkv, D, cache_seq, past_len_dev, slot0, rotate_k));
    });
    MYNN_LAUNCH_OK("rope_kv_append_q8_kernel");
    return MYNN_OK;
}

// ---- decode attention over the int8 cache ----------------------------------------------------------------------------
template <int VB>
struct MapQ8 {  // accumulator tile i holds head-dim rows VB*g + 2i (+1): lane group g owns VB consecutive head-dim values
    static __device__ __forceinline__ int d(int i, int g) { return VB * g + 2 * i; }
};

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    // m16n8k32, rows 8..15 of A (padding heads) are zero
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 lds_16(const void *p) {  // volatile: re-read every iteration instead of pinning registers
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"((unsigned)__cvta_generic_to_shared(p)));
    return v;
}
template <typename T>
__device__ __forceinline__ float2 unpack_pair(uint32_t w) {  // two packed 16-bit floats -> f32
    if constexpr (std::is_same<T, __half>::value) {
        return __half22float2(reinterpret_cast<const __half2 &>(w));
    } else {
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    }
}
// scales of rows (row, row + 1), row even, both clamped to `last`
template <typename T>
__device__ __forceinline__ uint32_t load_scale_pair(const T *sc, int row, int last, bool packed) {
    if (packed) return __ldg(reinterpret_cast<const uint32_t *>(sc + min(row, last & ~1)));
    const uint16_t *s16 = reinterpret_cast<const uint16_t *>(sc);
    return (uint32_t)__ldg(s16 + min(row, last)) | ((uint32_t)__ldg(s16 + min(row + 1, last)) << 16);
}

// grid (splits, Hkv, B), block 128.  A warp takes 32 kv rows per iteration (two 16-row sub-tiles u = 0, 1), which keeps
// as many bytes in flight per warp as the 16-bit kernel does with 16 rows.
//
// QK^T runs on the int8 tensor-core path with no conversion of K at all: the query row of each head enters as two
// signed 8-bit limbs of a 15-bit fixed-point value (per-head power-of-two scale, error <= 2^-15 of the row maximum, far
// below the rounding of the 16-bit output), S = (Q0 . K + 256 Q1 . K) / sc exactly in int32.
//
// RING (head_dim 128): as in the 16-bit kernel, every warp owns a ring of kQ8RingDepth tiles in shared memory that the TMA
// engine fills: one 32-row x 128-byte box of K and one of V per tile (2-D maps of the caches, 128-byte swizzle) plus the 32
// row scales of each by an untiled bulk copy; the fragments and scales are then taken from shared memory.  Lane 0 of the
// consuming warp issues the copies of tile j + depth once the warp has tile j in registers.
constexpr int kQ8RingDepth = 3;
__device__ int g_q8_ring_status;  // 32: a wait for a tile ran out of time
MYNN_DEFINE_WAIT_BUDGET_SETTER(kv_int8)

template <typename T, int D, bool RING>
__global__ void __launch_bounds__(kAttnWarps * 32, RING ? 2 : 4)
attention_decode_q8_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const DecodeParams p) {
    constexpr bool F16 = std::is_same<T, __half>::value;
    constexpr int KCH = D / 64;  // 16-byte K chunks per lane per row
    constexpr int VB = D / 8;    // V bytes per lane per row
    constexpr int VW = VB / 4;   // ... as 32-bit words
    constexpr int NACC = VB / 2;
    constexpr int QSTRIDE = D + 64;  // bytes between heads in a limb plane: the 8 lanes of a 128-bit access phase hit distinct banks
    __shared__ __align__(16) int8_t sm_q[2][8][QSTRIDE];
    __shared__ float sm_qinv[8];

    pdl_trigger();
    pdl_wait();
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int G = p.G;
    int active = p.active_dev ? *p.active_dev : p.active_host;
    active = max(0, min(active, p.cache_seq));
    // whole rounds of the CTA's four warps (128 rows): a split that ends inside a round leaves some warps a tile short
    const int rows_per_split = (((active + p.splits - 1) / p.splits) + 32 * kAttnWarps - 1) / (32 * kAttnWarps) * (32 * kAttnWarps);
    const int row_beg = split * rows_per_split;
    const int row_end = min(row_beg + rows_per_split, active);

    const size_t head = (size_t)(b * p.Hkv + kvh) * p.cache_seq;
    const int8_t *kbase = reinterpret_cast<const int8_t *>(p.k) + head * D;
    const int8_t *vbase = reinterpret_cast<const int8_t *>(p.v) + head * D;
    const T *ksc = reinterpret_cast<const T *>(p.k_scale) + head;
    const T *vsc = reinterpret_cast<const T *>(p.v_scale) + head;
    const bool packed_scales = (p.cache_seq & 1) == 0 && ((reinterpret_cast<uintptr_t>(p.k_scale) | reinterpret_cast<uintptr_t>(p.v_scale)) & 3) == 0;

    // ---- query limbs: 16 threads per head, E elements each ----
    {
        constexpr int E = D / 16;
        const int h = threadIdx.x >> 4, part = threadIdx.x & 15;
        float qv[E];
        const T *qrow = reinterpret_cast<const T *>(p.q) + (size_t)(b * p.Hq + kvh * G + min(h, G - 1)) * D + part * E;
        float mx = 0.f;
        bool bad = false;
#pragma unroll
        for (int i = 0; i < E; i++) {
            qv[i] = h < G ? to_f32<T>(qrow[i]) : 0.f;
            bad |= !(fabsf(qv[i]) <= 3.0e38f);
            mx = fmaxf(mx, fabsf(qv[i]));
        }
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) {
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            bad |= __shfl_xor_sync(0xffffffffu, (int)bad, o) != 0;
        }
        int e = 0;
        if (mx > 0.f) frexpf(mx, &e);
        const float sc = (mx > 0.f && !bad) ? ldexpf(1.0f, 14 - e) : 0.f;  // |q| * sc < 2^14
        uint32_t w0[E / 4], w1[E / 4];
#pragma unroll
        for (int i = 0; i < E / 4; i++) w0[i] = w1[i] = 0u;
#pragma unroll
        for (int i = 0; i < E; i++) {
            const int A = sc == 0.f ? 0 : __float2int_rn(qv[i] * sc);
            const int l0 = (int)(int8_t)(A & 0xFF);
            const int l1 = (A - l0) >> 8;
            w0[i >> 2] |= (uint32_t)(l0 & 0xFF) << (8 * (i & 3));
            w1[i >> 2] |= (uint32_t)(l1 & 0xFF) << (8 * (i & 3));
        }
#pragma unroll
        for (int i = 0; i < E / 4; i++) {
            *reinterpret_cast<uint32_t *>(&sm_q[0][h][part * E + 4 * i]) = w0[i];
            *reinterpret_cast<uint32_t *>(&sm_q[1][h][part * E + 4 * i]) = w1[i];
        }
        // a query row with a NaN or an infinity gives NaN scores, hence a NaN output row, as plain arithmetic would
        if (part == 0) sm_qinv[h] = bad ? __int_as_float(0x7fc00000) : (sc > 0.f ? 1.0f / sc : 0.f);
    }
    __syncthreads();
    const float qinv = sm_qinv[g] * p.scale;

    float o[NACC][4];
#pragma unroll
    for (int j = 0; j < NACC; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) o[j][i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    const int last = row_end - 1;

    // ring state (RING only)
    extern __shared__ __align__(1024) uint8_t ring_raw[];
    constexpr uint32_t kBox = 32 * 128, kTile = 2 * kBox;
    __shared__ uint64_t full[RING ? kAttnWarps : 1][kQ8RingDepth];
    __shared__ __align__(16) T sm_sc[RING ? kAttnWarps : 1][kQ8RingDepth][2][32];
    __shared__ int abort_flag;
    uint8_t *ring = ring_raw + (size_t)warp * kQ8RingDepth * kTile;
    const int first = row_beg + 32 * warp;
    const int ntile = first < row_end ? (row_end - first + 32 * kAttnWarps - 1) / (32 * kAttnWarps) : 0;
    auto issue = [&](int j) {  // lane 0: tile j of this warp into stage j % depth
        if constexpr (RING) {
            const int s = j % kQ8RingDepth, base = first + 32 * kAttnWarps * j;
            uint8_t *st = ring + (size_t)s * kTile;
            const uint32_t sc_bytes = (uint32_t)min(32, p.cache_seq - base) * (uint32_t)sizeof(T);  // a multiple of 16
            mbar_expect_tx(&full[warp][s], kTile + 2 * sc_bytes);
            tma_load_2d(st, &map_k, 0, (int)head + base, &full[warp][s]);
            tma_load_2d(st + kBox, &map_v, 0, (int)head + base, &full[warp][s]);
            bulk_load_1d(&sm_sc[warp][s][0][0], ksc + base, sc_bytes, &full[warp][s]);
            bulk_load_1d(&sm_sc[warp][s][1][0], vsc + base, sc_bytes, &full[warp][s]);
        }
    };
    if constexpr (RING) {
        if (threadIdx.x == 0) abort_flag = 0;
        if (lane == 0) {
#pragma unroll
            for (int s = 0; s < kQ8RingDepth; s++) mbar_init(&full[warp][s], 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncthreads();
        if (lane == 0)
            for (int j = 0; j < min(ntile, kQ8RingDepth); j++) issue(j);
    }

    for (int base = first, j = 0; base < row_end; base += 32 * kAttnWarps, j++) {
        uint4 kr[2][2][KCH];
        uint32_t vr[2][4][VW];
        uint32_t ksr[2][2], vsr[2][2];
        if constexpr (RING) {
            const int s = j % kQ8RingDepth;
            int ok_i = 1;
            if (lane == 0) ok_i = mbar_wait_spin(&full[warp][s], (j / kQ8RingDepth) & 1, &abort_flag) ? 1 : 0;
            if (!__shfl_sync(0xffffffffu, ok_i, 0)) {  // the copy never arrived: report it, leave the rows out
                if (lane == 0) {
                    atomicExch(&abort_flag, 1);
                    atomicExch(p.status ? p.status : &g_q8_ring_status, 32);
                }
                break;
            }
            const uint8_t *st = ring + (size_t)s * kTile;
#pragma unroll
            for (int u = 0; u < 2; u++)
#pragma unroll
                for (int nt = 0; nt < 2; nt++) {
                    const int row = 16 * u + 8 * nt + g;  // row % 8 == g
#pragma unroll
                    for (int i = 0; i < KCH; i++) kr[u][nt][i] = *reinterpret_cast<const uint4 *>(st + row * 128 + (((t + 4 * i) ^ g) << 4));
                    ksr[u][nt] = *reinterpret_cast<const uint32_t *>(&sm_sc[warp][s][0][16 * u + 8 * nt + 2 * t]);
                    vsr[u][nt] = *reinterpret_cast<const uint32_t *>(&sm_sc[warp][s][1][16 * u + 8 * nt + 2 * t]);
                }
#pragma unroll
            for (int u = 0; u < 2; u++)
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    const int row = 16 * u + 2 * t + (r & 1) + 8 * (r >> 1);
                    const uint4 w = *reinterpret_cast<const uint4 *>(st + kBox + row * 128 + ((g ^ (row & 7)) << 4));
                    vr[u][r][0] = w.x, vr[u][r][1] = w.y, vr[u][r][2] = w.z, vr[u][r][3] = w.w;
                }
            __syncwarp();  // every lane has its fragments: the stage may be refilled
            if (lane == 0 && j + kQ8RingDepth < ntile) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                issue(j + kQ8RingDepth);
            }
        } else {
        // ---- issue all loads of this tile (rows past the end are clamped to a valid row and masked below) ----
#pragma unroll
        for (int u = 0; u < 2; u++)
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                const int8_t *kp = kbase + (size_t)min(base + 16 * u + 8 * nt + g, last) * D + 16 * t;
#pragma unroll
                for (int i = 0; i < KCH; i++) kr[u][nt][i] = ldg_16(kp + 64 * i);
            }
#pragma unroll
        for (int u = 0; u < 2; u++)
#pragma unroll
            for (int r = 0; r < 4; r++) {
                const int row = base + 16 * u + 2 * t + (r & 1) + 8 * (r >> 1);
                const int8_t *vp = vbase + (size_t)min(row, last) * D + VB * g;
                if constexpr (VW == 4) {
                    const uint4 w = ldg_16(vp);
                    vr[u][r][0] = w.x, vr[u][r][1] = w.y, vr[u][r][2] = w.z, vr[u][r][3] = w.w;
                } else {
                    const uint2 w = ldg_8(vp);
                    vr[u][r][0] = w.x, vr[u][r][1] = w.y;
                }
            }
#pragma unroll
        for (int u = 0; u < 2; u++)
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                ksr[u][nt] = load_scale_pair<T>(ksc, base + 16 * u + 8 * nt + 2 * t, last, packed_scales);
                vsr[u][nt] = load_scale_pair<T>(vsc, base + 16 * u + 8 * nt + 2 * t, last, packed_scales);
            }
        }
        // ---- S = Q K^T in int32: k32 step (i, jj) pairs words (2jj, 2jj+1) of K chunk i with the same words of Q ----
        int s0[2][2][4], s1[2][2][4];
#pragma unroll
        for (int u = 0; u < 2; u++)
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int c = 0; c < 4; c++) s0[u][nt][c] = s1[u][nt][c] = 0;
#pragma unroll
        for (int i = 0; i < KCH; i++) {
            const uint4 q0 = lds_16(&sm_q[0][g][16 * (t + 4 * i)]), q1 = lds_16(&sm_q[1][g][16 * (t + 4 * i)]);
#pragma unroll
            for (int u = 0; u < 2; u++)
#pragma unroll
                for (int nt = 0; nt < 2; nt++) {
                    const uint4 kw = kr[u][nt][i];
                    mma_s8(s0[u][nt], q0.x, q0.y, kw.x, kw.y);
                    mma_s8(s0[u][nt], q0.z, q0.w, kw.z, kw.w);
                    mma_s8(s1[u][nt], q1.x, q1.y, kw.x, kw.y);
                    mma_s8(s1[u][nt], q1.z, q1.w, kw.z, kw.w);
                }
        }
        // ---- online softmax for head g over the 32 rows; qk = (q . k_int) * k_scale * scale ----
        float pv[2][2][2];
        float tmax = -INFINITY;
#pragma unroll
        for (int u = 0; u < 2; u++)
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                const float2 kf = unpack_pair<T>(ksr[u][nt]);
                const float kk[2] = {kf.x, kf.y};
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int row = base + 16 * u + 8 * nt + 2 * t + e;
                    const float dot = (float)(s0[u][nt][e] + (s1[u][nt][e] << 8));
                    pv[u][nt][e] = row < row_end ? dot * kk[e] * qinv : -INFINITY;
                    tmax = fmaxf(tmax, pv[u][nt][e]);
                }
            }
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        const float m_new = fmaxf(m_run, tmax);  // finite unless the scores are NaN: the tile has at least one valid row
        const float alpha = __expf(m_run - m_new);
        float psum = 0.f;
#pragma unroll
        for (int u = 0; u < 2; u++)
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                const float2 vf = unpack_pair<T>(vsr[u][nt]);
                const float vv[2] = {vf.x, vf.y};
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const float pe = __expf(pv[u][nt][e] - m_new);
                    psum += pe;
                    const bool live = base + 16 * u + 8 * nt + 2 * t + e < row_end;  // past the end the ring holds no scale
                    pv[u][nt][e] = live ? pe * vv[e] : 0.f;  // the V scale of the row rides on P
                }
            }
        l_run = l_run * alpha + psum;
        m_run = m_new;
        const float al0 = __shfl_sync(0xffffffffu, alpha, 8 * t), al1 = __shfl_sync(0xffffffffu, alpha, 8 * t + 4);
#pragma unroll
        for (int j = 0; j < NACC; j++) {
            o[j][0] *= al0;
            o[j][1] *= al1;
            o[j][2] *= al0;
            o[j][3] *= al1;
        }
        // ---- O^T += V^T P^T ----
#pragma unroll
        for (int u = 0; u < 2; u++) {
            uint32_t pb0h, pb0l, pb1h, pb1l;
            split_pack<T>(pv[u][0][0], pv[u][0][1], pb0h, pb0l);
            split_pack<T>(pv[u][1][0], pv[u][1][1], pb1h, pb1l);
#pragma unroll
            for (int j = 0; j < NACC; j++) {
                // bytes (2j, 2j+1) of this lane's V bytes, rows (2t, 2t+1) and (2t+8, 2t+9), interleaved by row and converted
                const uint32_t sel = (j & 1) ? 0x7362u : 0x5140u;
                uint32_t a0, a1, a2, a3;
                cvt_s8x4<F16>(__byte_perm(vr[u][0][j >> 1], vr[u][1][j >> 1], sel), a0, a1);
                cvt_s8x4<F16>(__byte_perm(vr[u][2][j >> 1], vr[u][3][j >> 1], sel), a2, a3);
                mma_kv<T>(o[j], a0, a1, a2, a3, pb0h, pb1h);
                mma_kv<T>(o[j], a0, a1, a2, a3, pb0l, pb1l);
            }
        }
    }
    if constexpr (RING) {
        __syncwarp();
        decode_tail<T, D, NACC, MapQ8<VB>, true>(p, o, m_run, l_run, reinterpret_cast<float *>(ring_raw), (int)(kQ8RingDepth * kTile / 4));
    } else {
        decode_tail<T, D, NACC, MapQ8<VB>>(p, o, m_run, l_run);
    }
}

// Generic form: one warp per (b, h, sq) query row, the CPU kernel's recurrence row by row with the two scales.
template <typename T, int MAXE>
__global__ void attention_q8_generic_kernel(T *out, const T *q, const int8_t *k, const int8_t *v, const T *k_scale,
                                            const T *v_scale, float scale, int B, int Hq, int Hkv, int Sq, int Sk, int D,
                                            int active_host, const int32_t *active_dev, int is_causal, int out_bshd) {
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)B * Hq * Sq) return;
    const int sq = (int)(wid % Sq);
    const long long bh = wid / Sq;
    const int h = (int)(bh % Hq), b = (int)(bh / Hq);
    const int kvh = h / (Hq / Hkv);
    const int active = active_dev ? *active_dev : active_host;
    int bound = active;
    if (is_causal) bound = min(bound, active - Sq + sq + 1);
    bound = min(bound, Sk);
    const T *qp = q + (size_t)wid * D;
    const size_t head = (size_t)(b * Hkv + kvh) * Sk;
    const int8_t *kp = k + head * D, *vp = v + head * D;
    float qr[MAXE], o[MAXE];
#pragma unroll
    for (int e = 0; e < MAXE; e++) {
        const int d = lane + 32 * e;
        qr[e] = d < D ? to_f32<T>(qp[d]) : 0.f;
        o[e] = 0.f;
    }
    float m = -INFINITY, s = 0.f;
    for (int r = 0; r < bound; r++) {
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < MAXE; e++) {
            const int d = lane + 32 * e;
            if (d < D) dot += qr[e] * (float)kp[(size_t)r * D + d];
        }
        const float qk = warp_sum(dot) * to_f32<T>(k_scale[head + r]) * scale;
        const float m_new = fmaxf(m, qk);
        const float f = expf(m - m_new), ev = expf(qk - m_new);
        s = s * f + ev;
        const float evs = ev * to_f32<T>(v_scale[head + r]);
#pragma unroll
        for (int e = 0; e < MAXE; e++) {
            const int d = lane + 32 * e;
            if (d < D) o[e] = o[e] * f + evs * (float)vp[(size_t)r * D + d];
        }
        m = m_new;
    }
#pragma unroll
    for (int e = 0; e < MAXE; e++) {
        const int d = lane + 32 * e;
        const size_t orow = out_bshd ? ((size_t)b * Sq + sq) * Hq + h : (size_t)wid;
        if (d < D) out[orow * D + d] = from_f32<T>(o[e] / s);
    }
}

template <typename T>
static int launch_q8_generic(cudaStream_t st, void *out, const void *q, const void *k, const void *v, const void *ks,
                             const void *vs, float scale, int B, int Hq, int Hkv, int Sq, int Sk, int D, int active,
                             const int32_t *active_dev, int causal, int out_bshd) {
    const long long rows = (long long)B * Hq * Sq;
    const unsigned blocks = (unsigned)((rows * 32 + 127) / 128);
#define GEN(MAXE)                                                                                                        \
    attention_q8_generic_kernel<T, MAXE><<<blocks, 128, 0, st>>>((T *)out, (const T *)q, (const int8_t *)k, (const int8_t *)v, \
                                                                (const T *)ks, (const T *)vs, scale, B, Hq, Hkv, Sq, Sk, D,   \
                                                                active, active_dev, causal, out_bshd)
    if (D <= 32) GEN(1);
    else if (D <= 64) GEN(2);
    else if (D <= 128) GEN(4);
    else if (D <= 256) GEN(8);
    else if (D <= 512) GEN(16);
    else return fail(MYNN_E_UNSUPPORTED, "attention_q8: head dim %d > 512", D);
#undef GEN
    MYNN_LAUNCH_OK("attention_q8_generic_kernel");
    return MYNN_OK;
}

// Reads and clears the status word of the ring form (the stream must be idle).
int attention_decode_q8_take_status(int *status) {
    *status = 0;
    MYNN_CUDA_OK(cudaMemcpyFromSymbol(status, g_q8_ring_status, sizeof *status));
    if (*status) {
        const int zero = 0;
        MYNN_CUDA_OK(cudaMemcpyToSymbol(g_q8_ring_status, &zero, sizeof zero));
    }
    return MYNN_OK;
}

// The ring form: head_dim 128 (a row is one 128-byte box line), scale rows that a 16-byte bulk copy can address, the
// driver's tensor-map encoder, and tensor rows that fit a 32-bit coordinate.
static bool q8_ring_possible(const DecodeParams &p, int B, int D) {
    return g_decode_ring && D == 128 && p.cache_seq % 8 == 0 && tensor_map_api_available() &&
           (((uintptr_t)p.k_scale | (uintptr_t)p.v_scale) % 16) == 0 && (long long)B * p.Hkv * p.cache_seq < (1ll << 31);
}

template <typename T, int D>
static int launch_decode_q8(cudaStream_t st, const DecodeParams &p, int B, bool ring) {
    CUtensorMap mk, mv;
    memset(&mk, 0, sizeof mk);
    memset(&mv, 0, sizeof mv);
    if constexpr (D == 128) {
        if (ring) {
            const uint64_t rows = (uint64_t)B * p.Hkv * p.cache_seq;
            if (int rc = make_map(&mk, p.k, rows, D, D, 32)) return rc;
            if (int rc = make_map(&mv, p.v, rows, D, D, 32)) return rc;
            constexpr size_t smem = (size_t)kAttnWarps * kQ8RingDepth * 2 * 32 * 128;
            auto kern = attention_decode_q8_kernel<T, D, true>;
            static bool attr_set = false;
            if (!attr_set) {
                MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                attr_set = true;
            }
            MYNN_CUDA_OK(launch_pdl(kern, dim3(p.splits, p.Hkv, B), dim3(kAttnWarps * 32), smem, st, mk, mv, p));
            MYNN_LAUNCH_OK("attention_decode_q8_kernel");
            return MYNN_OK;
        }
    }
    MYNN_CUDA_OK(launch_pdl(attention_decode_q8_kernel<T, D, false>, dim3(p.splits, p.Hkv, B), dim3(kAttnWarps * 32), 0, st, mk, mv, p));
    MYNN_LAUNCH_OK("attention_decode_q8_kernel");
    return MYNN_OK;
}

// out[bh, s, :] = T(cache[bh, s, :] * scale[bh, s]) for the live rows s < active: the 16-bit copy of an int8 cache that the
// tensor-core prefill attention reads (rounded once to T, like the rows of a 16-bit cache).  16 elements per thread.
template <typename T>
__global__ void __launch_bounds__(256)
dequant_kv_rows_kernel(T *out, const int8_t *cache, const T *scale, int cache_seq, int D, int active_host, const int32_t *active_dev) {
    const int active = min(active_dev ? *active_dev : active_host, cache_seq);
    const int groups = D >> 4;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)active * groups) return;
    const int s = (int)(idx / groups), g = (int)(idx - (long long)s * groups);
    const size_t row = (size_t)blockIdx.y * cache_seq + s;
    const float sc = to_f32<T>(scale[row]);
    int8_t q[16];
    *reinterpret_cast<uint4 *>(q) = *reinterpret_cast<const uint4 *>(cache + row * D + 16 * g);
    T o[16];
#pragma unroll
    for (int i = 0; i < 16; i++) o[i] = from_f32<T>((float)q[i] * sc);
    uint4 *dst = reinterpret_cast<uint4 *>(out + row * D + 16 * g);
    dst[0] = reinterpret_cast<const uint4 *>(o)[0];
    dst[1] = reinterpret_cast<const uint4 *>(o)[1];
}

int launch_dequant_kv_rows(cudaStream_t st, int dtype, void *out, const void *cache, const void *scale, int BH, int cache_seq, int D,
                           int active_host, const int32_t *active_dev) {
    if (BH == 0 || cache_seq == 0) return MYNN_OK;
    if (dtype == MYNN_F32 || D % 16 || (((uintptr_t)out | (uintptr_t)cache) % 16))
        return fail(MYNN_E_UNSUPPORTED, "dequant_kv_rows: 16-bit tensors with D a multiple of 16 and 16-byte aligned rows only");
    const int bound = active_dev ? cache_seq : (active_host < cache_seq ? active_host : cache_seq);
    if (bound <= 0) return MYNN_OK;
    const long long n = (long long)bound * (D / 16);
    const dim3 grid((unsigned)((n + 255) / 256), BH);
    if (dtype == MYNN_BF16)
        dequant_kv_rows_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((__nv_bfloat16 *)out, (const int8_t *)cache, (const __nv_bfloat16 *)scale, cache_seq, D, active_host, active_dev);
    else
        dequant_kv_rows_kernel<__half><<<grid, 256, 0, st>>>((__half *)out, (const int8_t *)cache, (const __half *)scale, cache_seq, D, active_host, active_dev);
    MYNN_LAUNCH_OK("dequant_kv_rows_kernel");
    return MYNN_OK;
}

int launch_attention_q8(cudaStream_t st, void *out, const void *q, const void *k, const void *v, const void *k_scale,
                        const void *v_scale, float scale, int B, int Hq, int Hkv, int Sq, int D, int cache_seq_len,
                        int active_seq_kv, const int32_t *active_seq_kv_dev, int is_causal, int dtype, void *workspace,
                        size_t workspace_bytes, int out_bshd) {
    if (B < 0 || Hq <= 0 || Hkv <= 0 || Sq < 0 || D <= 0 || cache_seq_len < 0 || active_seq_kv < 0)
        return fail(MYNN_E_ARG, "attention_q8: bad shape");
    if (Hq % Hkv != 0) return fail(MYNN_E_ARG, "attention_q8: %d query heads are not a multiple of %d kv heads", Hq, Hkv);
    if (!dtype_ok(dtype)) return fail(MYNN_E_ARG, "attention_q8: bad dtype %d", dtype);
    if (B == 0 || Sq == 0) return MYNN_OK;
    if (!out || !q || !k || !v || !k_scale || !v_scale) return fail(MYNN_E_ARG, "attention_q8: null pointer");
    const int G = Hq / Hkv;
    const bool aligned = (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) % 16) == 0;
    const bool fast = Sq == 1 && (D == 64 || D == 128) && G <= 8 && dtype != MYNN_F32 && aligned;
    if (!fast) {
        if (dtype == MYNN_F32) return launch_q8_generic<float>(st, out, q, k, v, k_scale, v_scale, scale, B, Hq, Hkv, Sq, cache_seq_len, D, active_seq_kv, active_seq_kv_dev, is_causal, out_bshd);
        if (dtype == MYNN_BF16) return launch_q8_generic<__nv_bfloat16>(st, out, q, k, v, k_scale, v_scale, scale, B, Hq, Hkv, Sq, cache_seq_len, D, active_seq_kv, active_seq_kv_dev, is_causal, out_bshd);
        return launch_q8_generic<__half>(st, out, q, k, v, k_scale, v_scale, scale, B, Hq, Hkv, Sq, cache_seq_len, D, active_seq_kv, active_seq_kv_dev, is_causal, out_bshd);
    }
    DecodeParams p;
    p.out = out;
    p.q = q;
    p.k = k;
    p.v = v;
    p.k_scale = k_scale;
    p.v_scale = v_scale;
    p.limbs = nullptr;
    p.ascale = nullptr;
    p.scale = scale;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.G = G;
    p.cache_seq = cache_seq_len;
    p.active_host = active_seq_kv;
    p.active_dev = active_seq_kv_dev;
    const int rows_bound = active_seq_kv_dev ? cache_seq_len : (active_seq_kv < cache_seq_len ? active_seq_kv : cache_seq_len);
    const bool ring = q8_ring_possible(p, B, D);
    p.splits = decode_splits(B, Hkv, rows_bound, 32, ring ? 2 : kAttnCtasPerSm);
    if (int rc = decode_bind_workspace(p, B, D, workspace, workspace_bytes)) return rc;
    if (dtype == MYNN_BF16) return D == 64 ? launch_decode_q8<__nv_bfloat16, 64>(st, p, B, ring) : launch_decode_q8<__nv_bfloat16, 128>(st, p, B, ring);
    return D == 64 ? launch_decode_q8<__half, 64>(st, p, B, ring) : launch_decode_q8<__half, 128>(st, p, B, ring);
}

}  // namespace mynn

using namespace mynn;

extern "C" int mynn_b200_quantizing_kv_cache_update(void *stream, int8_t *cache, void *scale, const void *new_kv, int BH,
                                                    int cache_seq_len, int new_seq_len, int D, int offset,
                                                    const int32_t *offset_dev, int dtype) {
    if (BH < 0 || cache_seq_len < 0 || new_seq_len < 0 || D <= 0) return fail(MYNN_E_ARG, "quantizing_kv_cache_update: bad shape");
    if (!dtype_ok(dtype)) return fail(MYNN_E_ARG, "quantizing_kv_cache_update: bad dtype %d", dtype);
    if (BH == 0 || new_seq_len == 0) return MYNN_OK;
    if (!cache || !scale || !new_kv) return fail(MYNN_E_ARG, "quantizing_kv_cache_update: null pointer");
    if (!offset_dev && (offset < 0 || offset + new_seq_len > cache_seq_len))
        return fail(MYNN_E_ARG, "quantizing_kv_cache_update: rows [%d, %d) fall outside the cache of %d rows", offset, offset + new_seq_len, cache_seq_len);
    const long long rows = (long long)BH * new_seq_len;
    const unsigned blocks = (unsigned)((rows * 32 + 255) / 256);
    MYNN_DISPATCH_DTYPE(dtype, T, {
        quant_kv_update_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>(cache, (T *)scale, (const T *)new_kv, rows, cache_seq_len,
                                                                            new_seq_len, D, offset, offset_dev);
    });
    MYNN_LAUNCH_OK("quant_kv_update_kernel");
    return MYNN_OK;
}

extern "C" int mynn_b200_attention_q8(void *stream, void *out, const void *q, const int8_t *k, const int8_t *v,
                                      const void *k_scale, const void *v_scale, float scale, int B, int Hq, int Hkv, int Sq,
                                      int D, int cache_seq_len, int active_seq_kv, const int32_t *active_seq_kv_dev,
                                      int is_causal, int dtype, void *workspace, size_t workspace_bytes) {
    return mynn::launch_attention_q8((cudaStream_t)stream, out, q, k, v, k_scale, v_scale, scale, B, Hq, Hkv, Sq, D,
                                     cache_seq_len, active_seq_kv, active_seq_kv_dev, is_causal, dtype, workspace,
                                     workspace_bytes, 0);
}
