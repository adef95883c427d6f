// Pieces shared by the decode-attention kernels (16-bit KV cache and int8 KV cache): launch parameters, the
// mma.m16n8k16 wrappers, the split of the kv rows over CTAs and the tail that merges warps and splits.
#pragma once
#include <type_traits>

#include "common.cuh"

namespace mynn {

constexpr int kAttnWarps = 4;
constexpr int kMaxSplits = 64;
constexpr int kAttnCtasPerSm = 4;  // resident CTAs per SM the kernels are built for (<= 128 registers, 17 KB smem)

__device__ __forceinline__ uint4 ldg_16(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_8(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

template <typename T>
__device__ __forceinline__ void mma_kv(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    if constexpr (std::is_same<T, __half>::value) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

// pack hi parts of (x, y) into one 32-bit register and the rounding remainders into another
template <typename T>
__device__ __forceinline__ void split_pack(float x, float y, uint32_t &hi, uint32_t &lo) {
    const T xh = from_f32<T>(x), yh = from_f32<T>(y);
    const T xl = from_f32<T>(x - to_f32<T>(xh)), yl = from_f32<T>(y - to_f32<T>(yh));
    hi = (uint32_t)reinterpret_cast<const uint16_t &>(xh) | ((uint32_t)reinterpret_cast<const uint16_t &>(yh) << 16);
    lo = (uint32_t)reinterpret_cast<const uint16_t &>(xl) | ((uint32_t)reinterpret_cast<const uint16_t &>(yl) << 16);
}

struct DecodeParams {
    void *out;
    const void *q, *k, *v;
    const void *k_scale, *v_scale;  // int8 cache only: one scale per (batch, kv head, row), storage dtype
    float scale;
    int Hq, Hkv, G, cache_seq;
    int active_host;
    const int32_t *active_dev;
    int splits;
    float *ws_o;          // [B*Hkv][splits][8][D]
    float *ws_ml;         // [B*Hkv][splits][8][2]
    unsigned *ws_ticket;  // [B*Hkv], zero before first use; the combining CTA re-zeroes it
    // Optional: the finished output row of a sequence ([Hq * D], one query row) is also left as activation limbs for the
    // DequantMatMul that follows (o_proj), by the CTA that completes the row.
    int8_t *limbs;        // [3 B][Hq * D] limb rows (3 b + l), or null
    float *ascale;        // [B] row scales
    unsigned *row_ticket; // [B], zero before first use; re-zeroed by the CTA that converts the row
    // Optional (16-bit decode kernel): RoPE and the KV append fused in.  q then points at the UNROTATED projection output
    // (row b at q + b * qkv_stride elements, heads contiguous), fused_k / fused_v at the new key / value of (row b, kv head h)
    // = fused_k + b * qkv_stride + h * D; the new row is rotated (k) at table row *fused_pos, written to cache row
    // *fused_row, and takes part in the attention as row *fused_row; the cache is read for the rows before it.
    const void *fused_k = nullptr, *fused_v = nullptr;
    long long qkv_stride = 0;
    const void *cos_t = nullptr, *sin_t = nullptr;
    const int64_t *fused_pos = nullptr;
    const int32_t *fused_row = nullptr;
    int *status = nullptr;  // ring kernel: where a timed-out wait is recorded (null: the library's own word, see attention_check)
};

// Called by every CTA that has stored final outputs of (batch b, one kv head): the last of the Hkv to arrive converts the
// whole row to limbs with the arithmetic of the limb pre-pass (23-bit fixed point, power-of-two row scale).
template <typename T, int D>
__device__ __forceinline__ void decode_row_limbs(const DecodeParams &p, int b, unsigned *sm_flag, float *sm_red) {
    if (p.limbs == nullptr) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) *sm_flag = (atomicAdd(&p.row_ticket[b], 1u) == (unsigned)(p.Hkv - 1)) ? 1u : 0u;
    __syncthreads();
    if (!*sm_flag) return;
    __threadfence();
    const int K = p.Hq * D;
    const T *row = reinterpret_cast<const T *>(p.out) + (size_t)b * K;
    // up to 8 x 4 elements per thread are fetched in one go (one L2 round trip) and kept for the second pass; longer rows
    // are read again
    constexpr int kKeep = 8, kStride = 4 * kAttnWarps * 32;
    uint2 raw[kKeep];
    float mx = 0.f;
    bool bad = false;
#pragma unroll
    for (int u = 0; u < kKeep; u++) {
        const int i = 4 * threadIdx.x + u * kStride;
        raw[u] = i < K ? __ldcg(reinterpret_cast<const uint2 *>(row + i)) : make_uint2(0u, 0u);
    }
    auto scan = [&](const uint2 &r) {
        const T *e = reinterpret_cast<const T *>(&r);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float v = to_f32<T>(e[j]);
            bad |= !(fabsf(v) <= 3.0e38f);
            mx = fmaxf(mx, fabsf(v));
        }
    };
#pragma unroll
    for (int u = 0; u < kKeep; u++) scan(raw[u]);
#pragma unroll 1
    for (int i = 4 * threadIdx.x + kKeep * kStride; i < K; i += kStride) scan(__ldcg(reinterpret_cast<const uint2 *>(row + i)));
    mx = warp_max(mx);
    const unsigned anybad = __syncthreads_or(bad);
    if ((threadIdx.x & 31) == 0) sm_red[threadIdx.x >> 5] = mx;
    __syncthreads();
    float t = sm_red[0];
#pragma unroll
    for (int w = 1; w < kAttnWarps; w++) t = fmaxf(t, sm_red[w]);
    int e2 = 0;
    if (t > 0.f) frexpf(t, &e2);
    const float sc1 = t > 0.f ? ldexpf(1.0f, 22 - e2) : 1.0f;
    const float sc = anybad ? 0.f : sc1;
    if (threadIdx.x == 0) p.ascale[b] = anybad ? __int_as_float(0x7fc00000) : 1.0f / sc1;
    uint32_t *l0 = reinterpret_cast<uint32_t *>(p.limbs + (size_t)(3 * b) * K);
    uint32_t *l1 = reinterpret_cast<uint32_t *>(p.limbs + (size_t)(3 * b + 1) * K);
    uint32_t *l2 = reinterpret_cast<uint32_t *>(p.limbs + (size_t)(3 * b + 2) * K);
    auto emit = [&](const uint2 &r, int i) {
        const T *e = reinterpret_cast<const T *>(&r);
        uint32_t w0 = 0, w1 = 0, w2 = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int A = sc == 0.f ? 0 : __float2int_rn(to_f32<T>(e[j]) * sc);
            const int d0 = (int)(int8_t)(A & 0xFF);
            A = (A - d0) >> 8;
            const int d1 = (int)(int8_t)(A & 0xFF);
            A = (A - d1) >> 8;
            w0 |= (uint32_t)(d0 & 0xFF) << (8 * j);
            w1 |= (uint32_t)(d1 & 0xFF) << (8 * j);
            w2 |= (uint32_t)(A & 0xFF) << (8 * j);
        }
        l0[i >> 2] = w0;
        l1[i >> 2] = w1;
        l2[i >> 2] = w2;
    };
#pragma unroll
    for (int u = 0; u < kKeep; u++) {
        const int i = 4 * threadIdx.x + u * kStride;
        if (i < K) emit(raw[u], i);
    }
#pragma unroll 1
    for (int i = 4 * threadIdx.x + kKeep * kStride; i < K; i += kStride) emit(__ldcg(reinterpret_cast<const uint2 *>(row + i)), i);
    if (threadIdx.x == 0) p.row_ticket[b] = 0u;
}

// Tail of a decode CTA.  Every lane holds NACC accumulator tiles of O^T: tile i, registers {0,1,2,3} are
// (head 2t, d), (head 2t+1, d), (head 2t, d+1), (head 2t+1, d+1) with d = DMap::d(i, g).  The warps are merged through
// shared memory; with more than one split the partial result goes to the workspace and the last CTA of the
// (batch, kv head) pair to arrive (atomic ticket, no spinning) combines the splits and writes the output.
// ext != nullptr: the per-warp output staging rows live in caller-provided shared memory, warp w's [8][D] floats at
// ext + w * ext_stride (the ring kernel hands every warp a piece of its own, by then idle, ring).
template <typename T, int D, int NACC, typename DMap, bool EXT = false>
__device__ __forceinline__ void decode_tail(const DecodeParams &p, const float (&o)[NACC][4], float m_run, float l_run,
                                            float *ext = nullptr, int ext_stride = 0) {
    float *so_base;
    int so_stride;
    if constexpr (EXT) {
        so_base = ext;
        so_stride = ext_stride;
    } else {
        __shared__ float sm_o[kAttnWarps][8][D];
        so_base = &sm_o[0][0][0];
        so_stride = 8 * D;
    }
    __shared__ float sm_m[kAttnWarps][8], sm_l[kAttnWarps][8];
    __shared__ unsigned sm_last, sm_row_last;
    __shared__ float sm_red[kAttnWarps];
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int G = p.G;

    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (t == 0) {
        sm_m[warp][g] = m_run;
        sm_l[warp][g] = l_run;
    }
#pragma unroll
    for (int i = 0; i < NACC; i++) {
        const int d = DMap::d(i, g);
        float *so = so_base + (size_t)warp * so_stride;
        so[(2 * t) * D + d] = o[i][0];
        so[(2 * t + 1) * D + d] = o[i][1];
        so[(2 * t) * D + d + 1] = o[i][2];
        so[(2 * t + 1) * D + d + 1] = o[i][3];
    }
    __syncthreads();

    const size_t pair = (size_t)b * p.Hkv + kvh;
    T *outp = reinterpret_cast<T *>(p.out) + (size_t)(b * p.Hq + kvh * G) * D;
    for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
        const int hd = idx / D, d = idx - hd * D;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; w++) mx = fmaxf(mx, sm_m[w][hd]);
        float L = 0.f, O = 0.f;
        if (mx > -INFINITY) {
#pragma unroll
            for (int w = 0; w < kAttnWarps; w++) {
                const float f = __expf(sm_m[w][hd] - mx);
                L += sm_l[w][hd] * f;
                O += so_base[(size_t)w * so_stride + hd * D + d] * f;
            }
        }
        if (p.splits == 1) {
            outp[(size_t)hd * D + d] = from_f32<T>(O / L);
        } else {
            const size_t slot = (pair * p.splits + split) * 8 + hd;
            p.ws_o[slot * D + d] = O;
            if (d == 0) {
                p.ws_ml[slot * 2] = mx;
                p.ws_ml[slot * 2 + 1] = L;
            }
        }
    }
    if (p.splits == 1) {
        decode_row_limbs<T, D>(p, b, &sm_row_last, sm_red);
        return;
    }

    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) sm_last = (atomicAdd(&p.ws_ticket[pair], 1u) == (unsigned)(p.splits - 1)) ? 1u : 0u;
    __syncthreads();
    if (!sm_last) return;
    __threadfence();
    for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
        const int hd = idx / D, d = idx - hd * D;
        // eight splits at a time, all of their loads issued before any is used: the combine costs one L2 round trip per
        // eight splits instead of four dependent ones per split
        float mx = -INFINITY, L = 0.f, O = 0.f;
        for (int s0 = 0; s0 < p.splits; s0 += 8) {
            float ms[8], ls[8], os[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const bool in = s0 + j < p.splits;
                const size_t slot = (pair * p.splits + (in ? s0 + j : s0)) * 8 + hd;
                ms[j] = in ? __ldcg(&p.ws_ml[slot * 2]) : -INFINITY;
                ls[j] = in ? __ldcg(&p.ws_ml[slot * 2 + 1]) : 0.f;
                os[j] = in ? __ldcg(&p.ws_o[slot * D + d]) : 0.f;
            }
            float cm = mx;
#pragma unroll
            for (int j = 0; j < 8; j++) cm = fmaxf(cm, ms[j]);
            if (cm == -INFINITY) continue;  // nothing but empty splits so far
            const float f0 = __expf(mx - cm);  // 0 while mx is still -inf
            L *= f0;
            O *= f0;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                if (ms[j] == -INFINITY) continue;
                const float f = __expf(ms[j] - cm);
                L += ls[j] * f;
                O += os[j] * f;
            }
            mx = cm;
        }
        outp[(size_t)hd * D + d] = from_f32<T>(O / L);
    }
    if (threadIdx.x == 0) p.ws_ticket[pair] = 0u;
    decode_row_limbs<T, D>(p, b, &sm_row_last, sm_red);
}

// How many CTAs share the rows of one (batch, kv head) pair.  All CTAs of a launch last equally long, so the grid should fit
// in ONE wave of resident CTAs (148 SMs): a partly filled second wave would cost as much time as a full one.  A split is not
// free either: its partial result goes through the merge (a round trip through L2 per eight splits, plus the tail of one
// more CTA), so a split gets at least four tiles per warp, and more than eight splits are only used when a split would
// otherwise be longer than 32 tiles per warp.  (Measured, 2048 rows, 32 pairs: 1 / 2 / 4 / 8 / 16 / 32 splits = 30 / 21 / 15 /
// 16 / 22 / 33 us; 256 rows, 4 pairs: 1 / 2 / 4 splits = 4.8 / 7.4 / 7.2 us.)
inline int decode_splits(int B, int Hkv, int rows_bound, int tile_rows = 16, int ctas_per_sm = kAttnCtasPerSm) {
    const int pairs = B * Hkv;
    const int round = tile_rows * kAttnWarps;  // rows the four warps of a CTA take at a time
    int s = (ctas_per_sm * 148) / pairs;
    int cap = rows_bound / (4 * round);
    if (cap < 1) cap = 1;
    if (s > cap) s = cap;
    if (s < 1) s = 1;
    if (s > 8) {
        const int long_rows = rows_bound / (32 * round);
        s = s < long_rows ? s : long_rows;
        if (s < 8) s = 8;
        s &= ~7;  // the merge takes the splits eight at a time
    }
    if (s > kMaxSplits) s = kMaxSplits;
    return s;
}

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Splits `workspace` into the ticket / (max, sum) / partial-output areas of a decode launch; fails if it is too small.
int decode_bind_workspace(DecodeParams &p, int B, int D, void *workspace, size_t workspace_bytes);

}  // namespace mynn
