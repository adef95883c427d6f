// GQA attention over the KV cache for sm_100a.
//
// Decode (one query token per sequence) is bound by reading K and V once from HBM.  The decode kernel
//   * assigns one CTA to (kv-row split, kv head, batch) so that all query heads of a GQA group share a single
//     pass over their KV head (the engine's kernel re-reads the KV head once per query head and walks the rows
//     serially, src/codegen/cuda/cpp/attention.cuh:495-606);
//   * lets each of its 4 warps take 16-row tiles laid out as mma.m16n8k16 operand fragments: the head-dim index (for
//     QK^T) and the kv-row pairing (for PV) are permuted so that a 16-byte piece of a row IS a fragment and no transpose
//     is needed.  The pieces come out of per-warp rings in shared memory that the TMA engine fills three tiles ahead
//     (default), or straight from global memory with 128-bit loads (MYNN_OPT_DECODE_RING = 0: 128 registers, 4 CTAs per SM);
//   * computes S = Q K^T (A = Q, padded to 16 heads) and O^T = V^T P^T (A = V^T, B = P^T, so the 8-column B tile is
//     the head group and no accumulator register is wasted) on the tensor cores with f32 accumulation and an
//     online softmax in f32; P enters as a high 16-bit part plus its rounding remainder (~16 significant bits);
//   * in the decoder step also rotates q and the new key and appends the new key / value rows (RoPE + KVCacheUpdate),
//     and leaves a finished output row as the activation limbs of the o_proj DequantMatMul;
//   * merges the warps through shared memory, and the splits through a small global workspace where the last
//     CTA to arrive (atomic ticket, no spinning) combines the partial results and writes the output.
// Everything else (f32 tensors, head dims other than 64/128, groups larger than 8, more than one query row,
// causal masks) goes to a generic one-warp-per-query-row kernel that follows the CPU recurrence literally.
#include <atomic>
#include <cstring>
#include <type_traits>

#include "attention_internal.cuh"
#include "common.cuh"
#include "i8_gemm.cuh"
#include "ops_internal.cuh"
#include "tcgen05.cuh"

namespace mynn {

struct Map16 {  // accumulator tile i = 4h + j of the 16-bit kernel holds head-dim rows 64h + 8g + 2j (+1)
    static __device__ __forceinline__ int d(int i, int g) { return 64 * (i >> 2) + 8 * g + 2 * (i & 3); }
};

// grid (splits, Hkv, B), block 128.
// RING: the K / V rows do not go from global memory into the registers of the thread that needs them; every warp keeps a
// ring of kRingDepth 16-row tiles in shared memory that the TMA engine fills (cp.async.bulk.tensor over 2-D maps of the two
// caches, 16 rows x 128 bytes per box, 128-byte swizzle; tensor maps of this GPU's own memory, no multicast), and takes its
// fragments from there with 16-byte shared loads.  The loads of the next kRingDepth - 1 tiles are in flight while a tile
// is computed, without holding registers.  Each warp owns its ring and its barriers: the lane that issues the copies is
// lane 0 of the consuming warp, after the warp has copied a tile into registers, so no second barrier is needed.
constexpr int kRingDepth = 3;
__device__ int g_ring_status;  // 31: a wait for a tile ran out of time (read and cleared by mynn_b200_attention_check)
MYNN_DEFINE_WAIT_BUDGET_SETTER(attention_decode)

template <typename T, int D, bool RING>
__global__ void __launch_bounds__(kAttnWarps * 32, RING ? 2 : 4)
attention_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const DecodeParams p) {
    constexpr int KS = D / 16;   // k16 steps of QK^T
    constexpr int KCH = D / 32;  // 16-byte K chunks per lane per row
    constexpr int VH = D / 64;   // 16-byte V chunks per lane per row
    pdl_trigger();
    pdl_wait();  // q, the newest kv row and the active length come from the preceding kernels
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int G = p.G;
    int active = p.active_dev ? *p.active_dev : p.active_host;
    active = max(0, min(active, p.cache_seq));
    // whole rounds of the CTA's four warps (64 rows): a split that ends inside a round leaves some warps a tile short
    const int rows_per_split = (((active + p.splits - 1) / p.splits) + 16 * kAttnWarps - 1) / (16 * kAttnWarps) * (16 * kAttnWarps);
    const int row_beg = split * rows_per_split;
    const int row_end = min(row_beg + rows_per_split, active);

    const T *kbase = reinterpret_cast<const T *>(p.k) + (size_t)(b * p.Hkv + kvh) * p.cache_seq * D;
    const T *vbase = reinterpret_cast<const T *>(p.v) + (size_t)(b * p.Hkv + kvh) * p.cache_seq * D;

    const bool fused = p.fused_k != nullptr;  // RoPE + KV append happen here instead of in a kernel of their own
    const int new_row = fused ? *p.fused_row : -1;
    const size_t tab = fused ? (size_t)(*p.fused_pos) * D : 0;
    const T *cos_t = reinterpret_cast<const T *>(p.cos_t), *sin_t = reinterpret_cast<const T *>(p.sin_t);
    // the rows this CTA reads from the cache: with the fused append the new row is not there yet
    const int cache_end = fused ? min(row_end, new_row) : row_end;

    // Ring set-up and the copies of the first tiles come first: they travel while the query fragments are built.
    extern __shared__ __align__(1024) uint8_t ring_raw[];
    constexpr int NB = D / 64;                      // 128-byte boxes per K (and per V) row
    constexpr uint32_t kBox = 16 * 128;             // one box: 16 rows x 128 bytes
    constexpr uint32_t kTile = 2 * NB * kBox;       // K boxes, then V boxes
    __shared__ uint64_t full[RING ? kAttnWarps : 1][kRingDepth];
    __shared__ int abort_flag;
    uint8_t *ring = ring_raw + (size_t)warp * kRingDepth * kTile;
    const int first = row_beg + 16 * warp;
    const int ntile = first < cache_end ? (cache_end - first + 16 * kAttnWarps - 1) / (16 * kAttnWarps) : 0;
    const int y0 = (b * p.Hkv + kvh) * p.cache_seq + first;  // tensor row of this warp's first tile
    auto issue = [&](int j) {  // lane 0: tile j of this warp into stage j % depth
        if constexpr (RING) {
            const int s = j % kRingDepth;
            uint8_t *st = ring + (size_t)s * kTile;
            const int y = y0 + 16 * kAttnWarps * j;
            mbar_expect_tx(&full[warp][s], kTile);
#pragma unroll
            for (int hf = 0; hf < NB; hf++) {
                tma_load_2d(st + hf * kBox, &map_k, 128 * hf, y, &full[warp][s]);  // byte maps: x counts bytes
                tma_load_2d(st + (NB + hf) * kBox, &map_v, 128 * hf, y, &full[warp][s]);
            }
        }
    };
    if constexpr (RING) {
        if (threadIdx.x == 0) abort_flag = 0;
        if (lane == 0) {
#pragma unroll
            for (int s = 0; s < kRingDepth; s++) mbar_init(&full[warp][s], 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncthreads();
        if (lane == 0)
            for (int j = 0; j < min(ntile, kRingDepth); j++) issue(j);
    }
    // x rotated against its partner xp (the element half a head away): low half x c - xp s, high half x c + xp s, rounded to
    // the storage type as the stand-alone RoPE kernel rounds it
    auto rot4 = [&](uint2 x, uint2 xp, int d0, bool low) {
        const uint2 c = *reinterpret_cast<const uint2 *>(cos_t + tab + d0), sn = *reinterpret_cast<const uint2 *>(sin_t + tab + d0);
        const T *xe = reinterpret_cast<const T *>(&x), *pe = reinterpret_cast<const T *>(&xp);
        const T *ce = reinterpret_cast<const T *>(&c), *se = reinterpret_cast<const T *>(&sn);
        uint2 r;
        T *re = reinterpret_cast<T *>(&r);
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float a = to_f32<T>(xe[e]), b_ = to_f32<T>(pe[e]);
            re[e] = from_f32<T>(low ? rope_low(a, b_, to_f32<T>(ce[e]), to_f32<T>(se[e])) : rope_high(b_, a, to_f32<T>(ce[e]), to_f32<T>(se[e])));
        }
        return r;
    };

    // Q fragments of head g (zero for padding rows g >= G)
    uint32_t qa0[KS], qa2[KS];
    {
        const T *qrow = fused ? reinterpret_cast<const T *>(p.q) + (size_t)b * p.qkv_stride + (size_t)(kvh * G + min(g, G - 1)) * D
                              : reinterpret_cast<const T *>(p.q) + (size_t)(b * p.Hq + kvh * G + min(g, G - 1)) * D;
        uint2 raw[KS];
#pragma unroll
        for (int ks = 0; ks < KS; ks++) raw[ks] = *reinterpret_cast<const uint2 *>(qrow + 8 * (t + 4 * (ks >> 1)) + 4 * (ks & 1));
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            // the partner of elements d0 .. d0+3 lies half a head away: fragment ks ^ (KS / 2) of this same lane
            const int d0 = 8 * (t + 4 * (ks >> 1)) + 4 * (ks & 1);
            const uint2 w = fused ? rot4(raw[ks], raw[ks ^ (KS / 2)], d0, d0 < D / 2) : raw[ks];
            qa0[ks] = g < G ? w.x : 0u;
            qa2[ks] = g < G ? w.y : 0u;
        }
    }

    // O^T accumulators: tile (h, j) holds head-dim rows d = 64h + 8g + 2j (+1 for the g+8 half) against head columns
    // 2t, 2t+1 -- every register is useful for an 8-head group, so the whole output needs D/4 registers.
    float o[VH * 4][4];
#pragma unroll
    for (int j = 0; j < VH * 4; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) o[j][i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;

    // One 16-row tile whose K / V fragments are in registers: rows base .. base+15, of which those below `end` count.
    auto tile = [&](const uint4 (&kr)[2][KCH], const uint4 (&vr)[4][VH], int base, int end) {
        // ---- S = Q K^T: s[nt][e] = S[head g][kv row base + 8nt + 2t + e] ----
        float s[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
            for (int i = 0; i < KCH; i++) {
                mma_kv<T>(s[nt], qa0[2 * i], 0u, qa2[2 * i], 0u, kr[nt][i].x, kr[nt][i].y);
                mma_kv<T>(s[nt], qa0[2 * i + 1], 0u, qa2[2 * i + 1], 0u, kr[nt][i].z, kr[nt][i].w);
            }
        }
        // ---- online softmax for head g ----
        float pv[2][2];
        float tmax = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int row = base + 8 * nt + 2 * t + e;
                pv[nt][e] = row < end ? s[nt][e] * p.scale : -INFINITY;
                tmax = fmaxf(tmax, pv[nt][e]);
            }
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        const float m_new = fmaxf(m_run, tmax);  // finite: the tile has at least one valid row
        const float alpha = __expf(m_run - m_new);
        float psum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                pv[nt][e] = __expf(pv[nt][e] - m_new);
                psum += pv[nt][e];
            }
        l_run = l_run * alpha + psum;  // per-lane partial; lanes of a group are summed at the end
        m_run = m_new;
        // P^T is the B operand of O^T = V^T P^T: (kv rows 2t,2t+1 | 2t+8,2t+9) x head g is exactly what this lane
        // holds.  P enters as a high 16-bit part and its rounding remainder (two MMAs), i.e. with ~16 significant bits.
        uint32_t pb0h, pb0l, pb1h, pb1l;
        split_pack<T>(pv[0][0], pv[0][1], pb0h, pb0l);
        split_pack<T>(pv[1][0], pv[1][1], pb1h, pb1l);
        // the accumulator columns of this lane are heads 2t and 2t+1: fetch their rescale factors
        const float al0 = __shfl_sync(0xffffffffu, alpha, 8 * t), al1 = __shfl_sync(0xffffffffu, alpha, 8 * t + 4);
        // ---- O^T = O^T * alpha + V^T P^T ----
#pragma unroll
        for (int h = 0; h < VH; h++) {
            const uint32_t r0[4] = {vr[0][h].x, vr[0][h].y, vr[0][h].z, vr[0][h].w};
            const uint32_t r1[4] = {vr[1][h].x, vr[1][h].y, vr[1][h].z, vr[1][h].w};
            const uint32_t r2[4] = {vr[2][h].x, vr[2][h].y, vr[2][h].z, vr[2][h].w};
            const uint32_t r3[4] = {vr[3][h].x, vr[3][h].y, vr[3][h].z, vr[3][h].w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                // A = V^T: rows (g | g+8) are head-dim elements 2j | 2j+1 of this lane's 8, columns are kv-row pairs
                const uint32_t a0 = __byte_perm(r0[j], r1[j], 0x5410u), a1 = __byte_perm(r0[j], r1[j], 0x7632u);
                const uint32_t a2 = __byte_perm(r2[j], r3[j], 0x5410u), a3 = __byte_perm(r2[j], r3[j], 0x7632u);
                float(&acc)[4] = o[4 * h + j];
                acc[0] *= al0;
                acc[1] *= al1;
                acc[2] *= al0;
                acc[3] *= al1;
                mma_kv<T>(acc, a0, a1, a2, a3, pb0h, pb1h);
                mma_kv<T>(acc, a0, a1, a2, a3, pb0l, pb1l);
            }
        }
    };

    const int last = cache_end - 1;
    if constexpr (RING) {
        for (int j = 0; j < ntile; j++) {
            const int s = j % kRingDepth;
            const int base = first + 16 * kAttnWarps * j;
            int ok_i = 1;
            if (lane == 0) ok_i = mbar_wait_spin(&full[warp][s], (j / kRingDepth) & 1, &abort_flag) ? 1 : 0;
            if (!__shfl_sync(0xffffffffu, ok_i, 0)) {  // the copy never arrived: report it, leave the rows out
                if (lane == 0) {
                    atomicExch(&abort_flag, 1);
                    atomicExch(p.status ? p.status : &g_ring_status, 31);
                }
                break;
            }
            const uint8_t *st = ring + (size_t)s * kTile;
            uint4 kr[2][KCH], vr[4][VH];
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                const int row = 8 * nt + g;  // row & 7 == g
#pragma unroll
                for (int i = 0; i < KCH; i++) {
                    // element 8t + 32i of the row = box i / 2, 16-byte chunk t + 4 (i % 2), stored at chunk ^ (row % 8)
                    const int c = (t + 4 * (i & 1)) ^ g;
                    kr[nt][i] = *reinterpret_cast<const uint4 *>(st + (i >> 1) * kBox + row * 128 + (c << 4));
                }
            }
#pragma unroll
            for (int r = 0; r < 4; r++) {
                const int row = 2 * t + (r & 1) + 8 * (r >> 1);
                const bool live = base + row < cache_end;  // rows past the end may hold anything: keep them out of P V
#pragma unroll
                for (int h = 0; h < VH; h++) {
                    const uint4 w = *reinterpret_cast<const uint4 *>(st + (NB + h) * kBox + row * 128 + ((g ^ (row & 7)) << 4));
                    vr[r][h] = live ? w : make_uint4(0u, 0u, 0u, 0u);
                }
            }
            __syncwarp();  // every lane has its fragments: the stage may be refilled
            if (lane == 0 && j + kRingDepth < ntile) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                issue(j + kRingDepth);
            }
            tile(kr, vr, base, cache_end);
        }
    } else {
    for (int base = row_beg + 16 * warp; base < cache_end; base += 16 * kAttnWarps) {
        // ---- issue all loads of this tile (rows past the end are clamped to a valid row and masked in the tile) ----
        uint4 kr[2][KCH], vr[4][VH];
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            const T *kp = kbase + (size_t)min(base + 8 * nt + g, last) * D + 8 * t;
#pragma unroll
            for (int i = 0; i < KCH; i++) kr[nt][i] = ldg_16(kp + 32 * i);
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int row = base + 2 * t + (r & 1) + 8 * (r >> 1);
            const T *vp = vbase + (size_t)min(row, last) * D + 8 * g;
#pragma unroll
            for (int h = 0; h < VH; h++) vr[r][h] = ldg_16(vp + 64 * h);
        }
        tile(kr, vr, base, cache_end);
    }
    }
    if (fused && warp == 0 && new_row >= row_beg && new_row < row_end) {
        // The new row of this (batch, kv head): rotate the key, store key and value into the cache for the steps to come, and
        // run them through one more tile in which only row 0 counts.  K row 0 of the tile lives in lanes g == 0 (chunks
        // 8t + 32i), V row 0 in lanes t == 0 (chunks 8g + 64h); everything else is zero.
        uint4 kr[2][KCH], vr[4][VH];
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int i = 0; i < KCH; i++) kr[nt][i] = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int h = 0; h < VH; h++) vr[r][h] = make_uint4(0u, 0u, 0u, 0u);
        T *kcache = const_cast<T *>(kbase) + (size_t)new_row * D, *vcache = const_cast<T *>(vbase) + (size_t)new_row * D;
        if (g == 0) {
            const T *kraw = reinterpret_cast<const T *>(p.fused_k) + (size_t)b * p.qkv_stride + (size_t)kvh * D;
            uint4 raw[KCH];
#pragma unroll
            for (int i = 0; i < KCH; i++) raw[i] = *reinterpret_cast<const uint4 *>(kraw + 8 * t + 32 * i);
#pragma unroll
            for (int i = 0; i < KCH; i++) {
                const int d0 = 8 * t + 32 * i;
                const uint4 x = raw[i], xp = raw[i ^ (KCH / 2)];
                const uint2 lo = rot4(make_uint2(x.x, x.y), make_uint2(xp.x, xp.y), d0, d0 < D / 2);
                const uint2 hi = rot4(make_uint2(x.z, x.w), make_uint2(xp.z, xp.w), d0 + 4, d0 < D / 2);
                kr[0][i] = make_uint4(lo.x, lo.y, hi.x, hi.y);
                *reinterpret_cast<uint4 *>(kcache + d0) = kr[0][i];
            }
        }
        if (t == 0) {
            const T *vraw = reinterpret_cast<const T *>(p.fused_v) + (size_t)b * p.qkv_stride + (size_t)kvh * D;
#pragma unroll
            for (int h = 0; h < VH; h++) {
                vr[0][h] = *reinterpret_cast<const uint4 *>(vraw + 8 * g + 64 * h);
                *reinterpret_cast<uint4 *>(vcache + 8 * g + 64 * h) = vr[0][h];
            }
        }
        tile(kr, vr, new_row, new_row + 1);
    }

    if constexpr (RING) {
        // the warps' staging rows for the merge reuse each warp's own ring (all of its copies have landed and been read)
        __syncwarp();
        decode_tail<T, D, VH * 4, Map16, true>(p, o, m_run, l_run, reinterpret_cast<float *>(ring_raw), (int)(kRingDepth * kTile / 4));
    } else {
        decode_tail<T, D, VH * 4, Map16>(p, o, m_run, l_run);
    }
}

// Generic attention: one warp per (b, h, sq) query row, the CPU kernel's recurrence row by row
// (m' = max(m, qk); f = exp(m - m'); e = exp(qk - m'); s = s f + e; o = o f + e v; out = o / s).
template <typename T, int MAXE>
__global__ void attention_generic_kernel(T *out, const T *q, const T *k, const T *v, float scale, int B, int Hq,
                                         int Hkv, int Sq, int Sk, int D, int active_host, const int32_t *active_dev,
                                         int is_causal, int out_bshd, int ring_sink, int ring_window, int ring_start,
                                         const T *mask, long long mask_outer_stride, long long mask_row_stride) {
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
    const T *kp = k + (size_t)(b * Hkv + kvh) * Sk * D;
    const T *vp = v + (size_t)(b * Hkv + kvh) * Sk * D;
    float qr[MAXE], o[MAXE];
#pragma unroll
    for (int e = 0; e < MAXE; e++) {
        const int d = lane + 32 * e;
        qr[e] = d < D ? to_f32<T>(qp[d]) : 0.f;
        o[e] = 0.f;
    }
    float m = -INFINITY, s = 0.f;
    for (int lr = 0; lr < bound; lr++) {
        // logical row -> physical slot of a sink + ring cache (identity when ring_window == 0)
        const int r = (ring_window == 0 || lr < ring_sink) ? lr : ring_sink + (ring_start + (lr - ring_sink)) % ring_window;
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < MAXE; e++) {
            const int d = lane + 32 * e;
            if (d < D) dot += qr[e] * to_f32<T>(kp[(size_t)r * D + d]);
        }
        float qk = warp_sum(dot) * scale;
        // additive mask, indexed as the engine's kernels do: (b * Hq + h) * outer stride + query row * row stride + kv row
        if (mask != nullptr) qk += to_f32<T>(mask[bh * mask_outer_stride + sq * mask_row_stride + lr]);
        const float m_new = fmaxf(m, qk);
        const float f = expf(m - m_new), ev = expf(qk - m_new);
        s = s * f + ev;
#pragma unroll
        for (int e = 0; e < MAXE; e++) {
            const int d = lane + 32 * e;
            if (d < D) o[e] = o[e] * f + ev * to_f32<T>(vp[(size_t)r * D + d]);
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

int decode_bind_workspace(DecodeParams &p, int B, int D, void *workspace, size_t workspace_bytes) {
    p.ws_o = nullptr;
    p.ws_ml = nullptr;
    p.ws_ticket = nullptr;
    p.row_ticket = nullptr;
    const size_t need = mynn_b200_attention_workspace_bytes(B, p.Hq, p.Hkv, D, p.cache_seq);
    const bool have_ws = workspace && workspace_bytes >= need;
    const size_t pairs = (size_t)B * p.Hkv;
    if (have_ws) p.row_ticket = (unsigned *)workspace + pairs;
    if (p.limbs && !have_ws) return fail(MYNN_E_ARG, "attention: the limb output needs the attention workspace (%zu bytes)", need);
    if (p.splits <= 1) return MYNN_OK;
    if (!have_ws)
        return fail(MYNN_E_ARG, "attention: workspace of %zu bytes needed, %zu given", need, workspace ? workspace_bytes : (size_t)0);
    char *w = (char *)workspace;
    p.ws_ticket = (unsigned *)w;
    w += align_up((pairs + (size_t)B) * sizeof(unsigned), 256);
    p.ws_ml = (float *)w;
    w += align_up(pairs * kMaxSplits * 8 * 2 * sizeof(float), 256);
    p.ws_o = (float *)w;
    return MYNN_OK;
}

}  // namespace mynn

using namespace mynn;

extern "C" size_t mynn_b200_attention_workspace_bytes(int B, int Hq, int Hkv, int D, int cache_seq_len) {
    if (B <= 0 || Hkv <= 0 || D <= 0) return 0;
    const size_t pairs = (size_t)B * Hkv;
    const size_t tickets = align_up((pairs + (size_t)B) * sizeof(unsigned), 256);  // per (batch, kv head) and per batch row
    const size_t ml = align_up(pairs * kMaxSplits * 8 * 2 * sizeof(float), 256);
    const size_t o = pairs * kMaxSplits * 8 * (size_t)D * sizeof(float);
    (void)Hq;
    (void)cache_seq_len;
    return tickets + ml + o;
}

template <typename T>
static int launch_generic(cudaStream_t st, void *out, const void *q, const void *k, const void *v, float scale, int B,
                          int Hq, int Hkv, int Sq, int Sk, int D, int active, const int32_t *active_dev, int causal,
                          int out_bshd, int ring_sink = 0, int ring_window = 0, int ring_start = 0, const void *mask = nullptr,
                          long long mask_outer_stride = 0, long long mask_row_stride = 0) {
    const long long rows = (long long)B * Hq * Sq;
    const unsigned blocks = (unsigned)((rows * 32 + 127) / 128);
#define GEN(MAXE)                                                                                                     \
    attention_generic_kernel<T, MAXE><<<blocks, 128, 0, st>>>((T *)out, (const T *)q, (const T *)k, (const T *)v, scale, B, \
                                                             Hq, Hkv, Sq, Sk, D, active, active_dev, causal, out_bshd,   \
                                                             ring_sink, ring_window, ring_start, (const T *)mask, mask_outer_stride,   \
                                                             mask_row_stride)
    if (D <= 32) GEN(1);
    else if (D <= 64) GEN(2);
    else if (D <= 128) GEN(4);
    else if (D <= 256) GEN(8);
    else if (D <= 512) GEN(16);
    else return fail(MYNN_E_UNSUPPORTED, "attention: head dim %d > 512", D);
#undef GEN
    MYNN_LAUNCH_OK("attention_generic_kernel");
    return MYNN_OK;
}

// The ring form needs the driver's tensor-map encoder and tensor rows that fit a 32-bit coordinate.
static bool decode_ring_possible(int B, int Hkv, int cache_seq) {
    return g_decode_ring && tensor_map_api_available() && (long long)B * Hkv * cache_seq < (1ll << 31);
}
// resident CTAs per SM of the decode kernel: the ring form at head_dim 128 holds 96 KB of tiles per CTA
static int decode_ctas_per_sm(bool ring, int D) { return ring && D == 128 ? 2 : kAttnCtasPerSm; }

template <typename T, int D>
static int launch_decode(cudaStream_t st, const DecodeParams &p, int B, bool ring) {
    CUtensorMap mk, mv;
    memset(&mk, 0, sizeof mk);
    memset(&mv, 0, sizeof mv);
    if (ring) {
        // the caches as [B * Hkv * cache_seq rows][D * 2 bytes]: boxes of 16 rows x 128 bytes, 128-byte swizzle
        const uint64_t rows = (uint64_t)B * p.Hkv * p.cache_seq, row_bytes = (uint64_t)D * sizeof(T);
        if (int rc = make_map(&mk, p.k, rows, row_bytes, row_bytes, 16)) return rc;
        if (int rc = make_map(&mv, p.v, rows, row_bytes, row_bytes, 16)) return rc;
        constexpr size_t smem = (size_t)kAttnWarps * kRingDepth * 2 * (D / 64) * 16 * 128;
        auto kern = attention_decode_kernel<T, D, true>;
        static bool attr_set = false;
        if (!attr_set) {  // with the kernel's static shared memory every head_dim is past the 48 KB that need no opt-in
            MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            attr_set = true;
        }
        MYNN_CUDA_OK(launch_pdl(kern, dim3(p.splits, p.Hkv, B), dim3(kAttnWarps * 32), smem, st, mk, mv, p));
    } else {
        MYNN_CUDA_OK(launch_pdl(attention_decode_kernel<T, D, false>, dim3(p.splits, p.Hkv, B), dim3(kAttnWarps * 32), 0, st, mk, mv, p));
    }
    MYNN_LAUNCH_OK("attention_decode_kernel");
    return MYNN_OK;
}

// Reads and clears the library's own status word of the ring kernel (the stream must be idle).
int mynn::attention_decode_take_status(int *status) {
    *status = 0;
    MYNN_CUDA_OK(cudaMemcpyFromSymbol(status, g_ring_status, sizeof *status));
    if (*status) {
        const int zero = 0;
        MYNN_CUDA_OK(cudaMemcpyToSymbol(g_ring_status, &zero, sizeof zero));
    }
    return MYNN_OK;
}

extern "C" int mynn_b200_attention_decode_splits(int B, int Hkv, int rows_bound, int ctas_per_sm) {
    if (B < 1 || Hkv < 1 || rows_bound < 0 || ctas_per_sm < 1) return 0;
    return mynn::decode_splits(B, Hkv, rows_bound, 16, ctas_per_sm);
}

extern "C" int mynn_b200_attention(void *stream, void *out, const void *q, const void *k, const void *v, float scale,
                                   int B, int Hq, int Hkv, int Sq, int D, int cache_seq_len, int active_seq_kv,
                                   const int32_t *active_seq_kv_dev, int is_causal, int dtype, void *workspace,
                                   size_t workspace_bytes) {
    return mynn::launch_attention((cudaStream_t)stream, out, q, k, v, scale, B, Hq, Hkv, Sq, D, cache_seq_len,
                                  active_seq_kv, active_seq_kv_dev, is_causal, dtype, workspace, workspace_bytes, 0);
}

// Attention with the operator's additive MASK operand (src/graph/operator.rs:1027): qk = scale * q.k + mask[...] before the
// softmax, on the row-by-row kernel that follows the CPU recurrence (src/codegen/cpu/translator.rs:4854-4881).  The mask is
// addressed as the engine's CUDA launch addresses it (src/codegen/cuda.rs:1297-1325): element
// (b * Hq + h) * mask_outer_stride + sq * mask_row_stride + kv_row, a stride of 0 broadcasting that dimension.
extern "C" int mynn_b200_attention_masked(void *stream, void *out, const void *q, const void *k, const void *v, const void *mask,
                                          long long mask_outer_stride, long long mask_row_stride, float scale, int B, int Hq,
                                          int Hkv, int Sq, int D, int cache_seq_len, int active_seq_kv,
                                          const int32_t *active_seq_kv_dev, int is_causal, int dtype) {
    if (B < 0 || Hq <= 0 || Hkv <= 0 || Sq < 0 || D <= 0 || cache_seq_len < 0 || active_seq_kv < 0 || Hq % Hkv)
        return fail(MYNN_E_ARG, "attention_masked: bad shape");
    if (!dtype_ok(dtype)) return fail(MYNN_E_ARG, "attention_masked: bad dtype %d", dtype);
    if (mask_outer_stride < 0 || mask_row_stride < 0) return fail(MYNN_E_ARG, "attention_masked: negative mask stride");
    if (B == 0 || Sq == 0) return MYNN_OK;
    if (!out || !q || !k || !v || !mask) return fail(MYNN_E_ARG, "attention_masked: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == MYNN_F32) return launch_generic<float>(st, out, q, k, v, scale, B, Hq, Hkv, Sq, cache_seq_len, D, active_seq_kv, active_seq_kv_dev, is_causal, 0, 0, 0, 0, mask, mask_outer_stride, mask_row_stride);
    if (dtype == MYNN_BF16) return launch_generic<__nv_bfloat16>(st, out, q, k, v, scale, B, Hq, Hkv, Sq, cache_seq_len, D, active_seq_kv, active_seq_kv_dev, is_causal, 0, 0, 0, 0, mask, mask_outer_stride, mask_row_stride);
    return launch_generic<__half>(st, out, q, k, v, scale, B, Hq, Hkv, Sq, cache_seq_len, D, active_seq_kv, active_seq_kv_dev, is_causal, 0, 0, 0, 0, mask, mask_outer_stride, mask_row_stride);
}

// Attention over a sink + ring cache.  One query row: the softmax does not depend on the order of the rows, and the
// logical rows 0..active-1 occupy the physical slots 0..active-1 whenever the ring is either not yet wrapped
// (ring_start == 0) or full (active == sink + window), so the tuned decode kernel runs unchanged; every other case
// (several query rows with a causal bound per logical rank, a partly filled wrapped ring) walks the ring in the plain
// kernel.
extern "C" int mynn_b200_attention_ring(void *stream, void *out, const void *q, const void *k, const void *v, float scale,
                                        int B, int Hq, int Hkv, int Sq, int D, int cache_seq_len, int active_seq_kv,
                                        int is_causal, int ring_sink, int ring_window, int ring_start, int dtype,
                                        void *workspace, size_t workspace_bytes) {
    if (ring_sink < 0 || ring_window < 0 || ring_start < 0 || (ring_window > 0 && ring_start >= ring_window) ||
        ring_sink + ring_window > cache_seq_len)
        return fail(MYNN_E_ARG, "attention_ring: bad ring (sink %d, window %d, start %d, cache %d)", ring_sink, ring_window, ring_start, cache_seq_len);
    if (ring_window > 0 && active_seq_kv > ring_sink + ring_window)
        return fail(MYNN_E_ARG, "attention_ring: %d active rows exceed sink + window = %d", active_seq_kv, ring_sink + ring_window);
    const bool identity = ring_window == 0 || ring_start == 0 || active_seq_kv <= ring_sink;
    const bool full = ring_window > 0 && active_seq_kv == ring_sink + ring_window;
    if (Sq == 1 && (identity || full))
        return mynn::launch_attention((cudaStream_t)stream, out, q, k, v, scale, B, Hq, Hkv, Sq, D, cache_seq_len, active_seq_kv,
                                      nullptr, is_causal, dtype, workspace, workspace_bytes, 0);
    if (B < 0 || Hq <= 0 || Hkv <= 0 || Sq < 0 || D <= 0 || cache_seq_len < 0 || active_seq_kv < 0 || Hq % Hkv)
        return fail(MYNN_E_ARG, "attention_ring: bad shape");
    if (!dtype_ok(dtype)) return fail(MYNN_E_ARG, "attention_ring: bad dtype %d", dtype);
    if (B == 0 || Sq == 0) return MYNN_OK;
    if (!out || !q || !k || !v) return fail(MYNN_E_ARG, "attention_ring: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    const int rs = identity ? 0 : ring_sink, rw = identity ? 0 : ring_window, r0 = identity ? 0 : ring_start;
    if (dtype == MYNN_F32) return launch_generic<float>(st, out, q, k, v, scale, B, Hq, Hkv, Sq, cache_seq_len, D, active_seq_kv, nullptr, is_causal, 0, rs, rw, r0);
    if (dtype == MYNN_BF16) return launch_generic<__nv_bfloat16>(st, out, q, k, v, scale, B, Hq, Hkv, Sq, cache_seq_len, D, active_seq_kv, nullptr, is_causal, 0, rs, rw, r0);
    return launch_generic<__half>(st, out, q, k, v, scale, B, Hq, Hkv, Sq, cache_seq_len, D, active_seq_kv, nullptr, is_causal, 0, rs, rw, r0);
}

bool mynn::attention_decode_fast_path(int Sq, int D, int Hq, int Hkv, int dtype, const void *q, const void *k, const void *v) {
    const bool aligned = (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) % 16) == 0;
    return Sq == 1 && (D == 64 || D == 128) && Hkv > 0 && Hq % Hkv == 0 && Hq / Hkv <= 8 && dtype != MYNN_F32 && aligned;
}

int mynn::launch_attention(cudaStream_t st, void *out, const void *q, const void *k, const void *v, float scale, int B,
                           int Hq, int Hkv, int Sq, int D, int cache_seq_len, int active_seq_kv,
                           const int32_t *active_seq_kv_dev, int is_causal, int dtype, void *workspace,
                           size_t workspace_bytes, int out_bshd, int8_t *limbs_out, float *ascale_out, const AttentionFuse *fuse, int *status_word) {
    if (B < 0 || Hq <= 0 || Hkv <= 0 || Sq < 0 || D <= 0 || cache_seq_len < 0 || active_seq_kv < 0)
        return fail(MYNN_E_ARG, "attention: bad shape");
    if (Hq % Hkv != 0) return fail(MYNN_E_ARG, "attention: %d query heads are not a multiple of %d kv heads", Hq, Hkv);
    if (!dtype_ok(dtype)) return fail(MYNN_E_ARG, "attention: bad dtype %d", dtype);
    if (B == 0 || Sq == 0) return MYNN_OK;
    if (!out || !q || !k || !v) return fail(MYNN_E_ARG, "attention: null pointer");
    const int G = Hq / Hkv;
    const bool aligned = (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) % 16) == 0;
    const bool fast = Sq == 1 && (D == 64 || D == 128) && G <= 8 && dtype != MYNN_F32 && aligned;
    if (!fast && (limbs_out || fuse)) return fail(MYNN_E_UNSUPPORTED, "attention: the limb output and the fused RoPE + append exist only on the decode fast path");
    if (!fast) {
        const bool use_tiled = g_prefill_attention_mode >= 0;  // -1: only the row-serial kernel
        if (use_tiled && attention_prefill_tc_supported(B, Hq, Hkv, Sq, D, cache_seq_len, dtype, q, k, v, out))
            return launch_attention_prefill_tc(st, out, q, k, v, scale, B, Hq, Hkv, Sq, D, cache_seq_len, active_seq_kv, active_seq_kv_dev,
                                               is_causal, dtype, out_bshd);
        if (use_tiled && attention_prefill_supported(Sq, D, dtype, q, k, v, out))
            return launch_attention_prefill(st, out, q, k, v, scale, B, Hq, Hkv, Sq, D, cache_seq_len, active_seq_kv, active_seq_kv_dev,
                                            is_causal, dtype, out_bshd);
        if (dtype == MYNN_F32) return launch_generic<float>(st, out, q, k, v, scale, B, Hq, Hkv, Sq, cache_seq_len, D, active_seq_kv, active_seq_kv_dev, is_causal, out_bshd);
        if (dtype == MYNN_BF16) return launch_generic<__nv_bfloat16>(st, out, q, k, v, scale, B, Hq, Hkv, Sq, cache_seq_len, D, active_seq_kv, active_seq_kv_dev, is_causal, out_bshd);
        return launch_generic<__half>(st, out, q, k, v, scale, B, Hq, Hkv, Sq, cache_seq_len, D, active_seq_kv, active_seq_kv_dev, is_causal, out_bshd);
    }
    // decode: is_causal with one query row means bound = min(active, active - 1 + 0 + 1) = active, no extra mask
    DecodeParams p;
    p.out = out;
    p.q = q;
    p.k = k;
    p.v = v;
    p.scale = scale;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.G = G;
    p.cache_seq = cache_seq_len;
    p.active_host = active_seq_kv;
    p.active_dev = active_seq_kv_dev;
    const int rows_bound = active_seq_kv_dev ? cache_seq_len : (active_seq_kv < cache_seq_len ? active_seq_kv : cache_seq_len);
    const bool ring = decode_ring_possible(B, Hkv, cache_seq_len);
    p.splits = decode_splits(B, Hkv, rows_bound, 16, decode_ctas_per_sm(ring, D));
    p.k_scale = nullptr;
    p.v_scale = nullptr;
    p.limbs = limbs_out;
    p.ascale = ascale_out;
    p.status = status_word;
    if (fuse) {
        if (!fuse->k_new || !fuse->v_new || !fuse->cos_t || !fuse->sin_t || !fuse->pos || !fuse->row || fuse->qkv_stride % 8 ||
            (((uintptr_t)fuse->k_new | (uintptr_t)fuse->v_new | (uintptr_t)fuse->cos_t | (uintptr_t)fuse->sin_t) % 16))
            return fail(MYNN_E_ARG, "attention: fused RoPE + append needs 16-byte aligned rows, tables and device scalars");
        p.fused_k = fuse->k_new;
        p.fused_v = fuse->v_new;
        p.qkv_stride = fuse->qkv_stride;
        p.cos_t = fuse->cos_t;
        p.sin_t = fuse->sin_t;
        p.fused_pos = fuse->pos;
        p.fused_row = fuse->row;
    }
    if (int rc = decode_bind_workspace(p, B, D, workspace, workspace_bytes)) return rc;
    if (dtype == MYNN_BF16) return D == 64 ? launch_decode<__nv_bfloat16, 64>(st, p, B, ring) : launch_decode<__nv_bfloat16, 128>(st, p, B, ring);
    return D == 64 ? launch_decode<__half, 64>(st, p, B, ring) : launch_decode<__half, 128>(st, p, B, ring);
}

// ------------------------------------------------------------------------------------------------------------
// Decode attention for callers that have no scratch memory to give and must not allocate.
//
// Who that is: the engine's Attention operator has no workspace operand (its 13 input slots are tensors and scalars,
// src/graph/operator.rs:1024-1042), and its memory planner assigns every device byte to arenas when the model is
// compiled; an operator called from that generated code therefore has neither a buffer to pass for the split-KV
// partial results nor an allocator it may call in the middle of a step.  The same holds for any host that fixes its
// device-memory budget up front.
//
// The partial results live in the fixed array below instead.  It is part of the library image: every GPU that loads
// the library sets aside kStaticScratchBytes for it until the process exits.
//
// Rules that follow from sharing one array:
//   * it keeps whatever the previous call left; the arrival counters, the only part that must start at zero, are
//     cleared on the stream at the beginning of every call;
//   * two calls whose kernels overlap on the GPU (different streams, different threads) race on it: order them;
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress, once per device, with
//     that device current); make that first call before beginning any stream capture;
//   * problems whose partial results exceed the array are refused with MYNN_E_UNSUPPORTED.
namespace mynn {

constexpr size_t kStaticScratchBytes = 4u << 20;  // 4 MiB: a full wave of CTAs (4 per SM) at head_dim 128 needs 2.4 MiB
static __device__ __align__(256) unsigned char g_attn_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static std::atomic<unsigned char *> g_static_scratch_ptr[kMaxDevices];

// In host code `g_attn_static_scratch` names a host-side shadow, not device memory: the device address has to be
// asked for, per device.
static int static_scratch_address(unsigned char **out) {
    int dev = -1;
    MYNN_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(MYNN_E_UNSUPPORTED, "attention_decode_noalloc: device index %d not supported", dev);
    unsigned char *p = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
    if (!p) {
        void *sym = nullptr;
        MYNN_CUDA_OK(cudaGetSymbolAddress(&sym, g_attn_static_scratch));
        if (!sym) return fail(MYNN_E_CUDA, "attention_decode_noalloc: the scratch array has no device address");
        p = static_cast<unsigned char *>(sym);
        g_static_scratch_ptr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return MYNN_OK;
}

}  // namespace mynn

extern "C" size_t mynn_b200_attention_decode_noalloc_max_bytes(void) { return mynn::kStaticScratchBytes; }

extern "C" int mynn_b200_attention_decode_noalloc(void *stream, void *out, const void *q, const void *k, const void *v,
                                                  float scale, int B, int Hq, int Hkv, int D, int cache_seq_len,
                                                  int active_seq_kv, const int32_t *active_seq_kv_dev, int dtype) {
    if (B < 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || cache_seq_len < 0 || active_seq_kv < 0)
        return fail(MYNN_E_ARG, "attention_decode_noalloc: bad shape");
    if (Hq % Hkv != 0) return fail(MYNN_E_ARG, "attention_decode_noalloc: %d query heads are not a multiple of %d kv heads", Hq, Hkv);
    if (B == 0) return MYNN_OK;
    if (!out || !q || !k || !v) return fail(MYNN_E_ARG, "attention_decode_noalloc: null pointer");
    const int G = Hq / Hkv;
    const bool aligned = (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) % 16) == 0;
    if (!((D == 64 || D == 128) && G <= 8 && (dtype == MYNN_BF16 || dtype == MYNN_F16) && aligned))
        return fail(MYNN_E_UNSUPPORTED, "attention_decode_noalloc: needs bf16/f16, head_dim 64 or 128, group size <= 8, 16-byte aligned tensors");
    cudaStream_t st = (cudaStream_t)stream;
    DecodeParams p;
    p.out = out;
    p.q = q;
    p.k = k;
    p.v = v;
    p.scale = scale;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.G = G;
    p.cache_seq = cache_seq_len;
    p.active_host = active_seq_kv;
    p.active_dev = active_seq_kv_dev;
    p.k_scale = nullptr;
    p.v_scale = nullptr;
    const int rows_bound = active_seq_kv_dev ? cache_seq_len : (active_seq_kv < cache_seq_len ? active_seq_kv : cache_seq_len);
    p.splits = decode_splits(B, Hkv, rows_bound);
    p.ws_o = nullptr;
    p.ws_ml = nullptr;
    p.ws_ticket = nullptr;
    p.limbs = nullptr;
    p.ascale = nullptr;
    p.row_ticket = nullptr;
    if (p.splits > 1) {
        const size_t pairs = (size_t)B * Hkv;
        const size_t tickets = align_up(pairs * sizeof(unsigned), 256);
        const size_t ml = align_up(pairs * p.splits * 8 * 2 * sizeof(float), 256);
        const size_t o = pairs * p.splits * 8 * (size_t)D * sizeof(float);
        if (tickets + ml + o > kStaticScratchBytes)
            return fail(MYNN_E_UNSUPPORTED, "attention_decode_noalloc: %zu bytes of partial results exceed the %zu-byte built-in scratch (B=%d, kv heads=%d, %d splits)",
                        tickets + ml + o, kStaticScratchBytes, B, Hkv, p.splits);
        unsigned char *base = nullptr;
        int rc = static_scratch_address(&base);
        if (rc) return rc;
        MYNN_CUDA_OK(cudaMemsetAsync(base, 0, tickets, st));  // arrival counters start from zero on every call
        p.ws_ticket = (unsigned *)base;
        p.ws_ml = (float *)(base + tickets);
        p.ws_o = (float *)(base + tickets + ml);
    }
    if (dtype == MYNN_BF16) return D == 64 ? launch_decode<__nv_bfloat16, 64>(st, p, B, false) : launch_decode<__nv_bfloat16, 128>(st, p, B, false);
    return D == 64 ? launch_decode<__half, 64>(st, p, B, false) : launch_decode<__half, 128>(st, p, B, false);
}
