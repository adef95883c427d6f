// Prefill attention on the 5th-generation tensor cores (tcgen05.mma kind::f16, accumulators in tensor memory).
//
// Both products of a prefill chunk, S = Q K^T and O = P V, are dense 16-bit contractions.  Two kernels: the one used whenever
// the GQA group size is even puts two query heads of one kv head into a CTA (second half of this file); the one described
// first serves the other group sizes.  There one CTA owns 128 query rows of one (batch, query head) pair, i.e. one TMEM lane
// per query row, and walks the kv rows in tiles of 128:
//
//   warp 0     TMA producer: the Q tile once, then K and V tiles through two buffers each (a K buffer is released by the
//              first product, a V buffer by the second), every tile as 64-element (128-byte) slabs with the 128-byte
//              swizzle;
//   warp 1     MMA issuer (one lane) and TMEM owner: S_j = Q K_j^T into one of two 128-column S buffers, so that the
//              product of tile j+1 runs while tile j is in the softmax; then O += P_j V_j into 64/128 further columns.
//              K is a K-major operand (head dim contiguous).  V is used as it lies in the cache, [kv][head dim]: for the
//              second product that is an MN-major B operand, which the matrix descriptor expresses directly;
//   warps 2-9  softmax, two threads per query row (64 kv columns each; the row maximum is exchanged through shared
//              memory): tcgen05.ld of the row of S, causal / length mask, running maximum and sum in f32 in units of
//              log2(e), probabilities rounded to the 16-bit storage type and written to shared memory in the swizzled
//              K-major layout the second product reads (or, as an option, into tensor memory over the S columns, as the
//              two-head kernel always does); finally O / sum -> global memory.
//
// The grid is one-dimensional, query tile slowest and last tile first, so that with a causal mask the longest CTAs of all
// heads are dispatched first.
//
// Rescaling O when the running maximum moves costs a TMEM round trip (tcgen05.ld, multiply, tcgen05.st), so the maximum
// in use is only advanced when the true maximum has moved by more than 8 (a factor 256): probabilities then are at most
// 2^8, which both 16-bit formats and the f32 sums hold without loss, and the final O / sum is unchanged because numerator
// and denominator carry the same factor.
//
// V rows at or past the active length may hold anything (the cache is the caller's memory); their probabilities are 0,
// but 0 x NaN is NaN, so the rows of the last tile that lie past the active length are zeroed in shared memory before the
// second product.
//
// Every mbarrier wait is bounded; on expiry the kernel sets a status word (mynn_b200_attention_check reads it), stops
// issuing work, still frees its tensor memory and returns.
#include <cuda.h>

#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "i8_gemm.cuh"
#include "ops_internal.cuh"
#include "tcgen05.cuh"

namespace mynn {

constexpr int kTcRows = 128;     // query rows per CTA = TMEM lanes
constexpr int kTcCols = 128;     // kv rows per tile
constexpr int kTcThreads = 320;    // TMA warp, MMA warp, 8 softmax warps
constexpr uint32_t kTcSlab = 128 * 128;  // bytes of one slab: 128 rows x 64 16-bit elements
constexpr float kTcMaxSlack = 8.0f;      // log2 units the running maximum may lag behind the true one

__device__ int g_pfa_status;
MYNN_DEFINE_WAIT_BUDGET_SETTER(attention_prefill_tc)

struct TcAttnParams {
    void *out;
    float scale;
    int Hq, Hkv, Sq, cache_seq, active_host;
    const int32_t *active_dev;
    int is_causal, out_bshd;
    uint32_t v_lbo, v_sbo;  // byte offsets of the MN-major V descriptor
    int n_qt, heads_per_grid, B;  // 1-D grid: query tiles x (heads or head pairs) x batch, query tile slowest
    int p_tmem;  // probabilities handed to the second product through tensor memory (over the S columns) instead of shared memory
};

// (x, y) -> two 16-bit values in one register, x in the low half: one cvt instruction
template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float x, float y);
template <>
__device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float x, float y) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
    return reinterpret_cast<const uint32_t &>(v);
}
template <>
__device__ __forceinline__ uint32_t pack_pair<__half>(float x, float y) {
    const __half2 v = __floats2half2_rn(x, y);
    return reinterpret_cast<const uint32_t &>(v);
}
// 2^x on the special-function unit (one instruction; exp2f adds range handling that the softmax does not need)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// One lane polls, the whole warp learns the outcome (tcgen05.ld / st below need the warp to stay converged).
__device__ __forceinline__ bool warp_wait(uint64_t *bar, uint32_t parity, const int *abort_flag) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();  // what lane 0 acquired is ordered before the other lanes' reads
    return ok != 0;
}

__device__ __forceinline__ bool warp_wait_spin(uint64_t *bar, uint32_t parity, const int *abort_flag) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait_spin(bar, parity, abort_flag) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();
    return ok != 0;
}

// One arrival for the whole warp: the lanes' earlier writes are ordered before it by the warp barrier.
__device__ __forceinline__ void warp_arrive(uint64_t *bar) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}

// grid ceil(Sq / 128) x Hq x B (one dimension), block 320
template <typename T, int D>
__global__ void __launch_bounds__(kTcThreads, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const TcAttnParams p) {
    constexpr int SL = D / 64;                      // slabs per tile
    constexpr uint32_t kTile = SL * kTcSlab;        // bytes of a Q, K or V tile
    constexpr uint32_t kPBytes = 2 * kTcSlab;       // P: 128 query rows x 128 kv
    constexpr uint32_t kStage = 2 * kTile;          // K then V
    constexpr uint32_t kColS = 0, kColO = 256;      // TMEM columns: S buffers at 0 and 128, O at 256
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *s_q = smem, *s_p = s_q + kTile, *s_kv = s_p + kPBytes;
    __shared__ uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], s_empty[2], p_full, pv_done, x_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ float sh_max[2][2][kTcRows];  // [tile parity][column half][row]: the halves of a row exchange their maxima

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // 1-D grid with the query tile as the slowest index, last tile first: with a causal mask the work of a CTA grows with its
    // query tile, and CTAs are dispatched in index order, so the longest ones of ALL heads start first
    const int per_qt = p.heads_per_grid * p.B;
    const int qt = p.n_qt - 1 - (int)blockIdx.x / per_qt, h = ((int)blockIdx.x % per_qt) % p.heads_per_grid, b = ((int)blockIdx.x % per_qt) / p.heads_per_grid;
    const int kvh = h / (p.Hq / p.Hkv);
    int active = p.active_dev ? *p.active_dev : p.active_host;
    active = max(0, min(active, p.cache_seq));
    const int q0 = qt * kTcRows;
    const int past = active - p.Sq;
    const int last_row = min(q0 + kTcRows, p.Sq) - 1;
    const int kv_end = p.is_causal ? max(0, min(active, past + last_row + 1)) : active;
    const int n_tiles = (kv_end + kTcCols - 1) / kTcCols;
    const int q_row0 = (b * p.Hq + h) * p.Sq + q0;      // row of the Q map
    const int kv_row0 = (b * p.Hkv + kvh) * p.cache_seq;  // row of the K and V maps

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int s = 0; s < 2; s++) {
            mbar_init(&k_full[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1);
            mbar_init(&s_empty[s], 8);  // one arrival per softmax warp
        }
        mbar_init(&p_full, 8);
        mbar_init(&pv_done, 1);
        mbar_init(&x_bar, 8);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    auto give_up = [&](int code) {
        atomicExch(&abort_flag, 1);
        atomicExch(&g_pfa_status, code);
    };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0 && n_tiles > 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
            mbar_expect_tx(&q_full, kTile);
            for (int sl = 0; sl < SL; sl++) tma_load_2d(s_q + sl * kTcSlab, &map_q, sl * 128, q_row0, &q_full);
            // K of a stage is free again once its S product has completed, V once its O product has: the loads are issued
            // in the order in which the MMA warp releases the buffers (K0, K1, V0, K2, V1, K3, V2, ...)
            auto load_k = [&](int j) {
                const int s = j & 1, u = j >> 1;
                if (u >= 1 && !mbar_wait(&k_empty[s], (u - 1) & 1, &abort_flag)) return false;
                uint8_t *kb = s_kv + s * kStage;
                mbar_expect_tx(&k_full[s], kTile);
                for (int sl = 0; sl < SL; sl++) tma_load_2d(kb + sl * kTcSlab, &map_k, sl * 128, kv_row0 + j * kTcCols, &k_full[s]);
                return true;
            };
            auto load_v = [&](int j) {
                const int s = j & 1, u = j >> 1;
                if (u >= 1 && !mbar_wait(&v_empty[s], (u - 1) & 1, &abort_flag)) return false;
                uint8_t *vb = s_kv + s * kStage + kTile;
                mbar_expect_tx(&v_full[s], kTile);
                for (int sl = 0; sl < SL; sl++) tma_load_2d(vb + sl * kTcSlab, &map_v, sl * 128, kv_row0 + j * kTcCols, &v_full[s]);
                return true;
            };
            bool ok = load_k(0);
            for (int j = 0; j < n_tiles && ok; j++) {
                if (j + 1 < n_tiles) ok = load_k(j + 1);
                ok = ok && load_v(j);
            }
            if (!ok) give_up(1);
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && n_tiles > 0) {
            constexpr uint32_t ab = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;  // operand format: 0 = f16, 1 = bf16
            // D = f32; A and B 16-bit; M = 128.  S: both operands K-major, N = 128.  O: B (= V) MN-major, N = D.
            const uint32_t idesc_s = (1u << 4) | (ab << 7) | (ab << 10) | ((uint32_t)(kTcCols >> 3) << 17) | ((uint32_t)(kTcRows >> 4) << 24);
            const uint32_t idesc_o = (1u << 4) | (ab << 7) | (ab << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(kTcRows >> 4) << 24);
            bool ok = mbar_wait(&q_full, 0, &abort_flag);
            if (!ok) give_up(2);
            auto issue_s = [&](int j) {
                const int s = j & 1, u = j >> 1;
                if (!mbar_wait(&k_full[s], u & 1, &abort_flag) || (u >= 1 && !p.p_tmem && !mbar_wait(&s_empty[s], (u - 1) & 1, &abort_flag))) {
                    give_up(3);
                    return false;
                }
                tc_fence_after();
                const uint32_t qa = smem_u32(s_q), ka = smem_u32(s_kv + s * kStage);
#pragma unroll
                for (int ks = 0; ks < D / 16; ks++) {
                    const uint32_t off = (uint32_t)(ks >> 2) * kTcSlab + (uint32_t)(ks & 3) * 32;
                    umma_f16(tmem_base + kColS + s * 128, make_kmajor_sw128_desc(qa + off), make_kmajor_sw128_desc(ka + off), idesc_s, ks ? 1u : 0u);
                }
                umma_commit(&s_full[s]);
                umma_commit(&k_empty[s]);  // the K buffer may be refilled once these MMAs have read it
                return true;
            };
            ok = ok && issue_s(0);
            for (int j = 0; j < n_tiles && ok; j++) {
                if (j + 1 < n_tiles && !issue_s(j + 1)) break;
                const int s = j & 1, u = j >> 1;
                if (!mbar_wait(&p_full, j & 1, &abort_flag) || !mbar_wait(&v_full[s], u & 1, &abort_flag)) {
                    give_up(4);
                    break;
                }
                tc_fence_after();
                const uint32_t pa = smem_u32(s_p), va = smem_u32(s_kv + s * kStage + kTile);
#pragma unroll
                for (int kk = 0; kk < kTcCols / 16; kk++) {
                    const uint32_t aoff = (uint32_t)(kk >> 2) * kTcSlab + (uint32_t)(kk & 3) * 32;
                    const uint64_t vdesc = make_sw128_desc(va + kk * 16 * 128, p.v_lbo, p.v_sbo);
                    if (p.p_tmem) umma_f16_ta(tmem_base + kColO, tmem_base + kColS + s * 128 + kk * 8, vdesc, idesc_o, (j | kk) ? 1u : 0u);
                    else umma_f16(tmem_base + kColO, make_kmajor_sw128_desc(pa + aoff), vdesc, idesc_o, (j | kk) ? 1u : 0u);
                }
                umma_commit(&v_empty[s]);  // the V buffer may be refilled once these MMAs have read it
                umma_commit(&pv_done);
            }
        }
        __syncwarp();
    } else {
        // ---------------- softmax: two threads per query row (= TMEM lane), 64 kv columns each ----------------
        // warps 2-5 take columns 0-63 of every S tile and the lower half of O, warps 6-9 the rest; a warp reaches the
        // TMEM lanes 32 * (warp % 4) .. + 31, so warps w and w + 4 serve the same rows.
        const int quad = warp & 3, row = quad * 32 + lane, half = (warp - 2) >> 2;
        constexpr int HC = kTcCols / 2;  // S columns per thread
        constexpr int OC = D / 2;        // O columns per thread
        const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
        const int qi = min(q0 + row, p.Sq - 1);  // rows past Sq repeat the last one; they are not stored
        const int bound = p.is_causal ? min(active, past + qi + 1) : active;
        const float sl2 = p.scale * 1.4426950408889634f;
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; j++) {
            const int sb = j & 1, u = j >> 1, kv0 = j * kTcCols, col0 = kv0 + half * HC;
            if (!warp_wait(&s_full[sb], u & 1, &abort_flag)) {
                if (lane == 0) give_up(5);
                ok = false;
                break;
            }
            tc_fence_after();
            float s[HC];
#pragma unroll
            for (int c = 0; c < HC / 32; c++) tmem_ld32(t_lane + kColS + sb * 128 + half * HC + c * 32, reinterpret_cast<uint32_t *>(s) + c * 32);
            tmem_ld_wait();
            tc_fence_before();
            if (!p.p_tmem) warp_arrive(&s_empty[sb]);  // the rows are in registers: the S buffer may take tile j + 2

            if (col0 + HC > bound) {  // only the diagonal and the last tile carry masked columns
#pragma unroll
                for (int i = 0; i < HC; i++)
                    if (col0 + i >= bound) s[i] = -INFINITY;
            }
            float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
            for (int i = 0; i < HC; i += 2) {
                t0 = fmaxf(t0, s[i]);
                t1 = fmaxf(t1, s[i + 1]);
            }
            // the maximum of the row is the larger of the two halves' maxima
            sh_max[sb][half][row] = fmaxf(t0, t1);
            warp_arrive(&x_bar);  // an mbarrier rather than bar.sync: its wait is bounded, so a warp that gave up cannot strand the others
            if (!warp_wait(&x_bar, j & 1, &abort_flag)) {
                if (lane == 0) give_up(9);
                ok = false;
                break;
            }
            const float tmax = fmaxf(sh_max[sb][0][row], sh_max[sb][1][row]) * sl2;  // scale > 0: the maximum commutes with it
            float alpha = 1.f;
            bool moved = false;
            if (tmax > m_used + kTcMaxSlack) {  // also the first visible tile (m_used = -inf)
                alpha = fast_exp2(m_used - tmax);
                m_used = tmax;
                l *= alpha;
                moved = true;
            }
            const float neg_m = m_used == -INFINITY ? 0.f : -m_used;  // nothing visible yet: keep exp2 finite
            uint32_t pk[HC / 2];
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int i = 0; i < HC / 2; i++) {
                const float p0 = fast_exp2(fmaf(s[2 * i], sl2, neg_m)), p1 = fast_exp2(fmaf(s[2 * i + 1], sl2, neg_m));
                sum0 += p0;
                sum1 += p1;
                pk[i] = pack_pair<T>(p0, p1);
            }
            l += sum0 + sum1;

            if (j > 0) {
                // the previous second product has read P and written O
                if (!warp_wait(&pv_done, (j - 1) & 1, &abort_flag)) {
                    if (lane == 0) give_up(6);
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
                    for (int c = 0; c < OC / 32; c++) {
                        uint32_t o[32];
                        tmem_ld32(t_lane + kColO + half * OC + c * 32, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st32(t_lane + kColO + half * OC + c * 32, o);
                    }
                    tmem_st_wait();
                }
            }
            if (kv0 + kTcCols > active) {
                // rows past the active length: zero them in the V tile (the rows are whole, the swizzle does not matter)
                if (!warp_wait(&v_full[sb], u & 1, &abort_flag)) {
                    if (lane == 0) give_up(7);
                    ok = false;
                    break;
                }
                if (kv0 + row >= active) {
                    uint8_t *vb = s_kv + sb * kStage + kTile;
#pragma unroll
                    for (int sl = 0; sl < SL; sl++)
#pragma unroll
                        for (int c = 0; c < 4; c++)
                            *reinterpret_cast<uint4 *>(vb + sl * kTcSlab + row * 128 + (half * 4 + c) * 16) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            // P -> shared memory, K-major with the 128-byte swizzle: this thread's 64 columns are row `row` of slab `half`,
            // and 16-byte chunk c of a row sits at chunk c ^ (row & 7)
            if (p.p_tmem) {
                // P over the first 64 columns of this tile's S buffer, two elements per column; every warp has read its part
                // of S before the maximum exchange above, and the next S product into this buffer is issued after this
                // tile's second product
                tmem_st32(t_lane + kColS + sb * 128 + half * (HC / 2), pk);
                tmem_st_wait();
            } else {
#pragma unroll
                for (int c = 0; c < HC / 8; c++) {
                    uint8_t *dst = s_p + half * kTcSlab + row * 128 + ((c ^ (row & 7)) << 4);
                    *reinterpret_cast<uint4 *>(dst) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
                }
            }
            fence_proxy_async_smem();
            tc_fence_before();
            warp_arrive(&p_full);
        }
        // ---- finish: O / sum -> global memory ----
        if (ok && n_tiles > 0) {
            if (!warp_wait(&pv_done, (n_tiles - 1) & 1, &abort_flag)) {
                if (lane == 0) give_up(8);
                ok = false;
            }
        }
        if (ok && n_tiles > 0) {
            // the two halves of a row have summed disjoint columns under the same maxima
            sh_max[n_tiles & 1][half][row] = l;
            warp_arrive(&x_bar);
            if (!warp_wait(&x_bar, n_tiles & 1, &abort_flag)) {
                if (lane == 0) give_up(10);
                ok = false;
            }
            l = sh_max[n_tiles & 1][0][row] + sh_max[n_tiles & 1][1][row];
        }
        T *out = reinterpret_cast<T *>(p.out);
        const int qrow = q0 + row;
        const size_t orow = p.out_bshd ? ((size_t)b * p.Sq + qrow) * p.Hq + h : ((size_t)(b * p.Hq + h)) * p.Sq + qrow;
        T *orow_p = out + orow * D + half * OC;
        if (n_tiles == 0) {
            if (qrow < p.Sq)
                for (int c = 0; c < OC / 8; c++) *reinterpret_cast<uint4 *>(orow_p + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        } else if (ok) {
            tc_fence_after();
            const float inv = 1.0f / l;
#pragma unroll
            for (int c = 0; c < OC / 32; c++) {
                uint32_t o[32];
                tmem_ld32(t_lane + kColO + half * OC + c * 32, o);
                tmem_ld_wait();
                if (qrow < p.Sq) {
#pragma unroll
                    for (int g = 0; g < 4; g++) {
                        uint4 w;
                        w.x = pack_pair<T>(__uint_as_float(o[8 * g]) * inv, __uint_as_float(o[8 * g + 1]) * inv);
                        w.y = pack_pair<T>(__uint_as_float(o[8 * g + 2]) * inv, __uint_as_float(o[8 * g + 3]) * inv);
                        w.z = pack_pair<T>(__uint_as_float(o[8 * g + 4]) * inv, __uint_as_float(o[8 * g + 5]) * inv);
                        w.w = pack_pair<T>(__uint_as_float(o[8 * g + 6]) * inv, __uint_as_float(o[8 * g + 7]) * inv);
                        *reinterpret_cast<uint4 *>(orow_p + c * 32 + g * 8) = w;
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// -------------------------------------------------------------------------------------------------------------------------
// Two query tiles per CTA ("ping-pong"): the 128 query rows of TWO query heads of the same kv group share one stream of K/V
// tiles.  While the softmax warps of one head work on their S tile, the tensor core runs the products of the other head, so
// neither waits for the other, and every K/V byte that enters shared memory is used twice.  Each softmax thread owns a
// whole row (no exchange between threads).  The probabilities never touch shared memory: they are written over the first
// 64 columns of the head's S tile in tensor memory (two 16-bit values per column) and the second product reads its A
// operand from there, which halves that product's shared-memory traffic; at M = N = 128 with both operands in shared
// memory the tensor core would be bound by the 128 bytes per clock of shared-memory bandwidth.
//
//   TMEM columns   S/P of head 0: [0, 128)   S/P of head 1: [128, 256)   O of head 0: [256, 256 + D)   O of head 1: [384, 384 + D)
//   MMA order      S0(0) S1(0) | P0(0)? -> O0(0) S0(1) | P1(0)? -> O1(0) S1(1) | P0(1)? -> O0(1) S0(2) | ...
// The tensor core executes one thread's MMAs in issue order, so S_t(j+1), issued behind O_t(j), cannot overwrite P_t(j) early,
// and the completion of S_t(j+1) tells the softmax warps that O_t(j) is complete as well (they may rescale O_t).
//
// grid ceil(Sq / 128) x Hq / 2 x B (one dimension), block 320: warp 0 TMA, warp 1 MMA, warps 2-5 softmax of head 0, warps 6-9 of head 1.
template <typename T, int D>
__global__ void __launch_bounds__(kTcThreads, 1)
attention_prefill_tc2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, const TcAttnParams p) {
    constexpr int SL = D / 64;
    constexpr uint32_t kTile = SL * kTcSlab;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *s_q = smem, *s_k = s_q + 2 * kTile, *s_v = s_k + 2 * kTile;  // [Q0][Q1][K0][K1][V0][V1]
    __shared__ uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], p_full[2], o_done[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_qt = p.heads_per_grid * p.B;  // 1-D grid, query tile slowest and last tile first (see the one-head kernel)
    const int qt = p.n_qt - 1 - (int)blockIdx.x / per_qt, h0 = 2 * (((int)blockIdx.x % per_qt) % p.heads_per_grid), b = ((int)blockIdx.x % per_qt) / p.heads_per_grid;
    const int kvh = h0 / (p.Hq / p.Hkv);  // the group size is even: both heads read the same kv head
    int active = p.active_dev ? *p.active_dev : p.active_host;
    active = max(0, min(active, p.cache_seq));
    const int q0 = qt * kTcRows;
    const int past = active - p.Sq;
    const int last_row = min(q0 + kTcRows, p.Sq) - 1;
    const int kv_end = p.is_causal ? max(0, min(active, past + last_row + 1)) : active;
    const int n_tiles = (kv_end + kTcCols - 1) / kTcCols;
    const int kv_row0 = (b * p.Hkv + kvh) * p.cache_seq;

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int s = 0; s < 2; s++) {
            mbar_init(&k_full[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1);
            mbar_init(&p_full[s], 4);  // one arrival per softmax warp of the head
            mbar_init(&o_done[s], 1);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    // the MMA thread and the softmax warps' wait for S sit on the critical path: hardware-suspended waits, no back-off
    auto wait_fast = [&](uint64_t *bar, uint32_t parity) { return mbar_wait_spin(bar, parity, &abort_flag); };
    auto give_up = [&](int code) {
        atomicExch(&abort_flag, 1);
        atomicExch(&g_pfa_status, code);
    };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0 && n_tiles > 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
            mbar_expect_tx(&q_full, 2 * kTile);
            for (int t = 0; t < 2; t++)
                for (int sl = 0; sl < SL; sl++)
                    tma_load_2d(s_q + t * kTile + sl * kTcSlab, &map_q, sl * 128, (b * p.Hq + h0 + t) * p.Sq + q0, &q_full);
            // a K buffer is free once both heads' S products have read it, a V buffer once both O products have; the loads are
            // issued in the order in which the MMA warp releases the buffers (K0, K1, V0, K2, V1, K3, V2, ...)
            auto load = [&](int j, uint8_t *base, const CUtensorMap *map, uint64_t *full, uint64_t *empty) {
                const int s = j & 1, u = j >> 1;
                if (u >= 1 && !mbar_wait(&empty[s], (u - 1) & 1, &abort_flag)) return false;
                mbar_expect_tx(&full[s], kTile);
                for (int sl = 0; sl < SL; sl++) tma_load_2d(base + s * kTile + sl * kTcSlab, map, sl * 128, kv_row0 + j * kTcCols, &full[s]);
                return true;
            };
            bool ok = load(0, s_k, &map_k, k_full, k_empty);
            for (int j = 0; j < n_tiles && ok; j++) {
                if (j + 1 < n_tiles) ok = load(j + 1, s_k, &map_k, k_full, k_empty);
                ok = ok && load(j, s_v, &map_v, v_full, v_empty);
            }
            if (!ok) give_up(11);
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && n_tiles > 0) {
            constexpr uint32_t ab = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            const uint32_t idesc_s = (1u << 4) | (ab << 7) | (ab << 10) | ((uint32_t)(kTcCols >> 3) << 17) | ((uint32_t)(kTcRows >> 4) << 24);
            const uint32_t idesc_o = (1u << 4) | (ab << 7) | (ab << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(kTcRows >> 4) << 24);
            auto issue_s = [&](int t, int j) {  // S_t(j) = Q_t K_j^T; the caller has waited for K_j
                const uint32_t qa = smem_u32(s_q + t * kTile), ka = smem_u32(s_k + (j & 1) * kTile);
#pragma unroll
                for (int ks = 0; ks < D / 16; ks++) {
                    const uint32_t off = (uint32_t)(ks >> 2) * kTcSlab + (uint32_t)(ks & 3) * 32;
                    umma_f16(tmem_base + t * 128, make_kmajor_sw128_desc(qa + off), make_kmajor_sw128_desc(ka + off), idesc_s, ks ? 1u : 0u);
                }
                umma_commit(&s_full[t]);
            };
            bool ok = wait_fast(&q_full, 0) && wait_fast(&k_full[0], 0);
            if (!ok) give_up(12);
            if (ok) {
                tc_fence_after();
                issue_s(0, 0);
                issue_s(1, 0);
                umma_commit(&k_empty[0]);
            }
            for (int j = 0; j < n_tiles && ok; j++) {
                const int st = j & 1, u = j >> 1;
#pragma unroll
                for (int t = 0; t < 2; t++) {
                    if (!wait_fast(&p_full[t], j & 1) || (t == 0 && !wait_fast(&v_full[st], u & 1))) {
                        give_up(13);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t va = smem_u32(s_v + st * kTile);
#pragma unroll
                    for (int kk = 0; kk < kTcCols / 16; kk++)
                        umma_f16_ta(tmem_base + 256 + t * 128, tmem_base + t * 128 + kk * 8, make_sw128_desc(va + kk * 16 * 128, p.v_lbo, p.v_sbo),
                                    idesc_o, (j | kk) ? 1u : 0u);
                    umma_commit(&o_done[t]);
                    if (t == 1) umma_commit(&v_empty[st]);
                    if (j + 1 < n_tiles) {
                        if (t == 0 && !wait_fast(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1)) {
                            give_up(14);
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        issue_s(t, j + 1);
                        if (t == 1) umma_commit(&k_empty[(j + 1) & 1]);
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------- softmax: one thread per query row of its head ----------------
        const int t = (warp - 2) >> 2, quad = warp & 3, row = quad * 32 + lane, h = h0 + t;
        const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
        const uint32_t colS = t * 128, colO = 256 + t * 128;
        const int qi = min(q0 + row, p.Sq - 1);  // rows past Sq repeat the last one; they are not stored
        const int bound = p.is_causal ? min(active, past + qi + 1) : active;
        const float sl2 = p.scale * 1.4426950408889634f;
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; j++) {
            const int kv0 = j * kTcCols;
            if (!warp_wait_spin(&s_full[t], j & 1, &abort_flag)) {
                if (lane == 0) give_up(15);
                ok = false;
                break;
            }
            tc_fence_after();
            float s[kTcCols];
#pragma unroll
            for (int c = 0; c < kTcCols / 32; c++) tmem_ld32(t_lane + colS + c * 32, reinterpret_cast<uint32_t *>(s) + c * 32);
            tmem_ld_wait();
            if (kv0 + kTcCols > bound) {  // only the diagonal and the last tile carry masked columns
#pragma unroll
                for (int i = 0; i < kTcCols; i++)
                    if (kv0 + i >= bound) s[i] = -INFINITY;
            }
            float t0 = -INFINITY, t1 = -INFINITY, t2 = -INFINITY, t3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < kTcCols; i += 4) {
                t0 = fmaxf(t0, s[i]);
                t1 = fmaxf(t1, s[i + 1]);
                t2 = fmaxf(t2, s[i + 2]);
                t3 = fmaxf(t3, s[i + 3]);
            }
            const float tmax = fmaxf(fmaxf(t0, t1), fmaxf(t2, t3)) * sl2;  // scale > 0: the maximum commutes with it
            float alpha = 1.f;
            bool moved = false;
            if (tmax > m_used + kTcMaxSlack) {  // also the first visible tile (m_used = -inf)
                alpha = fast_exp2(m_used - tmax);
                m_used = tmax;
                l *= alpha;
                moved = true;
            }
            if (t == 0 && kv0 + kTcCols > active) {
                // rows past the active length: zero them in the V tile before either head's second product reads it (head 0's is
                // issued first and waits for this warp group)
                if (!warp_wait(&v_full[j & 1], (j >> 1) & 1, &abort_flag)) {
                    if (lane == 0) give_up(16);
                    ok = false;
                    break;
                }
                if (kv0 + row >= active) {
                    uint8_t *vb = s_v + (j & 1) * kTile;
#pragma unroll
                    for (int sl = 0; sl < SL; sl++)
#pragma unroll
                        for (int c = 0; c < 8; c++) *reinterpret_cast<uint4 *>(vb + sl * kTcSlab + row * 128 + c * 16) = make_uint4(0u, 0u, 0u, 0u);
                }
                fence_proxy_async_smem();
            }
            const float neg_m = m_used == -INFINITY ? 0.f : -m_used;  // nothing visible yet: keep exp2 finite
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int c = 0; c < kTcCols / 64; c++) {  // 64 probabilities -> 32 packed columns over the start of the S tile
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    const float x0 = fmaf(s[64 * c + 2 * i], sl2, neg_m), x1 = fmaf(s[64 * c + 2 * i + 1], sl2, neg_m);
                    const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                    sum0 += p0;
                    sum1 += p1;
                    pk[i] = pack_pair<T>(p0, p1);
                }
                tmem_st32(t_lane + colS + c * 32, pk);
            }
            l += sum0 + sum1;
            // S_t(j) complete means O_t(j - 1) is complete too (same issue order): O may be rescaled (after the probabilities,
            // when the registers that held S are free again)
            if (j > 0 && __any_sync(0xffffffffu, moved)) {
#pragma unroll
                for (int c = 0; c < D / 32; c++) {
                    uint32_t o[32];
                    tmem_ld32(t_lane + colO + c * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(t_lane + colO + c * 32, o);
                }
            }
            tmem_st_wait();
            tc_fence_before();
            warp_arrive(&p_full[t]);
        }
        // ---- finish: O / sum -> global memory ----
        if (ok && n_tiles > 0) {
            if (!warp_wait(&o_done[t], (n_tiles - 1) & 1, &abort_flag)) {
                if (lane == 0) give_up(17);
                ok = false;
            }
        }
        T *out = reinterpret_cast<T *>(p.out);
        const int qrow = q0 + row;
        const size_t orow = p.out_bshd ? ((size_t)b * p.Sq + qrow) * p.Hq + h : ((size_t)(b * p.Hq + h)) * p.Sq + qrow;
        if (n_tiles == 0) {
            if (qrow < p.Sq)
                for (int c = 0; c < D / 8; c++) *reinterpret_cast<uint4 *>(out + orow * D + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        } else if (ok) {
            tc_fence_after();
            const float inv = 1.0f / l;
#pragma unroll
            for (int c = 0; c < D / 32; c++) {
                uint32_t o[32];
                tmem_ld32(t_lane + colO + c * 32, o);
                tmem_ld_wait();
                if (qrow < p.Sq) {
#pragma unroll
                    for (int g = 0; g < 4; g++) {
                        uint4 w;
                        w.x = pack_pair<T>(__uint_as_float(o[8 * g]) * inv, __uint_as_float(o[8 * g + 1]) * inv);
                        w.y = pack_pair<T>(__uint_as_float(o[8 * g + 2]) * inv, __uint_as_float(o[8 * g + 3]) * inv);
                        w.z = pack_pair<T>(__uint_as_float(o[8 * g + 4]) * inv, __uint_as_float(o[8 * g + 5]) * inv);
                        w.w = pack_pair<T>(__uint_as_float(o[8 * g + 6]) * inv, __uint_as_float(o[8 * g + 7]) * inv);
                        *reinterpret_cast<uint4 *>(out + orow * D + c * 32 + g * 8) = w;
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// g_prefill_attention_mode (MYNN_OPT_PREFILL_ATTENTION): -1 and 0 keep this file's kernels off; 1 (default): two heads per CTA
// where the group size is even, else one head per CTA; 2: always one head per CTA, P through shared memory; 3: the same with P
// through tensor memory.
bool attention_prefill_tc_supported(int B, int Hq, int Hkv, int Sq, int D, int cache_seq_len, int dtype, const void *q, const void *k,
                                    const void *v, const void *out) {
    if (g_prefill_attention_mode <= 0 || !tensor_map_api_available()) return false;
    const bool aligned = (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) % 16) == 0;
    // at least one full box of rows in every tensor map, and enough query rows for a 128-row tile to pay
    return Sq >= 64 && (D == 64 || D == 128) && (dtype == MYNN_BF16 || dtype == MYNN_F16) && aligned &&
           (long long)B * Hq * Sq >= kTcRows && (long long)B * Hkv * cache_seq_len >= kTcCols &&
           (long long)B * Hq * Sq < (1LL << 31) && (long long)B * Hkv * cache_seq_len < (1LL << 31);
}

template <typename T, int D>
static int launch_tc(cudaStream_t st, const CUtensorMap &mq, const CUtensorMap &mk, const CUtensorMap &mv, const TcAttnParams &p, int B) {
    constexpr size_t smem = (size_t)(D / 64) * kTcSlab * (1 + 4) + 2 * kTcSlab + 1024;  // Q, 2 x (K, V), P, alignment slack
    auto kern = attention_prefill_tc_kernel<T, D>;
    static bool attr_set = false;
    if (!attr_set) {
        MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set = true;
    }
    TcAttnParams q = p;
    q.n_qt = (p.Sq + kTcRows - 1) / kTcRows;
    q.heads_per_grid = p.Hq;
    q.B = B;
    kern<<<dim3((unsigned)((long long)q.n_qt * q.heads_per_grid * B)), kTcThreads, smem, st>>>(mq, mk, mv, q);
    MYNN_LAUNCH_OK("attention_prefill_tc_kernel");
    return MYNN_OK;
}

template <typename T, int D>
static int launch_tc2(cudaStream_t st, const CUtensorMap &mq, const CUtensorMap &mk, const CUtensorMap &mv, const TcAttnParams &p, int B) {
    constexpr size_t smem = (size_t)(D / 64) * kTcSlab * 6 + 1024;  // 2 x Q, 2 x K, 2 x V, alignment slack
    auto kern = attention_prefill_tc2_kernel<T, D>;
    static bool attr_set = false;
    if (!attr_set) {
        MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set = true;
    }
    TcAttnParams q = p;
    q.n_qt = (p.Sq + kTcRows - 1) / kTcRows;
    q.heads_per_grid = p.Hq / 2;
    q.B = B;
    kern<<<dim3((unsigned)((long long)q.n_qt * q.heads_per_grid * B)), kTcThreads, smem, st>>>(mq, mk, mv, q);
    MYNN_LAUNCH_OK("attention_prefill_tc2_kernel");
    return MYNN_OK;
}

int launch_attention_prefill_tc(cudaStream_t st, void *out, const void *q, const void *k, const void *v, float scale, int B, int Hq,
                                int Hkv, int Sq, int D, int cache_seq_len, int active_seq_kv, const int32_t *active_seq_kv_dev,
                                int is_causal, int dtype, int out_bshd) {
    TcAttnParams p;
    p.out = out;
    p.scale = scale;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.Sq = Sq;
    p.cache_seq = cache_seq_len;
    p.active_host = active_seq_kv;
    p.active_dev = active_seq_kv_dev;
    p.is_causal = is_causal;
    p.out_bshd = out_bshd;
    // V tile in shared memory: D / 64 slabs of [128 kv rows][64 head-dim elements]: the next 64 head-dim elements are one
    // slab further (leading offset), the next 8 kv rows 8 x 128 bytes further (stride offset)
    p.v_lbo = kTcSlab;
    p.v_sbo = 1024;
    p.p_tmem = g_prefill_attention_mode == 3;
    // the maps describe the tensors as bytes: rows of D * 2 bytes, boxes of 128 bytes x 128 rows
    CUtensorMap mq, mk, mv;
    const uint64_t row_bytes = (uint64_t)D * 2;
    if (int rc = make_map(&mq, q, (uint64_t)B * Hq * Sq, row_bytes, row_bytes, kTcRows)) return rc;
    if (int rc = make_map(&mk, k, (uint64_t)B * Hkv * cache_seq_len, row_bytes, row_bytes, kTcCols)) return rc;
    if (int rc = make_map(&mv, v, (uint64_t)B * Hkv * cache_seq_len, row_bytes, row_bytes, kTcCols)) return rc;
    // an even group size can put two query heads of one kv head into every CTA (mode 4)
    if ((Hq / Hkv) % 2 == 0 && g_prefill_attention_mode == 1) {
        if (dtype == MYNN_BF16) return D == 64 ? launch_tc2<__nv_bfloat16, 64>(st, mq, mk, mv, p, B) : launch_tc2<__nv_bfloat16, 128>(st, mq, mk, mv, p, B);
        return D == 64 ? launch_tc2<__half, 64>(st, mq, mk, mv, p, B) : launch_tc2<__half, 128>(st, mq, mk, mv, p, B);
    }
    if (dtype == MYNN_BF16) return D == 64 ? launch_tc<__nv_bfloat16, 64>(st, mq, mk, mv, p, B) : launch_tc<__nv_bfloat16, 128>(st, mq, mk, mv, p, B);
    return D == 64 ? launch_tc<__half, 64>(st, mq, mk, mv, p, B) : launch_tc<__half, 128>(st, mq, mk, mv, p, B);
}

// Reads and clears the status word of the tensor-core prefill kernels (the stream must be idle).
int attention_prefill_tc_take_status(int *status) {
    *status = 0;
    MYNN_CUDA_OK(cudaMemcpyFromSymbol(status, g_pfa_status, sizeof *status));
    if (*status) {
        const int zero = 0;
        MYNN_CUDA_OK(cudaMemcpyToSymbol(g_pfa_status, &zero, sizeof zero));
    }
    return MYNN_OK;
}

}  // namespace mynn

using namespace mynn;

// Synchronises the stream and reports (once) whether a bounded wait inside the tensor-core prefill attention kernel ran out.
extern "C" int mynn_b200_attention_check(void *stream) {
    MYNN_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
    int status = 0;
    if (int rc = attention_prefill_tc_take_status(&status)) return rc;
    if (status) return fail(MYNN_E_CUDA, "attention: pipeline wait %d timed out inside the tcgen05 prefill kernel", status);
    if (int rc = attention_decode_take_status(&status)) return rc;
    if (status) return fail(MYNN_E_CUDA, "attention: wait %d for a K/V tile timed out inside the decode kernel", status);
    if (int rc = attention_decode_q8_take_status(&status)) return rc;
    if (status) return fail(MYNN_E_CUDA, "attention: wait %d for a K/V tile timed out inside the int8-cache decode kernel", status);
    return MYNN_OK;
}
