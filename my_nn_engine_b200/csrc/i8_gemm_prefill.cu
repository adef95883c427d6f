// Prefill DequantMatMul (many activation rows) on tcgen05 kind::i8:  out[m,n] = scale[n] * sum_k act[m,k] * wq[n,k].
//
// This is a dense contraction, judged by tensor-pipe utilisation.  Like the decode kernel it never converts a weight:
// the activations are rewritten once as fixed point with a per-row power-of-two scale and split into TWO signed
// int8 limbs (15 significant bits relative to the row maximum: every bf16 element within 2^-7 of its row maximum is
// exact, the rest carry an absolute error below 2^-15 of the maximum -- finer than the bf16 rounding of the
// dequantised weights in the engine's own tensor-core prefill kernel).  The product is then an int8 GEMM with exact
// int32 accumulation, [N weight rows] x [2 x tokens] x K, and the int8 pipe runs at twice the bf16 rate, so two limbs
// cost the same tensor time as one bf16 product.
//
// Kernel: persistent CTAs (one per SM), tile = 128 weight rows x 128 tokens (256 limb columns), UMMA M=128 N=256 K=32;
// warp 0 streams weight and limb tiles by TMA through a 4-stage mbarrier ring (48 KB per stage), warp 1 issues the
// MMAs into one of two 256-column TMEM accumulators, warps 2-5 drain the other accumulator (tcgen05.ld), recombine
// the limbs, scale, add the optional residual and store -- so the epilogue of one tile overlaps the main loop of the
// next.  Tiles are walked with the token tile fastest, so concurrently running CTAs share weight tiles in L2.
// All waits are bounded and report through the workspace status word.
#include "common.cuh"
#include "i8_gemm.cuh"
#include "tcgen05.cuh"

namespace mynn {

MYNN_DEFINE_WAIT_BUDGET_SETTER(i8_gemm_prefill)

constexpr int kPfRows = 128;      // weight rows per tile (UMMA M)
constexpr int kPfCols = 256;      // accumulator columns per tile (UMMA N): LIMBS columns per activation row
constexpr int kPfTokens = kPfCols / 2;  // activation rows per tile with two limbs (DequantMatMul)
constexpr int kPfBlockK = 128;
constexpr int kPfStages = 4;
constexpr int kPfThreads = 192;
constexpr uint32_t kPfWBytes = kPfRows * kPfBlockK, kPfABytes = kPfCols * kPfBlockK;
constexpr uint32_t kPfStageBytes = kPfWBytes + kPfABytes;  // 48 KB

// ---- pre-pass: rows -> two int8 limbs + power-of-two row scale ----------------------------------------------------
// limbs [(2m + l)][K]; with max |row| < 2^e the row is scaled by 2^(14-e), so |A| <= 2^14 and the high limb is within
// [-64, 64]; ascale[m] = 2^(e-14).
// One CTA of 256 threads per row (several rows are resident per SM, which hides the two block-wide reductions); VEC: 16-bit
// activations read 8 at a time (rows 16-byte aligned); the limbs are always written 8 bytes at a time (K is a multiple of 16).
constexpr int kLimbThreads = 256;
template <typename T, bool VEC>
__global__ void __launch_bounds__(kLimbThreads) act_to_limbs2_kernel(int8_t *limbs, float *ascale, const T *act, int K) {
    extern __shared__ __align__(16) float row_s[];
    __shared__ float red[kLimbThreads / 32 + 1];
    pdl_trigger();
    pdl_wait();
    const int m = blockIdx.x;
    const T *src = act + (size_t)m * K;
    float mx = 0.f;
    bool bad = false;
    if constexpr (VEC) {
        for (int i = 8 * threadIdx.x; i < K; i += 8 * kLimbThreads) {
            T av[8];
            *reinterpret_cast<uint4 *>(av) = *reinterpret_cast<const uint4 *>(src + i);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float v = to_f32<T>(av[j]);
                row_s[i + j] = v;
                bad |= !(fabsf(v) <= 3.0e38f);
                mx = fmaxf(mx, fabsf(v));
            }
        }
    } else {
        for (int i = threadIdx.x; i < K; i += kLimbThreads) {
            const float v = to_f32<T>(src[i]);
            row_s[i] = v;
            bad |= !(fabsf(v) <= 3.0e38f);
            mx = fmaxf(mx, fabsf(v));
        }
    }
    mx = warp_max(mx);
    const unsigned anybad = __syncthreads_or(bad);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < kLimbThreads / 32; i++) t = fmaxf(t, red[i]);
        int e = 0;
        if (t > 0.f) frexpf(t, &e);
        const float sc = t > 0.f ? ldexpf(1.0f, 14 - e) : 1.0f;
        red[kLimbThreads / 32] = anybad ? 0.f : sc;
        ascale[m] = anybad ? __int_as_float(0x7fc00000) : 1.0f / sc;
    }
    __syncthreads();
    const float sc = red[kLimbThreads / 32];
    uint2 *l0 = reinterpret_cast<uint2 *>(limbs + (size_t)(2 * m) * K);
    uint2 *l1 = reinterpret_cast<uint2 *>(limbs + (size_t)(2 * m + 1) * K);
    for (int gi = threadIdx.x; gi < (K >> 3); gi += kLimbThreads) {
        uint32_t w0[2] = {0u, 0u}, w1[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 8; i++) {
            int A = sc == 0.f ? 0 : __float2int_rn(row_s[8 * gi + i] * sc);
            const int d0 = (int)(int8_t)(A & 0xFF);
            A = (A - d0) >> 8;
            w0[i >> 2] |= (uint32_t)(d0 & 0xFF) << (8 * (i & 3));
            w1[i >> 2] |= (uint32_t)(A & 0xFF) << (8 * (i & 3));
        }
        l0[gi] = make_uint2(w0[0], w0[1]);
        l1[gi] = make_uint2(w1[0], w1[1]);
    }
}

// ---- fused producers: the operator that makes a DequantMatMul's activations writes the two limbs itself -------------------
// (the prefill counterpart of rms_norm_limbs_kernel / swiglu_limbs_kernel of the decode step: no activation tensor is written
// and read back, and no separate pre-pass runs).  One CTA of 256 threads per row; D, F multiples of 8, rows 16-byte aligned.
__device__ __forceinline__ float limb2_scale(float mx, bool bad, float *ascale_m, float *red /* kLimbThreads / 32 + 1 floats */) {
    mx = warp_max(mx);
    const unsigned anybad = __syncthreads_or(bad);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < kLimbThreads / 32; i++) t = fmaxf(t, red[i]);
        int e = 0;
        if (t > 0.f) frexpf(t, &e);
        const float sc = t > 0.f ? ldexpf(1.0f, 14 - e) : 1.0f;
        red[kLimbThreads / 32] = anybad ? 0.f : sc;
        *ascale_m = anybad ? __int_as_float(0x7fc00000) : 1.0f / sc;
    }
    __syncthreads();
    return red[kLimbThreads / 32];
}
// row_s holds the row in the storage type T (the values are already rounded to T, so nothing is lost and twice as many
// rows fit per SM as with f32)
template <typename T>
__device__ __forceinline__ void smem_row_to_limbs2(const T *row_s, int K, int8_t *limb_row0, float sc) {
    uint2 *l0 = reinterpret_cast<uint2 *>(limb_row0);
    uint2 *l1 = reinterpret_cast<uint2 *>(limb_row0 + K);
    for (int gi = threadIdx.x; gi < (K >> 3); gi += kLimbThreads) {
        T x[8];
        *reinterpret_cast<uint4 *>(x) = reinterpret_cast<const uint4 *>(row_s)[gi];
        uint32_t w0[2] = {0u, 0u}, w1[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 8; i++) {
            int A = sc == 0.f ? 0 : __float2int_rn(to_f32<T>(x[i]) * sc);
            const int d0 = (int)(int8_t)(A & 0xFF);
            A = (A - d0) >> 8;
            w0[i >> 2] |= (uint32_t)(d0 & 0xFF) << (8 * (i & 3));
            w1[i >> 2] |= (uint32_t)(A & 0xFF) << (8 * (i & 3));
        }
        l0[gi] = make_uint2(w0[0], w0[1]);
        l1[gi] = make_uint2(w1[0], w1[1]);
    }
}
template <typename T>
__device__ __forceinline__ void ld8(const T *p, float (&v)[8]) {
    T raw[8];
    *reinterpret_cast<uint4 *>(raw) = *reinterpret_cast<const uint4 *>(p);
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = to_f32<T>(raw[i]);
}
template <typename T>
__device__ __forceinline__ void st8(T *p, const float (&v)[8]) {
    T raw[8];
#pragma unroll
    for (int i = 0; i < 8; i++) raw[i] = from_f32<T>(v[i]);
    *reinterpret_cast<uint4 *>(p) = *reinterpret_cast<const uint4 *>(raw);
}

// y = round(x * rsqrt(mean x^2 + eps) * w) -> two limbs per element
template <typename T>
__global__ void __launch_bounds__(kLimbThreads)
rms_norm_limbs2_kernel(int8_t *limbs, float *ascale, const T *x, const T *w, float eps, int D) {
    extern __shared__ __align__(16) uint8_t row_raw[];
    T *row_s = reinterpret_cast<T *>(row_raw);
    __shared__ float red[kLimbThreads / 32 + 2];
    pdl_trigger();
    pdl_wait();
    const int m = blockIdx.x;
    const size_t base = (size_t)m * D;
    float ss = 0.f;
    for (int i = 8 * threadIdx.x; i < D; i += 8 * kLimbThreads) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(x + base + i);
        *reinterpret_cast<uint4 *>(row_s + i) = raw;
        const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float v = to_f32<T>(e[j]);
            ss += v * v;
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int i = 0; i < kLimbThreads / 32; i++) tot += red[i];
        red[kLimbThreads / 32 + 1] = 1.0f / sqrtf(tot / (float)D + eps);
    }
    __syncthreads();
    const float inv = red[kLimbThreads / 32 + 1];
    float mx = 0.f;
    bool bad = false;
    for (int i = 8 * threadIdx.x; i < D; i += 8 * kLimbThreads) {  // each thread revisits the elements it wrote
        float xv[8], wv[8], y[8];
        ld8<T>(row_s + i, xv);
        ld8<T>(w + i, wv);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            y[j] = round_store<T>(xv[j] * inv * wv[j]);
            bad |= !(fabsf(y[j]) <= 3.0e38f);
            mx = fmaxf(mx, fabsf(y[j]));
        }
        st8<T>(row_s + i, y);
    }
    const float sc = limb2_scale(mx, bad, ascale + m, red);  // its barriers also publish row_s
    smem_row_to_limbs2<T>(row_s, D, limbs + (size_t)(2 * m) * D, sc);
}

// h = round(swish(gate) * up) -> two limbs per element; gate / up rows are in_stride elements apart
template <typename T>
__global__ void __launch_bounds__(kLimbThreads)
swiglu_limbs2_kernel(int8_t *limbs, float *ascale, const T *gate, const T *up, int F, long long in_stride) {
    extern __shared__ __align__(16) uint8_t row_raw[];
    T *row_s = reinterpret_cast<T *>(row_raw);
    __shared__ float red[kLimbThreads / 32 + 2];
    pdl_trigger();
    pdl_wait();
    const int m = blockIdx.x;
    float mx = 0.f;
    bool bad = false;
    for (int i = 8 * threadIdx.x; i < F; i += 8 * kLimbThreads) {
        float g[8], u[8], h[8];
        ld8<T>(gate + (size_t)m * in_stride + i, g);
        ld8<T>(up + (size_t)m * in_stride + i, u);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            h[j] = round_store<T>((g[j] / (1.0f + expf(-g[j]))) * u[j]);
            bad |= !(fabsf(h[j]) <= 3.0e38f);
            mx = fmaxf(mx, fabsf(h[j]));
        }
        st8<T>(row_s + i, h);
    }
    const float sc = limb2_scale(mx, bad, ascale + m, red);
    smem_row_to_limbs2<T>(row_s, F, limbs + (size_t)(2 * m) * F, sc);
}

struct PfParams {
    void *out;
    const void *scale, *resid;
    const float *ascale;    // f32 row scales (DequantMatMul pre-pass), or null when ascale_t is used
    const void *ascale_t;   // QuantizedMatMul: lhs scales in the output dtype, element m * ascale_stride
    int ascale_stride;      // 1 = one scale per row, 0 = one scale for the whole tensor
    int M, N, K;
    int w_tiles, t_tiles;
    int *status;
};

// grid = min(#SMs, #tiles) persistent CTAs; tile index = w_tile * t_tiles + t_tile, walked with stride gridDim.x.
// LIMBS = 2: DequantMatMul, limb rows (2m + l), 128 activation rows per tile.
// LIMBS = 1: QuantizedMatMul (W8A8), the int8 lhs matrix itself is the operand, 256 activation rows per tile.
template <typename OutT, int LIMBS>
__global__ void __launch_bounds__(kPfThreads, 1)
i8_prefill_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, const PfParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[kPfStages], empty_bar[kPfStages], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    constexpr int kTok = kPfCols / LIMBS;  // activation rows per tile
    __shared__ float sh_ascale[2][kTok];
    __shared__ int sh_go[2];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = p.w_tiles * p.t_tiles;
    const int kblocks = (p.K + kPfBlockK - 1) / kPfBlockK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPfStages; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);  // one arrival per epilogue warp
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    pdl_wait();  // limbs and row scales come from the pre-pass

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
            int kc = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int wt = tile / p.t_tiles, tt = tile - wt * p.t_tiles;
                for (int kb = 0; kb < kblocks; kb++, kc++) {
                    const int s = kc % kPfStages, use = kc / kPfStages;
                    if (use > 0 && !mbar_wait_spin(&empty_bar[s], (use - 1) & 1, &abort_flag)) {
                        atomicExch(&abort_flag, 1);
                        atomicExch(p.status, 11);
                        ok = false;
                        break;
                    }
                    uint8_t *st = smem + s * kPfStageBytes;
                    mbar_expect_tx(&full_bar[s], kPfStageBytes);
                    tma_load_2d(st, &map_w, kb * kPfBlockK, wt * kPfRows, &full_bar[s]);
                    tma_load_2d(st + kPfWBytes, &map_a, kb * kPfBlockK, tt * kPfCols, &full_bar[s]);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int kc = 0, it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, it++) {
                const int buf = it & 1, use = it >> 1;
                // N of the MMA = the accumulator columns this tile really has (rows past M are zero-filled by TMA and
                // need no tensor time), rounded up to the instruction's granularity of 16
                const int tt_ = tile % p.t_tiles;
                const int cols = min(kPfCols, (((p.M - tt_ * kTok) * LIMBS + 15) >> 4) << 4);
                const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(cols >> 3) << 17) | ((uint32_t)(kPfRows >> 4) << 24);
                if (use > 0 && !mbar_wait_spin(&acc_empty[buf], (use - 1) & 1, &abort_flag)) {  // epilogue has drained it
                    atomicExch(&abort_flag, 1);
                    atomicExch(p.status, 12);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * kPfCols);
                for (int kb = 0; kb < kblocks; kb++, kc++) {
                    const int s = kc % kPfStages;
                    if (!mbar_wait_spin(&full_bar[s], (kc / kPfStages) & 1, &abort_flag)) {
                        atomicExch(&abort_flag, 1);
                        atomicExch(p.status, 13);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + s * kPfStageBytes);
                    const uint64_t adesc = make_kmajor_sw128_desc(a_addr), bdesc = make_kmajor_sw128_desc(a_addr + kPfWBytes);
#pragma unroll
                    for (int k = 0; k < kPfBlockK / 32; k++)
                        umma_i8(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (kb | k) ? 1u : 0u);
                    umma_commit(&empty_bar[s]);
                }
                if (ok) umma_commit(&acc_full[buf]);
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue warps 2..5: TMEM lane quadrant = warp & 3, one weight row per thread ----------------
        const int quad = warp & 3, r_local = quad * 32 + lane, et = threadIdx.x - 64;
        const OutT *scale_p = reinterpret_cast<const OutT *>(p.scale);
        const OutT *resid_p = reinterpret_cast<const OutT *>(p.resid);
        OutT *out_p = reinterpret_cast<OutT *>(p.out);
        int it = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, it++) {
            const int wt = tile / p.t_tiles, tt = tile - wt * p.t_tiles;
            const int buf = it & 1, use = it >> 1;
            const int n = wt * kPfRows + r_local, tok0 = tt * kTok;
            const float wscale = n < p.N ? to_f32<OutT>(scale_p[n]) : 0.f;
            for (int i = et; i < kTok; i += 128) {
                float a = 0.f;
                if (tok0 + i < p.M)
                    a = p.ascale ? p.ascale[tok0 + i]
                                 : to_f32<OutT>(reinterpret_cast<const OutT *>(p.ascale_t)[(size_t)(tok0 + i) * p.ascale_stride]);
                sh_ascale[buf][i] = a;
            }
            // one thread waits for the accumulator and publishes the outcome, so that all four warps take the same
            // branch (a warp leaving alone would strand the others at the named barrier)
            if (et == 0) {
                const bool ok = mbar_wait_spin(&acc_full[buf], use & 1, &abort_flag);
                if (!ok) {
                    atomicExch(&abort_flag, 1);
                    atomicExch(p.status, 14);
                }
                sh_go[buf] = ok ? 1 : 0;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps: sh_ascale[buf], sh_go[buf] are set
            if (!sh_go[buf]) break;
            tc_fence_after();
            // 32 accumulator columns = R activation rows per chunk.  `out` may alias `resid` (x += ...), so a residual load written
            // next to its store could not be moved ahead of the previous store and every row would pay a global-memory round
            // trip: the residuals of a chunk are loaded together, two chunks ahead of their use (buffers ra / rb).
            constexpr int R = 32 / LIMBS;
            auto load_res = [&](int c0, float (&dst)[R]) {
                if (resid_p && n < p.N && c0 < kPfCols) {
#pragma unroll
                    for (int j = 0; j < R; j++) {
                        const int m = tok0 + c0 / LIMBS + j;
                        dst[j] = m < p.M ? to_f32<OutT>(resid_p[(size_t)m * p.N + n]) : 0.f;
                    }
                }
            };
            auto process = [&](int c0, const float (&res)[R]) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * kPfCols + c0), v);
                tmem_ld_wait();
                if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < R; j++) {
                        const int m = tok0 + c0 / LIMBS + j;
                        if (m < p.M) {
                            float acc;
                            if constexpr (LIMBS == 2) acc = (float)((long long)(int)v[2 * j + 1] * 256 + (long long)(int)v[2 * j]);
                            else acc = (float)(int)v[j];
                            // (acc * lhs scale) * weight scale with separate roundings, as the CPU kernels compute it
                            float r = __fmul_rn(__fmul_rn(acc, sh_ascale[buf][c0 / LIMBS + j]), wscale);
                            if (resid_p) r = __fadd_rn(round_store<OutT>(r), res[j]);
                            out_p[(size_t)m * p.N + n] = from_f32<OutT>(r);
                        }
                    }
                }
            };
            float ra[R], rb[R];
            load_res(0, ra);
            load_res(32, rb);
#pragma unroll 1
            for (int c0 = 0; c0 < kPfCols; c0 += 64) {
                if (tok0 + c0 / LIMBS >= p.M) break;  // uniform: the remaining columns belong to rows past M
                process(c0, ra);
                load_res(c0 + 64, ra);
                if (tok0 + (c0 + 32) / LIMBS >= p.M) break;
                process(c0 + 32, rb);
                load_res(c0 + 96, rb);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);  // this warp has drained its quadrant of the accumulator
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ---- host side ---------------------------------------------------------------------------------------------------
static size_t pf_scale_bytes(int M) { return ((size_t)M * sizeof(float) + 255) / 256 * 256; }

size_t i8_prefill_workspace_bytes(int M, int K) {
    if (M <= 0 || K <= 0) return 0;
    return 256 + pf_scale_bytes(M) + ((size_t)2 * M * K + 255) / 256 * 256;
}

bool i8_prefill_supported(int M, int N, int K, const void *wq, int act_dtype, int out_dtype) {
    (void)out_dtype;
    // two limbs carry 15 bits: right for 16-bit activations, not for f32 graphs (those keep the f32-accurate kernels)
    return act_dtype != MYNN_F32 && M > kI8MaxRows && N >= 1 && K >= 16 && K % 16 == 0 && (size_t)K * 4 <= 200 * 1024 && ((uintptr_t)wq % 16) == 0 &&
           tensor_map_api_available();
}

template <typename OutT, int LIMBS>
static int launch_pf(cudaStream_t st, const CUtensorMap &mw, const CUtensorMap &ma, const PfParams &p) {
    const size_t smem = (size_t)kPfStages * kPfStageBytes + 1024;
    auto kern = i8_prefill_gemm_kernel<OutT, LIMBS>;
    static bool attr_set = false;
    if (!attr_set) {
        MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set = true;
    }
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int tiles = p.w_tiles * p.t_tiles;
    MYNN_CUDA_OK(launch_pdl(kern, dim3(tiles < sms ? tiles : sms), dim3(kPfThreads), smem, st, mw, ma, p));
    MYNN_LAUNCH_OK("i8_prefill_gemm_kernel");
    return MYNN_OK;
}

int i8_prefill_launch(cudaStream_t st, void *out, const void *act, const int8_t *wq, const void *scale, const void *resid,
                      int M, int N, int K, int act_dtype, int out_dtype, void *workspace, size_t workspace_bytes) {
    const size_t need = i8_prefill_workspace_bytes(M, K);
    if (!workspace || workspace_bytes < need)
        return fail(MYNN_E_ARG, "dequant_matmul: workspace of %zu bytes needed, %zu given", need, workspace ? workspace_bytes : (size_t)0);
    if ((uintptr_t)workspace % 256) return fail(MYNN_E_ARG, "dequant_matmul: workspace must be 256-byte aligned");
    int *status = (int *)workspace;
    float *ascale = (float *)((char *)workspace + 256);
    int8_t *limbs = (int8_t *)workspace + 256 + pf_scale_bytes(M);
    const size_t smem = (size_t)K * 4;
    if (act != nullptr) {  // act == nullptr: a fused producer has left limbs and row scales in the workspace
    const bool vec = act_dtype != MYNN_F32 && K % 8 == 0 && ((uintptr_t)act % 16) == 0;
#define PREP(T)                                                                                                          \
    {                                                                                                                    \
        auto kern = vec ? act_to_limbs2_kernel<T, sizeof(T) == 2> : act_to_limbs2_kernel<T, false>;                      \
        if (smem > 48 * 1024) MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        MYNN_CUDA_OK(launch_pdl(kern, dim3(M), dim3(kLimbThreads), smem, st, limbs, ascale, (const T *)act, K));         \
    }
    switch (act_dtype) {
        case MYNN_BF16: PREP(__nv_bfloat16) break;
        case MYNN_F16: PREP(__half) break;
        case MYNN_F32: PREP(float) break;
        default: return fail(MYNN_E_ARG, "dequant_matmul: bad activation dtype %d", act_dtype);
    }
#undef PREP
    MYNN_LAUNCH_OK("act_to_limbs2_kernel");
    }
    CUtensorMap mw, ma;
    int rc = make_map(&mw, wq, (uint64_t)N, (uint64_t)K, (uint64_t)K, kPfRows);
    if (rc) return rc;
    rc = make_map(&ma, limbs, (uint64_t)2 * M, (uint64_t)K, (uint64_t)K, (uint32_t)kPfCols);
    if (rc) return rc;
    PfParams p;
    p.out = out;
    p.scale = scale;
    p.resid = resid;
    p.ascale = ascale;
    p.ascale_t = nullptr;
    p.ascale_stride = 1;
    p.M = M;
    p.N = N;
    p.K = K;
    p.w_tiles = (N + kPfRows - 1) / kPfRows;
    p.t_tiles = (M + kPfTokens - 1) / kPfTokens;
    p.status = status;
    if (out_dtype == MYNN_BF16) return launch_pf<__nv_bfloat16, 2>(st, mw, ma, p);
    if (out_dtype == MYNN_F16) return launch_pf<__half, 2>(st, mw, ma, p);
    return launch_pf<float, 2>(st, mw, ma, p);
}

// QuantizedMatMul (W8A8): out[m,n] = (sum_k lhs[m,k] * rhs[n,k]) * lhs_scale[m] * rhs_scale[n].  The int8 lhs matrix is
// the TMA source as it is (no pre-pass, one accumulator column per row), so the int8 pipe does a quarter of the work
// per output that a bf16 product would need.  workspace: 256 bytes (status word), zeroed once.
// Fused producers of the prefill DequantMatMul (rows > 32): limbs and row scales go to the layout i8_prefill_launch reads.
static int pf_fused_ws(void *workspace, size_t workspace_bytes, int rows, int K, int8_t **limbs, float **ascale) {
    const size_t need = i8_prefill_workspace_bytes(rows, K);
    if (!workspace || workspace_bytes < need)
        return fail(MYNN_E_ARG, "fused limb producer: workspace of %zu bytes needed, %zu given", need, workspace ? workspace_bytes : (size_t)0);
    if ((uintptr_t)workspace % 256) return fail(MYNN_E_ARG, "fused limb producer: workspace must be 256-byte aligned");
    *ascale = (float *)((char *)workspace + 256);
    *limbs = (int8_t *)workspace + 256 + pf_scale_bytes(rows);
    return MYNN_OK;
}

bool prefill_fused_supported(int dtype, int K, const void *a, const void *b) {
    return dtype != MYNN_F32 && K % 16 == 0 && (size_t)K * 4 <= 200 * 1024 && (((uintptr_t)a | (uintptr_t)b) % 16) == 0;
}

int launch_rms_norm_limbs2(cudaStream_t st, int dtype, void *workspace, size_t workspace_bytes, const void *x, const void *w, float eps,
                           int rows, int D) {
    int8_t *limbs;
    float *ascale;
    if (int rc = pf_fused_ws(workspace, workspace_bytes, rows, D, &limbs, &ascale)) return rc;
    const size_t smem = (size_t)D * 2;
#define RUN(T)                                                                                                                \
    {                                                                                                                         \
        auto kern = rms_norm_limbs2_kernel<T>;                                                                                \
        if (smem > 48 * 1024) MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        MYNN_CUDA_OK(launch_pdl(kern, dim3(rows), dim3(kLimbThreads), smem, st, limbs, ascale, (const T *)x, (const T *)w, eps, D)); \
    }
    if (dtype == MYNN_BF16) RUN(__nv_bfloat16) else if (dtype == MYNN_F16) RUN(__half) else return fail(MYNN_E_ARG, "rms_norm_limbs2: bad dtype %d", dtype);
#undef RUN
    MYNN_LAUNCH_OK("rms_norm_limbs2_kernel");
    return MYNN_OK;
}

int launch_swiglu_limbs2(cudaStream_t st, int dtype, void *workspace, size_t workspace_bytes, const void *gate, const void *up, int rows,
                         int F, long long in_stride) {
    int8_t *limbs;
    float *ascale;
    if (int rc = pf_fused_ws(workspace, workspace_bytes, rows, F, &limbs, &ascale)) return rc;
    const size_t smem = (size_t)F * 2;
#define RUN(T)                                                                                                                \
    {                                                                                                                         \
        auto kern = swiglu_limbs2_kernel<T>;                                                                                  \
        if (smem > 48 * 1024) MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        MYNN_CUDA_OK(launch_pdl(kern, dim3(rows), dim3(kLimbThreads), smem, st, limbs, ascale, (const T *)gate, (const T *)up, F, in_stride)); \
    }
    if (dtype == MYNN_BF16) RUN(__nv_bfloat16) else if (dtype == MYNN_F16) RUN(__half) else return fail(MYNN_E_ARG, "swiglu_limbs2: bad dtype %d", dtype);
#undef RUN
    MYNN_LAUNCH_OK("swiglu_limbs2_kernel");
    return MYNN_OK;
}

bool i8_w8a8_supported(int M, int N, int K, const void *lhs, const void *rhs) {
    return M >= 1 && N >= 1 && K >= 16 && K % 16 == 0 && (((uintptr_t)lhs | (uintptr_t)rhs) % 16) == 0 && tensor_map_api_available();
}

int i8_w8a8_launch(cudaStream_t st, void *out, const int8_t *lhs, const void *lhs_scale, int lhs_scale_per_row, const int8_t *rhs,
                   const void *rhs_scale, int M, int N, int K, int dtype, void *workspace, size_t workspace_bytes) {
    if (!workspace || workspace_bytes < 256 || (uintptr_t)workspace % 256)
        return fail(MYNN_E_ARG, "quantized_matmul: a 256-byte aligned workspace of at least 256 bytes is needed");
    CUtensorMap mw, ma;
    int rc = make_map(&mw, rhs, (uint64_t)N, (uint64_t)K, (uint64_t)K, kPfRows);
    if (rc) return rc;
    rc = make_map(&ma, lhs, (uint64_t)M, (uint64_t)K, (uint64_t)K, (uint32_t)kPfCols);
    if (rc) return rc;
    PfParams p;
    p.out = out;
    p.scale = rhs_scale;
    p.resid = nullptr;
    p.ascale = nullptr;
    p.ascale_t = lhs_scale;
    p.ascale_stride = lhs_scale_per_row ? 1 : 0;
    p.M = M;
    p.N = N;
    p.K = K;
    p.w_tiles = (N + kPfRows - 1) / kPfRows;
    p.t_tiles = (M + kPfCols - 1) / kPfCols;
    p.status = (int *)workspace;
    if (dtype == MYNN_BF16) return launch_pf<__nv_bfloat16, 1>(st, mw, ma, p);
    if (dtype == MYNN_F16) return launch_pf<__half, 1>(st, mw, ma, p);
    return launch_pf<float, 1>(st, mw, ma, p);
}

}  // namespace mynn
