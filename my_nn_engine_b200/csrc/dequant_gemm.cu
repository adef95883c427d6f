// DequantMatMul for the decode path on sm_100a:  out[m,n] = scale[n] * sum_k act[m,k] * wq[n,k].
//
// The decode step is bound by streaming the int8 weights from HBM once.  The streaming kernel
//   * gives each warp 16 weight rows and lets it pull them straight from global memory into registers with
//     128-bit loads (two rows x 16 bytes per lane per 64-wide k step), one whole 256-wide k stage ahead of
//     the math, so that every lane keeps eight 16-byte loads in flight;
//   * converts int8 -> bf16 (or fp16) in registers with byte-permute bit tricks (exact: |w| <= 128 fits the
//     8-bit significand), and feeds them as the A operand of mma.m16n8k16 with f32 accumulation;
//   * stages the few activation rows (M <= 32, the batch) through shared memory with cp.async double
//     buffering, shared by the 8 warps (128 weight rows) of the CTA; they are the B operand;
//   * splits K over a thread-block cluster and reduces the partial sums through distributed shared memory
//     in a fixed order (deterministic), then applies the per-row scale, an optional residual add, and stores.
// Because a dot product is invariant under a permutation of k, the k index inside each 64-wide step is
// permuted so that the 16 contiguous bytes one lane loads are exactly its A fragments of four MMAs.
//
// f32 activations (the engine's f32 graphs) are split into three bf16 terms (hi + mid + lo = 24 significant
// bits) that occupy three B columns, so the tensor-core product stays f32-accurate.
//
// Shapes outside the fast path (K % 64 != 0, N % 16 != 0, M > 32, [K,N] weight layout) use a plain generic
// kernel: correct for every shape the engine's tests use, not tuned.
#include <cooperative_groups.h>

#include "common.cuh"
#include "i8_cvt.cuh"
#include "i8_gemm.cuh"

namespace cg = cooperative_groups;

namespace mynn {

constexpr int kWarps = 8;            // warps per CTA
constexpr int kRowsPerCta = 16 * kWarps;
constexpr int kStageK = 256;         // k values per activation stage (4 MMA k64 steps)
constexpr int kActPad = 8;           // bf16 elements of row padding (16 B): conflict-free 16-byte fragment reads
constexpr int kActStride = kStageK + kActPad;

__device__ __forceinline__ uint4 ld_stream_16(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void cp_async_16(void *smem, const void *gmem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

template <bool F16>
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    if constexpr (F16) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

template <typename ActT>
struct ActTraits {
    static constexpr bool kF16 = false;
    static constexpr int kColsPerRow = 1;
};
template <>
struct ActTraits<__half> {
    static constexpr bool kF16 = true;
    static constexpr int kColsPerRow = 1;
};
template <>
struct ActTraits<float> {
    static constexpr bool kF16 = false;
    static constexpr int kColsPerRow = 3;  // hi / mid / lo bf16 terms
};

// Stage `klen` (multiple of 64, <= kStageK) activation columns starting at k0 into buf[col][k].
template <typename ActT, int NT>
__device__ __forceinline__ void stage_act(uint16_t *buf, const ActT *act, int M, int K, int k0, int klen) {
    if constexpr (sizeof(ActT) == 2) {
        const int chunks_per_row = klen >> 3;  // 16-byte chunks
        for (int i = threadIdx.x; i < M * chunks_per_row; i += blockDim.x) {
            int m = i / chunks_per_row, c = i - m * chunks_per_row;
            cp_async_16(buf + m * kActStride + c * 8, act + (size_t)m * K + k0 + c * 8);
        }
    } else {
        const int quads_per_row = klen >> 2;
        for (int i = threadIdx.x; i < M * quads_per_row; i += blockDim.x) {
            int m = i / quads_per_row, c = i - m * quads_per_row;
            float4 v = *reinterpret_cast<const float4 *>(act + (size_t)m * K + k0 + c * 4);
            float x[4] = {v.x, v.y, v.z, v.w};
            uint16_t h[4], md[4], l[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                __nv_bfloat16 bh = __float2bfloat16_rn(x[j]);
                float r1 = x[j] - __bfloat162float(bh);
                __nv_bfloat16 bm = __float2bfloat16_rn(r1);
                float r2 = r1 - __bfloat162float(bm);
                __nv_bfloat16 bl = __float2bfloat16_rn(r2);
                h[j] = __bfloat16_as_ushort(bh);
                md[j] = __bfloat16_as_ushort(bm);
                l[j] = __bfloat16_as_ushort(bl);
            }
            uint16_t *d = buf + (3 * m) * kActStride + c * 4;
            *reinterpret_cast<uint2 *>(d) = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
            *reinterpret_cast<uint2 *>(d + kActStride) = make_uint2(md[0] | (md[1] << 16), md[2] | (md[3] << 16));
            *reinterpret_cast<uint2 *>(d + 2 * kActStride) = make_uint2(l[0] | (l[1] << 16), l[2] | (l[3] << 16));
        }
    }
}

// grid (row tiles of 128, S) with cluster (1, S, 1): CTA (x, y) accumulates rows [128x, 128x+128) over the y-th
// contiguous share of the K/64 steps; the cluster then reduces over y.
template <typename ActT, typename OutT, int NT>
__global__ void __launch_bounds__(kWarps * 32)
dequant_gemm_stream_kernel(OutT *out, const ActT *__restrict__ act, const int8_t *__restrict__ wq,
                           const OutT *__restrict__ scale, const OutT *resid, int M, int N, int K) {
    constexpr bool F16 = ActTraits<ActT>::kF16;
    constexpr int CPR = ActTraits<ActT>::kColsPerRow;
    constexpr int COLS = 8 * NT;
    __shared__ __align__(16) uint16_t act_s[2][COLS * kActStride];
    static_assert(sizeof(act_s) >= kRowsPerCta * (COLS + 1) * sizeof(float), "reduction buffer aliases act_s");

    cg::cluster_group cluster = cg::this_cluster();
    const int S = gridDim.y, rank = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

    // this CTA's share of the k64 steps
    const int steps = K >> 6;
    const int q = steps / S, rem = steps - q * S;
    const int step_beg = rank * q + min(rank, rem);
    const int nsteps = q + (rank < rem ? 1 : 0);
    const int kbeg = step_beg << 6;
    const int nstages = (nsteps + 3) >> 2;

    const int row0 = blockIdx.x * kRowsPerCta + warp * 16;
    const bool warp_active = row0 < N;  // N % 16 == 0, so a warp's 16 rows are all in or all out
    const int8_t *w0 = wq + (size_t)(row0 + g) * K + kbeg + 16 * t;
    const int8_t *w1 = w0 + (size_t)8 * K;

    // zero the unused activation columns of both buffers once: they stay zero for the whole kernel
    {
        const int used = M * CPR, chunks = kActStride / 8;
        for (int i = threadIdx.x; i < 2 * (COLS - used) * chunks; i += blockDim.x) {
            const int b = i / ((COLS - used) * chunks), r = i - b * (COLS - used) * chunks;
            reinterpret_cast<uint4 *>(&act_s[b][(used + r / chunks) * kActStride])[r % chunks] = make_uint4(0, 0, 0, 0);
        }
    }
    __syncthreads();

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[j][i] = 0.f;

    uint4 wcur[4][2], wnext[4][2];
    auto load_weights = [&](uint4(&dst)[4][2], int stage) {
#pragma unroll
        for (int s = 0; s < 4; s++) {
            int st = stage * 4 + s;
            if (warp_active && st < nsteps) {
                dst[s][0] = ld_stream_16(w0 + (size_t)st * 64);
                dst[s][1] = ld_stream_16(w1 + (size_t)st * 64);
            } else {
                dst[s][0] = make_uint4(0, 0, 0, 0);
                dst[s][1] = make_uint4(0, 0, 0, 0);
            }
        }
    };

    if (nstages > 0) {
        load_weights(wcur, 0);
        stage_act<ActT, NT>(act_s[0], act, M, K, kbeg, min(4, nsteps) * 64);
        cp_async_commit();
    }
    for (int stage = 0; stage < nstages; stage++) {
        const int buf = stage & 1;
        if (stage + 1 < nstages) {
            load_weights(wnext, stage + 1);
            stage_act<ActT, NT>(act_s[buf ^ 1], act, M, K, kbeg + (stage + 1) * kStageK,
                                min(4, nsteps - (stage + 1) * 4) * 64);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int steps_here = min(4, nsteps - stage * 4);
#pragma unroll
        for (int s = 0; s < 4; s++) {
            if (s < steps_here) {
                // B fragments: 16 consecutive k values of column (8j + g), starting at 64 s + 16 t
                uint4 b[NT][2];
#pragma unroll
                for (int j = 0; j < NT; j++) {
                    const uint16_t *p = &act_s[buf][(8 * j + g) * kActStride + 64 * s + 16 * t];
                    b[j][0] = *reinterpret_cast<const uint4 *>(p);
                    b[j][1] = *reinterpret_cast<const uint4 *>(p + 8);
                }
                const uint32_t wa[4] = {wcur[s][0].x, wcur[s][0].y, wcur[s][0].z, wcur[s][0].w};
                const uint32_t wb[4] = {wcur[s][1].x, wcur[s][1].y, wcur[s][1].z, wcur[s][1].w};
#pragma unroll
                for (int i = 0; i < 4; i++) {  // MMA i covers bytes 4i..4i+3 of each lane's 16
                    uint32_t a0, a2, a1, a3;
                    cvt_s8x4<F16>(wa[i], a0, a2);
                    cvt_s8x4<F16>(wb[i], a1, a3);
#pragma unroll
                    for (int j = 0; j < NT; j++) {
                        const uint32_t *bw = reinterpret_cast<const uint32_t *>(&b[j][i >> 1]);
                        mma_16816<F16>(acc[j], a0, a1, a2, a3, bw[(i & 1) * 2], bw[(i & 1) * 2 + 1]);
                    }
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int s = 0; s < 4; s++) {
            wcur[s][0] = wnext[s][0];
            wcur[s][1] = wnext[s][1];
        }
    }

    // ---- cluster reduction through distributed shared memory ----
    float *red = reinterpret_cast<float *>(&act_s[0][0]);  // [128][COLS + 1]
    constexpr int RS = COLS + 1;
#pragma unroll
    for (int j = 0; j < NT; j++) {
        red[(warp * 16 + g) * RS + 8 * j + 2 * t] = acc[j][0];
        red[(warp * 16 + g) * RS + 8 * j + 2 * t + 1] = acc[j][1];
        red[(warp * 16 + g + 8) * RS + 8 * j + 2 * t] = acc[j][2];
        red[(warp * 16 + g + 8) * RS + 8 * j + 2 * t + 1] = acc[j][3];
    }
    cluster.sync();
    {
        // rank r finishes rows [r * rows_per_rank, ...) of the 128-row tile
        const int rows_per_rank = (kRowsPerCta + S - 1) / S;
        const int rbeg = rank * rows_per_rank;
        const int rcnt = max(0, min(rows_per_rank, kRowsPerCta - rbeg));
        for (int idx = threadIdx.x; idx < rcnt * M; idx += blockDim.x) {
            const int m = idx / rcnt, r = rbeg + (idx - m * rcnt);
            const int n = blockIdx.x * kRowsPerCta + r;
            if (n >= N) continue;
            // issue the (independent) remote reads together, then add in rank order
            float part[8];
#pragma unroll
            for (int rr = 0; rr < 8; rr++) {
                part[rr] = 0.f;
                if (rr < S) {
                    const float *remote = cluster.map_shared_rank(red, rr);
#pragma unroll
                    for (int c = 0; c < CPR; c++) part[rr] += remote[r * RS + CPR * m + c];
                }
            }
            float sum = 0.f;
#pragma unroll
            for (int rr = 0; rr < 8; rr++) sum += part[rr];
            float v = sum * to_f32<OutT>(scale[n]);
            if (resid != nullptr) v = round_store<OutT>(v) + to_f32<OutT>(resid[(size_t)m * N + n]);
            out[(size_t)m * N + n] = from_f32<OutT>(v);
        }
    }
    cluster.sync();  // keep shared memory alive until every peer has read it
}

// Generic kernel: one warp per output element, any shape and either weight layout (element strides given).
template <typename ActT, typename OutT>
__global__ void dequant_matmul_generic_kernel(OutT *out, const ActT *act, const int8_t *wq, const OutT *scale,
                                              const OutT *resid, int M, int N, int K, long long w_stride_n,
                                              long long w_stride_k) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= M * N) return;
    const int m = warp / N, n = warp - m * N;
    float acc = 0.f;
    for (int k = lane; k < K; k += 32)
        acc += to_f32<ActT>(act[(size_t)m * K + k]) * (float)wq[n * w_stride_n + k * w_stride_k];
    acc = warp_sum(acc);
    if (lane == 0) {
        float v = acc * to_f32<OutT>(scale[n]);
        if (resid != nullptr) v = round_store<OutT>(v) + to_f32<OutT>(resid[(size_t)m * N + n]);
        out[(size_t)m * N + n] = from_f32<OutT>(v);
    }
}

// [K,N] layout (per-column scale): each thread owns 4 adjacent columns, the block's y dimension splits K and the
// partial sums meet in shared memory.  Reads of W are coalesced along N.
template <typename ActT, typename OutT>
__global__ void __launch_bounds__(256)
dequant_gemv_kn_kernel(OutT *out, const ActT *act, const int8_t *wq, const OutT *scale, int N, int K) {
    __shared__ float part[8][128];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int n0 = blockIdx.x * 128 + tx * 4;
    const int m = blockIdx.y;
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    if (n0 < N) {
        for (int k = ty; k < K; k += 8) {
            const char4 w = *reinterpret_cast<const char4 *>(wq + (size_t)k * N + n0);
            const float x = to_f32<ActT>(act[(size_t)m * K + k]);
            a[0] += x * (float)w.x;
            a[1] += x * (float)w.y;
            a[2] += x * (float)w.z;
            a[3] += x * (float)w.w;
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) part[ty][tx * 4 + i] = a[i];
    __syncthreads();
    if (threadIdx.x < 128) {
        const int n = blockIdx.x * 128 + threadIdx.x;
        if (n < N) {
            float s = 0.f;
#pragma unroll
            for (int y = 0; y < 8; y++) s += part[y][threadIdx.x];
            out[(size_t)m * N + n] = from_f32<OutT>(s * to_f32<OutT>(scale[n]));
        }
    }
}

// [K,N] layout, the tuned form: the literal single-op graph DequantizeLinear(W [K,N], per-column scale) -> MatMul, which the
// engine runs unfused.  A thread owns 16 adjacent columns, i.e. one 128-bit load per k row (a warp reads 512 contiguous
// bytes); a CTA of 16 warps covers 512 columns x a k range in which every lane issues all its loads (up to 16) before it
// waits for anything; the k dimension is split over a cluster of 8 CTAs and reduced through distributed shared memory in a
// fixed order, so the result does not depend on timing.  int8 -> f32 is exact (byte-permute into the mantissa of 2^23,
// one subtraction), the products accumulate in f32 as in the engine's kernels.
// grid (ceil(N / 512), 8, M), cluster (1, 8, 1), block 512.  N % 16 == 0, wq 16-byte aligned.
constexpr int kKnThreads = 512, kKnCols = 512, kKnSplit = 8, kKnRowsPerWarp = 16;

template <typename ActT, typename OutT>
__global__ void __launch_bounds__(kKnThreads, 1)
dequant_gemv_kn_split_kernel(OutT *out, const ActT *act, const int8_t *wq, const OutT *scale, int N, int K) {
    __shared__ float part[kKnThreads / 32][kKnCols + 16];  // per-warp partial sums of the CTA's 512 columns (padded rows)
    __shared__ float cta_part[kKnCols];
    __shared__ float act_s[kKnThreads / 32 * kKnRowsPerWarp];
    cg::cluster_group cluster = cg::this_cluster();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m = blockIdx.z, rank = blockIdx.y;
    const int n0 = blockIdx.x * kKnCols + lane * 16;
    const bool col_live = n0 < N;
    // this CTA's k range, and inside it this warp's rows
    const int per_cta = (K + kKnSplit - 1) / kKnSplit;
    const int k_beg = rank * per_cta, k_end = min(K, k_beg + per_cta);
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; i++) acc[i] = 0.f;
    for (int kb = k_beg; kb < k_end; kb += (kKnThreads / 32) * kKnRowsPerWarp) {  // one pass when K <= 8 * 256
        const int k0 = kb + warp * kKnRowsPerWarp;
        uint4 w[kKnRowsPerWarp];
#pragma unroll
        for (int r = 0; r < kKnRowsPerWarp; r++)
            w[r] = (col_live && k0 + r < k_end) ? ld_stream_16(wq + (size_t)(k0 + r) * N + n0) : make_uint4(0u, 0u, 0u, 0u);
        __syncthreads();  // act_s of the previous pass has been read
        if (lane < kKnRowsPerWarp) act_s[warp * kKnRowsPerWarp + lane] = k0 + lane < k_end ? to_f32<ActT>(act[(size_t)m * K + k0 + lane]) : 0.f;
        __syncwarp();
#pragma unroll
        for (int r = 0; r < kKnRowsPerWarp; r++) {
            const float a = act_s[warp * kKnRowsPerWarp + r];
            const uint32_t ww[4] = {w[r].x ^ 0x80808080u, w[r].y ^ 0x80808080u, w[r].z ^ 0x80808080u, w[r].w ^ 0x80808080u};
#pragma unroll
            for (int q = 0; q < 4; q++)
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    // 0x4B0000bb is the float 2^23 + bb; with bb = byte + 128 the difference to 2^23 + 128 is the signed byte
                    const float f = __uint_as_float(__byte_perm(ww[q], 0x4B000000u, 0x7650 + b)) - 8388736.0f;
                    acc[4 * q + b] = fmaf(a, f, acc[4 * q + b]);
                }
        }
    }
#pragma unroll
    for (int i = 0; i < 16; i += 4)
        *reinterpret_cast<float4 *>(&part[warp][lane * 16 + i]) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
    __syncthreads();
    {
        float s = 0.f;
#pragma unroll
        for (int w_ = 0; w_ < kKnThreads / 32; w_++) s += part[w_][threadIdx.x];
        cta_part[threadIdx.x] = s;
    }
    cluster.sync();
    // rank r finishes columns [64 r, 64 r + 64) of the 512: the eight CTAs' sums in rank order, then the column scale
    if (threadIdx.x < kKnCols / kKnSplit) {
        const int c = rank * (kKnCols / kKnSplit) + threadIdx.x;
        const int n = blockIdx.x * kKnCols + c;
        float v[kKnSplit];
#pragma unroll
        for (int rr = 0; rr < kKnSplit; rr++) v[rr] = cluster.map_shared_rank(cta_part, rr)[c];
        float s = 0.f;
#pragma unroll
        for (int rr = 0; rr < kKnSplit; rr++) s += v[rr];
        if (n < N) out[(size_t)m * N + n] = from_f32<OutT>(s * to_f32<OutT>(scale[n]));
    }
    cluster.sync();  // keep shared memory alive until every peer has read it
}

template <typename ActT, typename OutT>
static int launch_kn_split(cudaStream_t st, OutT *out, const ActT *act, const int8_t *wq, const OutT *scale, int M, int N, int K) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((N + kKnCols - 1) / kKnCols, kKnSplit, M);
    cfg.blockDim = dim3(kKnThreads, 1, 1);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = kKnSplit;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MYNN_CUDA_OK(cudaLaunchKernelEx(&cfg, dequant_gemv_kn_split_kernel<ActT, OutT>, out, act, wq, scale, N, K));
    MYNN_LAUNCH_OK("dequant_gemv_kn_split_kernel");
    return MYNN_OK;
}

static int pick_ksplit(int row_tiles, int steps) {
    // Every CTA pays a fixed prologue and a cluster reduction, so split K only until there is about one CTA per
    // SM (148), keep at least 8 k64 steps (two stages) per CTA, and stay within the portable cluster size of 8.
    int s = 1;
    while (s < 8 && row_tiles * s < 148 && steps / (s * 2) >= 8) s *= 2;
    return s;
}

template <typename ActT, typename OutT, int NT>
static int launch_stream(cudaStream_t st, OutT *out, const ActT *act, const int8_t *wq, const OutT *scale,
                         const OutT *resid, int M, int N, int K, int ksplit_override) {
    const int row_tiles = (N + kRowsPerCta - 1) / kRowsPerCta;
    int S = ksplit_override > 0 ? ksplit_override : pick_ksplit(row_tiles, K / 64);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(row_tiles, S, 1);
    cfg.blockDim = dim3(kWarps * 32, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = S;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MYNN_CUDA_OK(cudaLaunchKernelEx(&cfg, dequant_gemm_stream_kernel<ActT, OutT, NT>, out, act, wq, scale, resid, M, N, K));
    MYNN_LAUNCH_OK("dequant_gemm_stream_kernel");
    return MYNN_OK;
}


template <typename ActT, typename OutT>
static int dequant_matmul_typed(cudaStream_t st, OutT *out, const ActT *act, const int8_t *wq, const OutT *scale,
                                const OutT *resid, int M, int N, int K, int w_layout) {
    constexpr int CPR = ActTraits<ActT>::kColsPerRow;
    const bool aligned = ((uintptr_t)wq % 16 == 0) && ((uintptr_t)act % 16 == 0);
    if (w_layout == MYNN_W_NK && K % 64 == 0 && N % 16 == 0 && M * CPR <= 32 && aligned) {
        const int cols = M * CPR;
        if (cols <= 8) return launch_stream<ActT, OutT, 1>(st, out, act, wq, scale, resid, M, N, K, g_ksplit_override);
        if (cols <= 16) return launch_stream<ActT, OutT, 2>(st, out, act, wq, scale, resid, M, N, K, g_ksplit_override);
        return launch_stream<ActT, OutT, 4>(st, out, act, wq, scale, resid, M, N, K, g_ksplit_override);
    }
    if (w_layout == MYNN_W_KN && N % 16 == 0 && ((uintptr_t)wq % 16 == 0) && resid == nullptr && M <= 4 && K >= 64)
        return launch_kn_split<ActT, OutT>(st, out, act, wq, scale, M, N, K);
    if (w_layout == MYNN_W_KN && N % 4 == 0 && ((uintptr_t)wq % 4 == 0) && resid == nullptr) {
        dequant_gemv_kn_kernel<ActT, OutT><<<dim3((N + 127) / 128, M), 256, 0, st>>>(out, act, wq, scale, N, K);
        MYNN_LAUNCH_OK("dequant_gemv_kn_kernel");
        return MYNN_OK;
    }
    const long long sn = w_layout == MYNN_W_NK ? K : 1, sk = w_layout == MYNN_W_NK ? 1 : N;
    const long long warps = (long long)M * N;
    const int blocks = (int)((warps * 32 + 255) / 256);
    dequant_matmul_generic_kernel<ActT, OutT><<<blocks, 256, 0, st>>>(out, act, wq, scale, resid, M, N, K, sn, sk);
    MYNN_LAUNCH_OK("dequant_matmul_generic_kernel");
    return MYNN_OK;
}

static int dequant_matmul_dispatch(void *stream, void *out, const void *act, const int8_t *wq, const void *scale,
                                   const void *resid, int M, int N, int K, int act_dtype, int out_dtype,
                                   int w_layout, void *workspace, size_t workspace_bytes) {
    if (M < 0 || N < 0 || K < 0) return fail(MYNN_E_ARG, "dequant_matmul: negative dimension (M=%d N=%d K=%d)", M, N, K);
    if (w_layout != MYNN_W_NK && w_layout != MYNN_W_KN) return fail(MYNN_E_ARG, "dequant_matmul: bad weight layout %d", w_layout);
    if (!dtype_ok(act_dtype) || !dtype_ok(out_dtype)) return fail(MYNN_E_ARG, "dequant_matmul: bad dtype");
    if (M == 0 || N == 0) return MYNN_OK;
    if (!out || !wq || !scale || (!act && K > 0)) return fail(MYNN_E_ARG, "dequant_matmul: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    // With scratch memory the tcgen05 int8 kernel takes every [N,K] problem of up to 32 rows.
    if (workspace && w_layout == MYNN_W_NK && i8_gemm_supported(M, N, K, wq, act_dtype, out_dtype))
        return i8_gemm_launch(st, out, act, wq, scale, resid, M, N, K, act_dtype, out_dtype, workspace, workspace_bytes);
    // More rows: the prefill kernel (two activation limbs, 128 x 128-token tiles) if the scratch is large enough.
    if (workspace && w_layout == MYNN_W_NK && i8_prefill_supported(M, N, K, wq, act_dtype, out_dtype) &&
        workspace_bytes >= i8_prefill_workspace_bytes(M, K))
        return i8_prefill_launch(st, out, act, wq, scale, resid, M, N, K, act_dtype, out_dtype, workspace, workspace_bytes);
#define CASE(AD, AT, OD, OT)                                                                                        \
    if (act_dtype == AD && out_dtype == OD)                                                                         \
        return dequant_matmul_typed<AT, OT>(st, (OT *)out, (const AT *)act, wq, (const OT *)scale, (const OT *)resid, \
                                            M, N, K, w_layout);
    CASE(MYNN_BF16, __nv_bfloat16, MYNN_BF16, __nv_bfloat16)
    CASE(MYNN_F16, __half, MYNN_F16, __half)
    CASE(MYNN_F32, float, MYNN_F32, float)
    CASE(MYNN_BF16, __nv_bfloat16, MYNN_F32, float)
    CASE(MYNN_F32, float, MYNN_BF16, __nv_bfloat16)
#undef CASE
    return fail(MYNN_E_UNSUPPORTED, "dequant_matmul: act dtype %d with out dtype %d is not supported", act_dtype, out_dtype);
}

}  // namespace mynn

extern "C" size_t mynn_b200_dequant_matmul_workspace_bytes(int M, int N, int K) {
    (void)N;
    if (M > mynn::kI8MaxRows) return mynn::i8_prefill_workspace_bytes(M, K);
    return mynn::i8_gemm_workspace_bytes(M, K);
}

extern "C" int mynn_b200_dequant_matmul(void *stream, void *out, const void *act, const int8_t *wq, const void *scale,
                                        int M, int N, int K, int act_dtype, int out_dtype, int w_layout,
                                        void *workspace, size_t workspace_bytes) {
    return mynn::dequant_matmul_dispatch(stream, out, act, wq, scale, nullptr, M, N, K, act_dtype, out_dtype, w_layout,
                                         workspace, workspace_bytes);
}

extern "C" int mynn_b200_dequant_matmul_residual(void *stream, void *out, const void *act, const int8_t *wq,
                                                 const void *scale, const void *residual, int M, int N, int K,
                                                 int dtype, void *workspace, size_t workspace_bytes) {
    return mynn::dequant_matmul_dispatch(stream, out, act, wq, scale, residual, M, N, K, dtype, dtype, MYNN_W_NK,
                                         workspace, workspace_bytes);
}

// DequantMatMul for activations that the PREVIOUS call on this workspace already converted: several weight matrices
// applied to one activation tensor (q, k and v of a layer; gate and up) need the conversion to limbs only once.
extern "C" int mynn_b200_dequant_matmul_same_act(void *stream, void *out, const int8_t *wq, const void *scale, int M, int N,
                                                 int K, int act_dtype, int out_dtype, void *workspace, size_t workspace_bytes) {
    using namespace mynn;
    if (M <= 0 || N <= 0 || K <= 0) return fail(MYNN_E_ARG, "dequant_matmul_same_act: bad shape");
    if (!out || !wq || !scale) return fail(MYNN_E_ARG, "dequant_matmul_same_act: null pointer");
    if (!dtype_ok(act_dtype) || !dtype_ok(out_dtype)) return fail(MYNN_E_ARG, "dequant_matmul_same_act: bad dtype");
    if (!workspace || !i8_gemm_supported(M, N, K, wq, act_dtype, out_dtype))
        return fail(MYNN_E_UNSUPPORTED, "dequant_matmul_same_act: needs the tensor-core path (a workspace, at most %d rows, K %% 16 == 0, 16-byte aligned weights)", kI8MaxRows);
    return i8_gemm_launch((cudaStream_t)stream, out, nullptr, wq, scale, nullptr, M, N, K, act_dtype, out_dtype, workspace, workspace_bytes);
}

// Reads the status word of a DequantMatMul workspace after synchronising the stream: non-zero means a pipeline
// wait inside the tcgen05 kernel ran out of time and the outputs of that call are invalid.
extern "C" int mynn_b200_dequant_matmul_check(void *stream, const void *workspace) {
    if (!workspace) return MYNN_OK;
    int status = 0;
    MYNN_CUDA_OK(cudaMemcpyAsync(&status, workspace, sizeof status, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    MYNN_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
    if (status) {  // reported once: clear the word so that later calls on this workspace start clean
        MYNN_CUDA_OK(cudaMemsetAsync(const_cast<void *>(workspace), 0, sizeof status, (cudaStream_t)stream));
        MYNN_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
        return mynn::fail(MYNN_E_CUDA, "dequant_matmul: pipeline wait %d timed out inside a kernel that uses this workspace (1-3: the tcgen05 DequantMatMul, 31: decode attention waiting for a K/V tile)", status);
    }
    return MYNN_OK;
}

#ifdef MYNN_TUNING
// Tuning build only: device buffer (8 x uint64) that CTA (0,0) of the tcgen05 GEMM fills with nanosecond timestamps of its
// phases (start, set-up done, predecessor complete, accumulators complete, cluster ready, outputs stored, end); NULL = off.
extern "C" int mynn_b200_tuning_set_timing_buffer(void *buf, int slots) {
    mynn::g_i8_timing = (unsigned long long *)buf;
    mynn::g_i8_timing_slots = slots > 0 ? slots : 1;
    mynn::g_i8_timing_next = 0;
    return MYNN_OK;
}
namespace mynn { int glue_timing_read(unsigned long long *out, unsigned *n); }
extern "C" int mynn_b200_tuning_read_glue(unsigned long long *out, unsigned *n) { return mynn::glue_timing_read(out, n); }
extern "C" int mynn_b200_tuning_set_stages(int n) {
    mynn::g_i8_stages_override = n;
    return MYNN_OK;
}
#endif
