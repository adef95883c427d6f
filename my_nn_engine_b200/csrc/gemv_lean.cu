// Lean DequantMatMul for one to four activation rows over small weight matrices (the GEMV of batch-1 decode).
//
//   out[m,n] = scale[n] * sum_k act[m,k] * wq[n,k],   M <= 4, wq [N,K] int8 of at most a few tens of MB
//
// A matrix of 10-30 MB streams from HBM in 2-5 us, so everything that is fixed cost in the tcgen05 kernel (tensor-memory
// allocation, tensor maps, mbarrier ring, a separate limb pre-pass launch, 128-row tiles that leave SMs idle) would dominate.
// This kernel has none of it (the engine's counterpart is dequant_gemv, src/codegen/cuda/cpp/dequant_gemv.cuh:11-59: one
// warp per row, one 16-byte load in flight per lane):
//   * one CTA per SM with an equal share of the rows, so the grid is a single balanced wave; a warp takes up to four weight
//     rows at a time and each lane issues all its 128-bit loads of those rows (up to 16) before it touches anything else, and
//     before the programmatic-dependent-launch wait, so the weights are in flight while the preceding kernel drains;
//   * the activation row(s) are held in shared memory as the same three signed 8-bit limbs of a 23-bit fixed-point value
//     the tensor-core kernel uses (either copied from the workspace, where a fused producer left them, or computed here from
//     the activation tensor: no extra launch), so a weight never needs converting: 16 weights x 3 limbs are 12 dp4a
//     instructions with exact int32 accumulation;
//   * warp-shuffle reduction, limbs recombined in int64, the same two roundings as the tensor-core kernel: the outputs are
//     bit-identical to that kernel's, whichever of the two a shape is dispatched to.
// Measured against it and dropped: staging the weights through shared memory with untiled bulk copies (cp.async.bulk) so that
// the next kernel's CTA fits beside this one (6.5 us against 4.3 us per launch on a 5632 x 2048 matrix), and 256-thread CTAs
// two per SM (4.7 us).
#include "common.cuh"
#include "i8_gemm.cuh"

namespace mynn {

constexpr int kLeanThreads = 512;

struct LeanParams {
    void *out;
    const void *act;        // [M,K] or null (then limbs_g / ascale_g hold the activations)
    const int8_t *wq;
    const void *scale, *resid;
    int8_t *limbs_g;        // workspace limb matrix [(3m + l)][K]; read when act == null, written by CTA 0 otherwise
    float *ascale_g;        // [M] row scales
    int N, K, act_dtype, rows_per_cta;
};

__device__ __forceinline__ uint4 ldg_stream_16(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// One activation row -> limbs in shared memory (and, from CTA 0, in the workspace), with the arithmetic of the limb pre-pass
// of the tensor-core kernel: |a| * 2^(22-e) rounded to an integer below 2^22, split into three signed bytes.  Rows of up to
// 8 elements per thread stay in registers between the two passes.
template <typename ActT>
__device__ __forceinline__ void row_to_limbs(const ActT *row, int K, int8_t *l_s, int8_t *l_g, float *ascale_s, float *ascale_g,
                                             float *red) {
    constexpr int kKeep = 8;
    float keep[kKeep];
    float mx = 0.f;
    bool bad = false;
#pragma unroll
    for (int u = 0; u < kKeep; u++) {
        const int i = threadIdx.x + u * kLeanThreads;
        keep[u] = i < K ? to_f32<ActT>(row[i]) : 0.f;
        bad |= !(fabsf(keep[u]) <= 3.0e38f);
        mx = fmaxf(mx, fabsf(keep[u]));
    }
    for (int i = threadIdx.x + kKeep * kLeanThreads; i < K; i += kLeanThreads) {
        const float a = to_f32<ActT>(row[i]);
        bad |= !(fabsf(a) <= 3.0e38f);
        mx = fmaxf(mx, fabsf(a));
    }
    mx = warp_max(mx);
    const unsigned anybad = __syncthreads_or(bad);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    float t = red[0];
#pragma unroll
    for (int w = 1; w < kLeanThreads / 32; w++) t = fmaxf(t, red[w]);
    int e = 0;
    if (t > 0.f) frexpf(t, &e);
    const float sc1 = t > 0.f ? ldexpf(1.0f, 22 - e) : 1.0f;
    const float sc = anybad ? 0.f : sc1;
    if (threadIdx.x == 0) {
        const float as = anybad ? __int_as_float(0x7fc00000) : 1.0f / sc1;  // a non-finite input row gives NaN outputs
        *ascale_s = as;
        if (ascale_g) *ascale_g = as;
    }
    auto emit = [&](float a, int i) {
        int A = sc == 0.f ? 0 : __float2int_rn(a * sc);
        const int d0 = (int)(int8_t)(A & 0xFF);
        A = (A - d0) >> 8;
        const int d1 = (int)(int8_t)(A & 0xFF);
        A = (A - d1) >> 8;
        l_s[i] = (int8_t)d0;
        l_s[K + i] = (int8_t)d1;
        l_s[2 * K + i] = (int8_t)A;
        if (l_g) {
            l_g[i] = (int8_t)d0;
            l_g[K + i] = (int8_t)d1;
            l_g[2 * (size_t)K + i] = (int8_t)A;
        }
    };
#pragma unroll
    for (int u = 0; u < kKeep; u++) {
        const int i = threadIdx.x + u * kLeanThreads;
        if (i < K) emit(keep[u], i);
    }
    for (int i = threadIdx.x + kKeep * kLeanThreads; i < K; i += kLeanThreads) emit(to_f32<ActT>(row[i]), i);
    __syncthreads();  // red is reused by the next row
}

// One CTA per SM owns a contiguous range of weight rows, so that the whole grid is one balanced wave.  A warp takes groups
// of RF consecutive rows; CPL = 16-byte chunks per lane and row (K <= 512 * CPL), so a group is RF * CPL <= 16 loads per lane,
// all issued before anything else happens.  K % 16 == 0; wq and limbs 16-byte aligned.
template <typename OutT, int M, int CPL, int RF>
__global__ void __launch_bounds__(kLeanThreads, 1) gemv_lean_kernel(const LeanParams p) {
    extern __shared__ __align__(16) int8_t sm_limbs[];  // [M][3][K]
    __shared__ float sm_ascale[4];
    __shared__ float red[kLeanThreads / 32];
    constexpr int kWarps = kLeanThreads / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K = p.K, chunks = K >> 4;
    const int cta_row0 = blockIdx.x * p.rows_per_cta;
    const int cta_rows = min(p.rows_per_cta, p.N - cta_row0);
    const int groups = (cta_rows + RF - 1) / RF;
    const OutT *scale_p = reinterpret_cast<const OutT *>(p.scale);
    const OutT *resid_p = reinterpret_cast<const OutT *>(p.resid);
    OutT *out_p = reinterpret_cast<OutT *>(p.out);

    uint4 w[RF][CPL];
    auto load_group = [&](int g) {
#pragma unroll
        for (int r = 0; r < RF; r++) {
            const int row = g * RF + r;
            const int8_t *wr = p.wq + (size_t)(cta_row0 + (row < cta_rows ? row : 0)) * K;
#pragma unroll
            for (int j = 0; j < CPL; j++) {
                const int c = lane + 32 * j;
                w[r][j] = (row < cta_rows && c < chunks) ? ldg_stream_16(wr + 16 * (size_t)c) : make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };
    // the first group of weights and its row scales depend on nothing an earlier kernel writes: get them moving before the wait
    if (warp < groups) load_group(warp);
    float wscale_first = 0.f;
    if (lane < RF && warp * RF + lane < cta_rows) wscale_first = to_f32<OutT>(scale_p[cta_row0 + warp * RF + lane]);
    pdl_trigger();
    pdl_wait();
    float resv_first[M];
#pragma unroll
    for (int m = 0; m < M; m++)
        resv_first[m] = (resid_p && lane < RF && warp * RF + lane < cta_rows) ? to_f32<OutT>(resid_p[(size_t)m * p.N + cta_row0 + warp * RF + lane]) : 0.f;
    // activations -> limbs in shared memory
    if (p.act != nullptr) {
        int8_t *lg = blockIdx.x == 0 ? p.limbs_g : nullptr;
        float *ag = blockIdx.x == 0 ? p.ascale_g : nullptr;
#pragma unroll 1
        for (int m = 0; m < M; m++) {
            int8_t *ls = sm_limbs + (size_t)m * 3 * K;
            if (p.act_dtype == MYNN_F32)
                row_to_limbs<float>((const float *)p.act + (size_t)m * K, K, ls, lg ? lg + (size_t)m * 3 * K : nullptr, &sm_ascale[m], ag ? ag + m : nullptr, red);
            else if (p.act_dtype == MYNN_BF16)
                row_to_limbs<__nv_bfloat16>((const __nv_bfloat16 *)p.act + (size_t)m * K, K, ls, lg ? lg + (size_t)m * 3 * K : nullptr, &sm_ascale[m], ag ? ag + m : nullptr, red);
            else
                row_to_limbs<__half>((const __half *)p.act + (size_t)m * K, K, ls, lg ? lg + (size_t)m * 3 * K : nullptr, &sm_ascale[m], ag ? ag + m : nullptr, red);
        }
    } else {
        const uint4 *src = reinterpret_cast<const uint4 *>(p.limbs_g);
        uint4 *dst = reinterpret_cast<uint4 *>(sm_limbs);
        for (int i = threadIdx.x; i < (M * 3 * K) >> 4; i += kLeanThreads) dst[i] = __ldcg(src + i);
        if (threadIdx.x < M) sm_ascale[threadIdx.x] = __ldcg(p.ascale_g + threadIdx.x);
    }
    __syncthreads();

    for (int g = warp; g < groups; g += kWarps) {
        if (g != warp) load_group(g);
        // weight-row scales (and residuals) of the group: requested before the arithmetic
        const int my_row = cta_row0 + g * RF + lane;  // lanes 0..RF-1 each finish one row of the group
        const bool my_live = lane < RF && g * RF + lane < cta_rows;
        float wscale = wscale_first;  // the first group's were requested at the top of the kernel
        float resv[M];
#pragma unroll
        for (int m = 0; m < M; m++) resv[m] = resv_first[m];
        if (g != warp) {
            wscale = my_live ? to_f32<OutT>(scale_p[my_row]) : 0.f;
#pragma unroll
            for (int m = 0; m < M; m++) resv[m] = (my_live && resid_p) ? to_f32<OutT>(resid_p[(size_t)m * p.N + my_row]) : 0.f;
        }
        int acc[RF][M][3];
#pragma unroll
        for (int r = 0; r < RF; r++)
#pragma unroll
            for (int m = 0; m < M; m++) acc[r][m][0] = acc[r][m][1] = acc[r][m][2] = 0;
#pragma unroll
        for (int j = 0; j < CPL; j++) {
            const int c = lane + 32 * j;
            if (c < chunks) {
#pragma unroll
                for (int m = 0; m < M; m++)
#pragma unroll
                    for (int l = 0; l < 3; l++) {
                        const uint4 a = *reinterpret_cast<const uint4 *>(sm_limbs + ((size_t)(m * 3 + l)) * K + 16 * (size_t)c);
#pragma unroll
                        for (int r = 0; r < RF; r++) {
                            int s = acc[r][m][l];
                            s = __dp4a((int)w[r][j].x, (int)a.x, s);
                            s = __dp4a((int)w[r][j].y, (int)a.y, s);
                            s = __dp4a((int)w[r][j].z, (int)a.z, s);
                            s = __dp4a((int)w[r][j].w, (int)a.w, s);
                            acc[r][m][l] = s;
                        }
                    }
            }
        }
        // warp reduction; lane r then finishes row r with the arithmetic of the tensor-core kernel's epilogue
#pragma unroll
        for (int r = 0; r < RF; r++)
#pragma unroll
            for (int m = 0; m < M; m++) {
                int v0 = acc[r][m][0], v1 = acc[r][m][1], v2 = acc[r][m][2];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    v0 += __shfl_xor_sync(0xffffffffu, v0, o);
                    v1 += __shfl_xor_sync(0xffffffffu, v1, o);
                    v2 += __shfl_xor_sync(0xffffffffu, v2, o);
                }
                const long long sum = (long long)v2 * 65536 + (long long)v1 * 256 + (long long)v0;
                if (lane == r && my_live) {
                    float v = __fmul_rn(__fmul_rn((float)sum, sm_ascale[m]), wscale);
                    if (resid_p) v = __fadd_rn(round_store<OutT>(v), resv[m]);
                    out_p[(size_t)m * p.N + my_row] = from_f32<OutT>(v);
                }
            }
    }
}

bool gemv_lean_supported(int M, int N, int K, const void *wq) {
    // small matrices only: larger ones amortise the tensor-core kernel's set-up and stream faster there
    return M >= 1 && M <= 4 && K >= 16 && K % 16 == 0 && K <= 6144 && (size_t)3 * M * K <= 96 * 1024 && (size_t)N * K <= ((size_t)32 << 20) &&
           ((uintptr_t)wq % 16) == 0;
}

template <typename OutT, int M, int CPL, int RF>
static int launch_lean(cudaStream_t st, LeanParams p) {
    const size_t smem = (size_t)3 * M * p.K;
    auto kern = gemv_lean_kernel<OutT, M, CPL, RF>;
    if (smem > 48 * 1024) MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    // one CTA per SM, each with an equal share of the rows (a multiple of RF)
    int rpc = (p.N + sms - 1) / sms;
    rpc = (rpc + RF - 1) / RF * RF;
    p.rows_per_cta = rpc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.N + rpc - 1) / rpc);
    cfg.blockDim = dim3(kLeanThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may start (and load weights) while its predecessor drains
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MYNN_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, p));
    MYNN_LAUNCH_OK("gemv_lean_kernel");
    return MYNN_OK;
}

// Same contract as i8_gemm_launch: `workspace` holds status word, row scales and the limb matrix; act == nullptr means a fused
// producer (or the previous call) left the limbs there.
int gemv_lean_launch(cudaStream_t st, void *out, const void *act, const int8_t *wq, const void *scale, const void *resid, int M, int N,
                     int K, int act_dtype, int out_dtype, void *workspace, size_t workspace_bytes) {
    const size_t need = i8_gemm_workspace_bytes(M, K);
    if (!workspace || workspace_bytes < need || (uintptr_t)workspace % 256)
        return fail(MYNN_E_ARG, "dequant_matmul: workspace of %zu bytes (256-byte aligned) needed", need);
    LeanParams p;
    p.out = out;
    p.act = act;
    p.wq = wq;
    p.scale = scale;
    p.resid = resid;
    p.ascale_g = (float *)((char *)workspace + 256);
    p.limbs_g = (int8_t *)workspace + 512;
    p.N = N;
    p.K = K;
    p.act_dtype = act_dtype;
    p.rows_per_cta = 0;
    // chunks per lane (K <= 2048 / 4096 / 6144) and rows in flight per warp: 16 loads per lane, at most 24 accumulators
#define BY_K(OT, MV, RF4, RF8)                                \
    if (K <= 2048) return launch_lean<OT, MV, 4, RF4>(st, p); \
    if (K <= 4096) return launch_lean<OT, MV, 8, RF8>(st, p); \
    return launch_lean<OT, MV, 12, 1>(st, p);
#define GO(OT)                    \
    switch (M) {                  \
        case 1: BY_K(OT, 1, 4, 2) \
        case 2: BY_K(OT, 2, 4, 2) \
        case 3: BY_K(OT, 3, 2, 2) \
        default: BY_K(OT, 4, 2, 2) \
    }
    if (out_dtype == MYNN_BF16) GO(__nv_bfloat16)
    if (out_dtype == MYNN_F16) GO(__half)
    GO(float)
#undef GO
#undef BY_K
}

}  // namespace mynn
