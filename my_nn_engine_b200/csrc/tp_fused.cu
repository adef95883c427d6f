// Tensor-parallel all-reduce fused with the operators around it, over NVLink peer memory (data flow: tp_fused.cuh).
//
// A row-parallel DequantMatMul (o_proj, down_proj) leaves an f32 partial sum [rows, hidden] on every rank.  The engine's
// schedule then needs: all-reduce(sum) -> round -> residual add -> RMSNorm -> (here) activation limbs for the next
// DequantMatMul on every rank (its AllReduce operator, src/graph/operator.rs, sums f32 in rank order:
// crates/comm/src/uds.rs:106-116).  Here the producing GEMM delivers its partial sums to every rank with peer STORES from its
// epilogue, and ONE kernel per rank sums the `world` partial rows it finds in its own memory, in rank order, and finishes
// the row: residual add, RMSNorm, limbs.
//
// Ordering without fences.  A partial sum is one 4-byte word; a slot that holds no value holds the EMPTY word (kTpEmpty, a
// NaN pattern that is never delivered).  The reader polls a 16-byte piece until none of its four words is EMPTY; a word that
// is not EMPTY is the value, because a 4-byte store is never torn.  Having read a piece, the reader stores EMPTY back, so the
// buffer is ready for its next use.  That next use is the reduction after the next one on the other buffer, and no value of
// it can arrive before the reader has put EMPTY back: a rank can only deliver partial sums of reduction j+2 after it has
// finished its own reduction j+1, which needed THIS rank's partial sums of j+1, which this rank computed after its reduction
// j, the kernel that put EMPTY back.
//
// The wait is bounded (MYNN_OPT_WAIT_BUDGET_US, default 2 s): on expiry the kernel records status 21, goes on with what it
// has (EMPTY reads as NaN), still puts EMPTY back and returns; the host reports MYNN_E_COMM at its next check.  A lost peer
// therefore never hangs a GPU.  After a rank that delivered NOTHING the group is in step again at the next reduction; after
// a rank that delivered LATE (past the budget) its stale values could be taken for those of a later reduction, so a caller
// that has seen MYNN_E_COMM and wants to go on re-initialises the blocks (mynn_b200_tp_block_init) with all ranks idle.
#include <cstring>

#include "common.cuh"
#include "i8_gemm.cuh"
#include "tcgen05.cuh"
#include "tp_fused.cuh"

namespace mynn {

MYNN_DEFINE_WAIT_BUDGET_SETTER(tp_fused)

static size_t up256(size_t x) { return (x + 255) / 256 * 256; }

TpLayout tp_layout(int max_rows, int hidden, int world) {
    TpLayout l;
    l.world = world;
    l.max_rows = max_rows;
    l.hidden = hidden;
    size_t off = sizeof(TpHeader);
    const size_t part = up256((size_t)world * max_rows * hidden * sizeof(uint32_t));
    l.part_off[0] = off;
    off += part;
    l.part_off[1] = off;
    off += part;
    l.bytes = off;
    return l;
}

// header zero, every partial-sum word EMPTY
int tp_block_init(cudaStream_t st, char *block, size_t bytes) {
    MYNN_CUDA_OK(cudaMemsetAsync(block, 0, sizeof(TpHeader), st));
    MYNN_CUDA_OK(cudaMemsetAsync(block + sizeof(TpHeader), 0xFF, bytes - sizeof(TpHeader), st));
    return MYNN_OK;
}

constexpr int kTpThreads = 1024;

// 16 bytes = four partial sums written by peer GPUs: a volatile load, so that every poll goes to L2
__device__ __forceinline__ uint4 ld_volatile_u4(const uint32_t *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// grid = rows.  limbs / ascale / w may be null (then only x is updated).  part = this rank's partial buffer `buf`.
template <typename T>
__global__ void __launch_bounds__(kTpThreads)
tp_reduce_norm_limbs_kernel(int8_t *limbs, float *ascale, T *x, const T *w, float eps, int D, TpHeader *hdr, uint32_t *part, int world,
                            int max_rows) {
    extern __shared__ __align__(16) float row_s[];
    __shared__ float red[40];
    pdl_trigger();  // the DequantMatMul that follows may set up and stream its first weight tiles while this kernel waits and sums
    const int m = blockIdx.x;
    // 1. read the partial rows of all ranks, re-reading a piece while any of its words is EMPTY (bounded), and put EMPTY back;
    // 2. add them in rank order; 3. residual add
    const size_t slot_stride = (size_t)max_rows * D;
    uint32_t *prow = part + (size_t)m * D;
    T *xrow = x + (size_t)m * D;
    float ss = 0.f;
    unsigned long long t0 = 0;
    bool gave_up = false;
    for (int i = 4 * threadIdx.x; i < D; i += 4 * kTpThreads) {
        float4 v[kTpMaxRanks];
#pragma unroll
        for (int r = 0; r < kTpMaxRanks; r++)
            if (r < world) {
                uint32_t *src = prow + (size_t)r * slot_stride + i;
                uint4 a;
                for (uint32_t it = 0;; it++) {
                    a = ld_volatile_u4(src);
                    if ((a.x != kTpEmpty && a.y != kTpEmpty && a.z != kTpEmpty && a.w != kTpEmpty) || gave_up) break;
                    if ((it & 63) == 63) {  // the clock is read rarely: the common case is no wait at all
                        const unsigned long long now = global_ns();
                        if (t0 == 0) t0 = now;
                        else if (now - t0 > d_wait_budget_ns) {
                            atomicExch(&hdr->status, 21);
                            gave_up = true;
                        }
                    }
                }
                *reinterpret_cast<uint4 *>(src) = make_uint4(kTpEmpty, kTpEmpty, kTpEmpty, kTpEmpty);  // ready for the next use
                v[r] = make_float4(__uint_as_float(a.x), __uint_as_float(a.y), __uint_as_float(a.z), __uint_as_float(a.w));
            }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < kTpMaxRanks; r++)
            if (r < world) {
                acc.x += v[r].x;
                acc.y += v[r].y;
                acc.z += v[r].z;
                acc.w += v[r].w;
            }
        const float s4[4] = {acc.x, acc.y, acc.z, acc.w};
        T xv[4];  // four residual elements with one access each way
        if constexpr (sizeof(T) == 2) *reinterpret_cast<uint2 *>(xv) = *reinterpret_cast<const uint2 *>(xrow + i);
        else *reinterpret_cast<float4 *>(xv) = *reinterpret_cast<const float4 *>(xrow + i);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float t = round_store<T>(to_f32<T>(xv[j]) + round_store<T>(s4[j]));
            xv[j] = from_f32<T>(t);
            row_s[i + j] = t;
            ss += t * t;
        }
        if constexpr (sizeof(T) == 2) *reinterpret_cast<uint2 *>(xrow + i) = *reinterpret_cast<const uint2 *>(xv);
        else *reinterpret_cast<float4 *>(xrow + i) = *reinterpret_cast<const float4 *>(xv);
    }
    if (w != nullptr) {
        ss = warp_sum(ss);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        if (threadIdx.x == 0) {
            float tot = 0.f;
            for (int i = 0; i < kTpThreads / 32; i++) tot += red[i];
            red[33] = 1.0f / sqrtf(tot / (float)D + eps);
        }
        __syncthreads();
        const float inv = red[33];
        float mx = 0.f;
        bool bad = false;
        for (int i = threadIdx.x; i < D; i += kTpThreads) {
            const float y = round_store<T>(row_s[i] * inv * to_f32<T>(w[i]));
            row_s[i] = y;
            bad |= !(fabsf(y) <= 3.0e38f);
            mx = fmaxf(mx, fabsf(y));
        }
        // block maximum -> power-of-two limb scale (|y| * sc < 2^22), as in the other limb producers
        mx = warp_max(mx);
        const unsigned anybad = __syncthreads_or(bad);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.f;
            for (int i = 0; i < kTpThreads / 32; i++) t = fmaxf(t, red[i]);
            int e = 0;
            if (t > 0.f) frexpf(t, &e);
            const float sc = t > 0.f ? ldexpf(1.0f, 22 - e) : 1.0f;
            red[32] = anybad ? 0.f : sc;
            ascale[m] = anybad ? __int_as_float(0x7fc00000) : 1.0f / sc;
        }
        __syncthreads();
        const float sc = red[32];
        uint32_t *l0 = reinterpret_cast<uint32_t *>(limbs + (size_t)(3 * m) * D);
        for (int gi = threadIdx.x; gi < (D >> 2); gi += kTpThreads) {
            uint32_t w0 = 0, w1 = 0, w2 = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                int A = sc == 0.f ? 0 : __float2int_rn(row_s[4 * gi + i] * sc);
                const int d0 = (int)(int8_t)(A & 0xFF);
                A = (A - d0) >> 8;
                const int d1 = (int)(int8_t)(A & 0xFF);
                A = (A - d1) >> 8;
                w0 |= (uint32_t)(d0 & 0xFF) << (8 * i);
                w1 |= (uint32_t)(d1 & 0xFF) << (8 * i);
                w2 |= (uint32_t)(A & 0xFF) << (8 * i);
            }
            l0[gi] = w0;
            l0[gi + (D >> 2)] = w1;
            l0[gi + 2 * (D >> 2)] = w2;
        }
    }
}

int launch_tp_gemm_push(cudaStream_t st, const TpPeers &peers, int buf, const void *act, const int8_t *wq, const float *scale, int M,
                        int N, int K, int act_dtype, void *workspace, size_t workspace_bytes, int skip_delivery) {
    if (buf != 0 && buf != 1) return fail(MYNN_E_ARG, "tp push: buffer %d", buf);
    if (M < 1 || M > peers.lay.max_rows || N != peers.lay.hidden)
        return fail(MYNN_E_ARG, "tp push: M=%d N=%d do not fit a group of %d rows x %d", M, N, peers.lay.max_rows, peers.lay.hidden);
    if (!i8_gemm_supported(M, N, K, wq, act_dtype, MYNN_F32))
        return fail(MYNN_E_UNSUPPORTED, "tp push: needs the tensor-core DequantMatMul (at most %d rows, K %% 16 == 0, aligned weights)", kI8MaxRows);
    I8Tp t;
    memset(&t, 0, sizeof t);
    t.mode = 1;
    t.world = peers.world;
    t.rank = peers.rank;
    t.max_rows = peers.lay.max_rows;
    for (int r = 0; r < peers.world; r++) t.part[r] = reinterpret_cast<uint32_t *>(peers.blocks[r] + peers.lay.part_off[buf]);
    t.skip = skip_delivery;
    return i8_gemm_launch_tp(st, nullptr, act, wq, scale, nullptr, M, N, K, act_dtype, MYNN_F32, workspace, workspace_bytes, &t, nullptr, nullptr);
}

int launch_tp_reduce_norm_limbs(cudaStream_t st, int dtype, const TpPeers &peers, int buf, void *workspace, size_t workspace_bytes,
                                void *x, const void *w, float eps, int M, bool after_push) {
    const int D = peers.lay.hidden;
    if (buf != 0 && buf != 1) return fail(MYNN_E_ARG, "tp reduce: buffer %d", buf);
    if (M < 1 || M > peers.lay.max_rows || D % 16) return fail(MYNN_E_UNSUPPORTED, "tp reduce: rows=%d D=%d not supported", M, D);
    if ((size_t)D * 4 > 200 * 1024) return fail(MYNN_E_UNSUPPORTED, "tp reduce: row of %d elements exceeds shared memory", D);
    int8_t *limbs = nullptr;
    float *ascale = nullptr;
    if (w != nullptr) {
        if (!workspace || workspace_bytes < i8_gemm_workspace_bytes(M, D) || (uintptr_t)workspace % 256)
            return fail(MYNN_E_ARG, "tp reduce: workspace too small or misaligned");
        ascale = (float *)((char *)workspace + 256);
        limbs = (int8_t *)workspace + 512;
    }
    char *own = peers.blocks[peers.rank];
    const size_t smem = (size_t)D * 4;
    MYNN_DISPATCH_DTYPE(dtype, T, {
        auto kern = tp_reduce_norm_limbs_kernel<T>;
        if (smem > 48 * 1024) MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        // after_push (the caller guarantees that the kernel in front of this one on the stream is the delivering DequantMatMul
        // of the same reduction): launched as a programmatic dependent of that grid, which triggers once its main loop is
        // over.  This kernel contains no griddepcontrol.wait because every value it needs from that grid is polled for, and
        // what else it reads (x) and writes (x, the limb workspace) that grid no longer touches by the time a row's values
        // are complete: a row is complete only when every CTA of the grid has finished its main loop and reached its epilogue.
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(M, 1, 1);
        cfg.blockDim = dim3(kTpThreads, 1, 1);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = after_push ? 1 : 0;
        MYNN_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, limbs, ascale, (T *)x, (const T *)w, eps, D, tp_header(own),
                                        reinterpret_cast<uint32_t *>(own + peers.lay.part_off[buf]), (int)peers.world, (int)peers.lay.max_rows));
    });
    MYNN_LAUNCH_OK("tp_reduce_norm_limbs_kernel");
    return MYNN_OK;
}

static int group_to_peers(const mynn_b200_tp_group *g, TpPeers &peers, const char *who) {
    if (!g) return fail(MYNN_E_ARG, "%s: null group", who);
    if (g->world < 1 || g->world > kTpMaxRanks || g->rank < 0 || g->rank >= g->world)
        return fail(MYNN_E_ARG, "%s: rank %d of %d (at most %d ranks)", who, g->rank, g->world, kTpMaxRanks);
    if (g->max_rows < 1 || g->max_rows > kI8MaxRows || g->hidden < 16 || g->hidden % 16)
        return fail(MYNN_E_ARG, "%s: a group holds 1..%d rows of a multiple of 16 elements (got %d x %d)", who, kI8MaxRows, g->max_rows, g->hidden);
    for (int r = 0; r < g->world; r++) {
        if (!g->blocks[r] || (uintptr_t)g->blocks[r] % 256) return fail(MYNN_E_ARG, "%s: block %d is null or not 256-byte aligned", who, r);
        peers.blocks[r] = (char *)g->blocks[r];
    }
    peers.rank = g->rank;
    peers.world = g->world;
    peers.lay = tp_layout(g->max_rows, g->hidden, g->world);
    return MYNN_OK;
}

}  // namespace mynn

using namespace mynn;

extern "C" size_t mynn_b200_tp_block_bytes(int max_rows, int hidden, int world) {
    if (max_rows < 1 || max_rows > kI8MaxRows || hidden < 16 || hidden % 16 || world < 1 || world > kTpMaxRanks) return 0;
    return tp_layout(max_rows, hidden, world).bytes;
}

extern "C" int mynn_b200_tp_block_init(void *stream, void *block, int max_rows, int hidden, int world) {
    const size_t bytes = mynn_b200_tp_block_bytes(max_rows, hidden, world);
    if (!bytes) return fail(MYNN_E_ARG, "tp_block_init: bad geometry (%d rows x %d, %d ranks)", max_rows, hidden, world);
    if (!block || (uintptr_t)block % 256) return fail(MYNN_E_ARG, "tp_block_init: block is null or not 256-byte aligned");
    return tp_block_init((cudaStream_t)stream, (char *)block, bytes);
}

extern "C" int mynn_b200_tp_dequant_matmul_push(void *stream, const mynn_b200_tp_group *group, int buffer, const void *act,
                                                const int8_t *wq, const float *scale, int M, int K, int act_dtype, void *workspace,
                                                size_t workspace_bytes) {
    TpPeers peers;
    if (int rc = group_to_peers(group, peers, "tp_dequant_matmul_push")) return rc;
    if (!act || !wq || !scale) return fail(MYNN_E_ARG, "tp_dequant_matmul_push: null pointer");
    if (!dtype_ok(act_dtype)) return fail(MYNN_E_ARG, "tp_dequant_matmul_push: bad dtype %d", act_dtype);
    int skip = 0, want = 2;
    if (g_inject_stall.compare_exchange_strong(want, 0)) skip = 1;
    return launch_tp_gemm_push((cudaStream_t)stream, peers, buffer, act, wq, scale, M, peers.lay.hidden, K, act_dtype, workspace, workspace_bytes, skip);
}

extern "C" int mynn_b200_tp_reduce_norm(void *stream, const mynn_b200_tp_group *group, int buffer, void *x, const void *weight, float eps,
                                        int M, int dtype, void *workspace, size_t workspace_bytes) {
    TpPeers peers;
    if (int rc = group_to_peers(group, peers, "tp_reduce_norm")) return rc;
    if (!x) return fail(MYNN_E_ARG, "tp_reduce_norm: null pointer");
    return launch_tp_reduce_norm_limbs((cudaStream_t)stream, dtype, peers, buffer, workspace, workspace_bytes, x, weight, eps, M, false);
}

extern "C" int mynn_b200_tp_check(void *stream, const mynn_b200_tp_group *group) {
    TpPeers peers;
    if (int rc = group_to_peers(group, peers, "tp_check")) return rc;
    MYNN_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
    int *word = &tp_header(peers.blocks[peers.rank])->status;
    int status = 0;
    MYNN_CUDA_OK(cudaMemcpy(&status, word, sizeof status, cudaMemcpyDeviceToHost));
    if (status) {
        MYNN_CUDA_OK(cudaMemset(word, 0, sizeof status));
        return fail(MYNN_E_COMM, "tensor-parallel reduction: a wait for a peer ran out of time (status %d)", status);
    }
    return MYNN_OK;
}
