// Tensor-parallel all-reduce fused with the operators around it, over NVLink peer memory (data flow: tp_fused.cuh).
//
// A row-parallel DequantMatMul (o_proj, down_proj) leaves an f32 partial sum [rows, hidden] on every rank.  The engine's
// schedule then needs: all-reduce(sum) -> round -> residual add -> RMSNorm -> (here) activation limbs for the next
// DequantMatMul on every rank (its AllReduce operator, src/graph/operator.rs, sums f32 in rank order:
// crates/comm/src/uds.rs:106-116).  Here the reduction is a reduce-scatter by rows that the producing GEMM performs with
// peer STORES from its epilogue, one kernel per rank that finishes the rows it owns, and an all-gather of the finished
// limb rows, again by peer stores, that the consuming GEMM waits for while its weights are already streaming.
//
// Ordering.  Data stores to a peer are followed by a CTA barrier, one system-scope fence and an increment of a counter
// in the peer's header; the reader polls the counter with acquire loads and only then touches the data (through L2: the
// lines were written by another GPU).  A buffer is only rewritten after its readers are provably done: a rank delivers
// partial sums for reduction j+1 only after its column-parallel GEMM has received the limb rows of reduction j from every
// rank, i.e. after every rank has finished reading the partial sums of reduction j; and a rank delivers limb rows of
// reduction j+1 to a peer only after that peer's row-parallel GEMM, which runs behind the reader of reduction j's limb rows
// in the peer's stream, has delivered its partial sums.
//
// Every wait is bounded (MYNN_OPT_WAIT_BUDGET_US, default 2 s): on expiry the kernel records a status (21 here, 22 in the
// GEMM's wait for limb rows), goes on with what it has, still delivers and signals, and returns; the host reports
// MYNN_E_COMM at its next check.  A lost peer therefore never hangs a GPU.
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
    l.rows_cap = (max_rows + world - 1) / world;
    l.nc = i8_gemm_limb_rows(max_rows);
    size_t off = sizeof(TpHeader);
    const size_t part = up256((size_t)world * l.rows_cap * hidden * sizeof(uint2));  // {value, tag} words
    l.part_off[0] = off;
    off += part;
    l.part_off[1] = off;
    off += part;
    l.limb_off = off;
    off += up256((size_t)l.nc * hidden);
    l.ascale_off = off;
    off += up256((size_t)max_rows * sizeof(float));
    l.bytes = off;
    return l;
}

struct TpReduceParams {
    char *blocks[kTpMaxRanks];
    size_t part_off, limb_off, ascale_off;
    int rank, world, rows_cap, buf, M, D, skip_signal;
    float eps;
};

constexpr int kTpThreads = 1024;

// 16 bytes = two {value, tag} words written by a peer GPU: a volatile load, so that every poll goes to L2
__device__ __forceinline__ uint4 ld_volatile_u4(const uint2 *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// grid = max(rows this rank owns, 1).  CTA j finishes row m = rank + j * world.  w may be null (then only x is updated and no
// limbs are delivered; the counters still advance).
template <typename T>
__global__ void __launch_bounds__(kTpThreads) tp_reduce_norm_gather_kernel(T *x, const T *w, const TpReduceParams p) {
    extern __shared__ __align__(16) float row_s[];
    __shared__ float red[40];
    TpHeader *hdr = tp_header(p.blocks[p.rank]);
    const int D = p.D;
    const int m = p.rank + (int)blockIdx.x * p.world;
    const bool have_row = m < p.M;
    // the tag the partial sums of THIS reduction carry (the previous reduction on this buffer was number part_tag)
    const uint32_t tag = *(volatile uint32_t *)&hdr->part_tag[p.buf] + 1u;
    if (have_row) {
        // 1. + 2. read the partial rows of all ranks (8-byte {value, tag} words in this rank's own memory, written by the peers'
        // GEMM epilogues), re-reading a word until it carries this reduction's tag (bounded); add them in rank order;
        // 3. residual add
        const uint2 *part = reinterpret_cast<const uint2 *>(p.blocks[p.rank] + p.part_off) + (size_t)blockIdx.x * D;
        const size_t slot_stride = (size_t)p.rows_cap * D;
        T *xrow = x + (size_t)m * D;
        float ss = 0.f;
        unsigned long long t0 = 0;
        bool gave_up = false;
        for (int i = 4 * threadIdx.x; i < D; i += 4 * kTpThreads) {
            float4 v[kTpMaxRanks];
#pragma unroll
            for (int r = 0; r < kTpMaxRanks; r++)
                if (r < p.world) {
                    const uint2 *src = part + (size_t)r * slot_stride + i;
                    uint4 a, b;
                    for (uint32_t it = 0;; it++) {
                        a = ld_volatile_u4(src);
                        b = ld_volatile_u4(src + 2);
                        if ((a.y == tag && a.w == tag && b.y == tag && b.w == tag) || gave_up) break;
                        if ((it & 63) == 63) {  // the clock is read rarely: the common case is no wait at all
                            const unsigned long long now = global_ns();
                            if (t0 == 0) t0 = now;
                            else if (now - t0 > d_wait_budget_ns) {
                                atomicExch(&hdr->status, 21);
                                gave_up = true;
                            }
                        }
                    }
                    v[r] = make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(b.x), __uint_as_float(b.z));
                }
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int r = 0; r < kTpMaxRanks; r++)
                if (r < p.world) {
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
                red[33] = 1.0f / sqrtf(tot / (float)D + p.eps);
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
                red[34] = anybad ? __int_as_float(0x7fc00000) : 1.0f / sc;
            }
            __syncthreads();
            const float sc = red[32];
            if (!p.skip_signal) {
                // 4. deliver the three limb rows and the row scale to every rank (peer stores; this rank's own copy too)
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
#pragma unroll
                    for (int r = 0; r < kTpMaxRanks; r++)
                        if (r < p.world) {
                            uint32_t *l0 = reinterpret_cast<uint32_t *>(p.blocks[r] + p.limb_off + (size_t)(3 * m) * D);
                            l0[gi] = w0;
                            l0[gi + (D >> 2)] = w1;
                            l0[gi + 2 * (D >> 2)] = w2;
                        }
                }
                if (threadIdx.x < p.world)
                    reinterpret_cast<float *>(p.blocks[threadIdx.x] + p.ascale_off)[m] = red[34];
            }
        }
    }
    // every store of this CTA is ordered before the increments: CTA barrier, then a release increment per destination (the
    // lanes of one warp in parallel: each release costs a system-scope fence)
    __syncthreads();
    if (have_row && w != nullptr && !p.skip_signal && threadIdx.x < p.world)
        red_release_sys_add_u32(&tp_header(p.blocks[threadIdx.x])->gather_cnt, 1u);
    // the last CTA to finish records what the counters must reach for the kernels that follow
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&hdr->ticket, 1u) == gridDim.x - 1) {
            hdr->ticket = 0u;
            hdr->part_tag[p.buf] = tag;
            if (w != nullptr) hdr->gather_expected += (uint32_t)p.M;
            __threadfence();
        }
    }
}

static void fill_i8tp(I8Tp &t, const TpPeers &peers, int mode, int buf) {
    memset(&t, 0, sizeof t);
    t.mode = mode;
    t.world = peers.world;
    t.rank = peers.rank;
    t.rows_cap = peers.lay.rows_cap;
    for (int r = 0; r < peers.world; r++) {
        t.part[r] = reinterpret_cast<uint2 *>(peers.blocks[r] + peers.lay.part_off[buf]);
    }
    TpHeader *own = tp_header(peers.blocks[peers.rank]);
    t.part_tag = &own->part_tag[buf];
    t.gather_cnt = &own->gather_cnt;
    t.gather_expected = &own->gather_expected;
    t.status = &own->status;
}

int launch_tp_gemm_scatter(cudaStream_t st, const TpPeers &peers, int buf, const void *act, const int8_t *wq, const float *scale,
                           int M, int N, int K, int act_dtype, void *workspace, size_t workspace_bytes) {
    if (buf != 0 && buf != 1) return fail(MYNN_E_ARG, "tp scatter: buffer %d", buf);
    if (M < 1 || M > peers.lay.max_rows || N != peers.lay.hidden)
        return fail(MYNN_E_ARG, "tp scatter: M=%d N=%d do not fit a group of %d rows x %d", M, N, peers.lay.max_rows, peers.lay.hidden);
    if (!i8_gemm_supported(M, N, K, wq, act_dtype, MYNN_F32))
        return fail(MYNN_E_UNSUPPORTED, "tp scatter: needs the tensor-core DequantMatMul (at most %d rows, K %% 16 == 0, aligned weights)", kI8MaxRows);
    I8Tp t;
    fill_i8tp(t, peers, 1, buf);
    return i8_gemm_launch_tp(st, nullptr, act, wq, scale, nullptr, M, N, K, act_dtype, MYNN_F32, workspace, workspace_bytes, &t, nullptr, nullptr);
}

int launch_tp_gemm_gathered(cudaStream_t st, const TpPeers &peers, void *out, const int8_t *wq, const void *scale, int M, int N,
                            int out_dtype, void *workspace, size_t workspace_bytes) {
    const int K = peers.lay.hidden;
    if (M < 1 || M > peers.lay.max_rows) return fail(MYNN_E_ARG, "tp gathered: M=%d exceeds the group's %d rows", M, peers.lay.max_rows);
    if (!i8_gemm_supported(M, N, K, wq, MYNN_BF16, out_dtype))
        return fail(MYNN_E_UNSUPPORTED, "tp gathered: needs the tensor-core DequantMatMul (K %% 16 == 0, aligned weights)");
    I8Tp t;
    fill_i8tp(t, peers, 2, 0);
    char *own = peers.blocks[peers.rank];
    return i8_gemm_launch_tp(st, out, nullptr, wq, scale, nullptr, M, N, K, MYNN_BF16, out_dtype, workspace, workspace_bytes, &t,
                             reinterpret_cast<const int8_t *>(own + peers.lay.limb_off),
                             reinterpret_cast<const float *>(own + peers.lay.ascale_off));
}

int launch_tp_reduce_norm_gather(cudaStream_t st, int dtype, const TpPeers &peers, int buf, void *x, const void *w, float eps, int M,
                                 int skip_signal) {
    const int D = peers.lay.hidden;
    if (buf != 0 && buf != 1) return fail(MYNN_E_ARG, "tp reduce: buffer %d", buf);
    if (M < 1 || M > peers.lay.max_rows || D % 16) return fail(MYNN_E_UNSUPPORTED, "tp reduce: rows=%d D=%d not supported", M, D);
    if ((size_t)D * 4 > 200 * 1024) return fail(MYNN_E_UNSUPPORTED, "tp reduce: row of %d elements exceeds shared memory", D);
    TpReduceParams p;
    for (int r = 0; r < kTpMaxRanks; r++) p.blocks[r] = r < peers.world ? peers.blocks[r] : nullptr;
    p.part_off = peers.lay.part_off[buf];
    p.limb_off = peers.lay.limb_off;
    p.ascale_off = peers.lay.ascale_off;
    p.rank = peers.rank;
    p.world = peers.world;
    p.rows_cap = peers.lay.rows_cap;
    p.buf = buf;
    p.M = M;
    p.D = D;
    p.skip_signal = skip_signal;
    p.eps = eps;
    const int own_rows = peers.rank < M ? (M - peers.rank + peers.world - 1) / peers.world : 0;
    const int grid = own_rows > 0 ? own_rows : 1;
    const size_t smem = (size_t)D * 4;
    MYNN_DISPATCH_DTYPE(dtype, T, {
        auto kern = tp_reduce_norm_gather_kernel<T>;
        if (smem > 48 * 1024) MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<grid, kTpThreads, smem, st>>>((T *)x, (const T *)w, p);
    });
    MYNN_LAUNCH_OK("tp_reduce_norm_gather_kernel");
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

extern "C" int mynn_b200_tp_dequant_matmul_scatter(void *stream, const mynn_b200_tp_group *group, int buffer, const void *act,
                                                   const int8_t *wq, const float *scale, int M, int K, int act_dtype,
                                                   void *workspace, size_t workspace_bytes) {
    TpPeers peers;
    if (int rc = group_to_peers(group, peers, "tp_dequant_matmul_scatter")) return rc;
    if (!act || !wq || !scale) return fail(MYNN_E_ARG, "tp_dequant_matmul_scatter: null pointer");
    if (!dtype_ok(act_dtype)) return fail(MYNN_E_ARG, "tp_dequant_matmul_scatter: bad dtype %d", act_dtype);
    return launch_tp_gemm_scatter((cudaStream_t)stream, peers, buffer, act, wq, scale, M, peers.lay.hidden, K, act_dtype, workspace, workspace_bytes);
}

extern "C" int mynn_b200_tp_reduce_norm_gather(void *stream, const mynn_b200_tp_group *group, int buffer, void *x, const void *weight,
                                               float eps, int M, int dtype) {
    TpPeers peers;
    if (int rc = group_to_peers(group, peers, "tp_reduce_norm_gather")) return rc;
    if (!x) return fail(MYNN_E_ARG, "tp_reduce_norm_gather: null pointer");
    int skip = 0;
    {
        int want = 2;
        if (g_inject_stall.compare_exchange_strong(want, 0)) skip = 1;
    }
    return launch_tp_reduce_norm_gather((cudaStream_t)stream, dtype, peers, buffer, x, weight, eps, M, skip);
}

extern "C" int mynn_b200_tp_dequant_matmul_gathered(void *stream, const mynn_b200_tp_group *group, void *out, const int8_t *wq,
                                                    const void *scale, int M, int N, int out_dtype, void *workspace,
                                                    size_t workspace_bytes) {
    TpPeers peers;
    if (int rc = group_to_peers(group, peers, "tp_dequant_matmul_gathered")) return rc;
    if (!out || !wq || !scale) return fail(MYNN_E_ARG, "tp_dequant_matmul_gathered: null pointer");
    if (!dtype_ok(out_dtype)) return fail(MYNN_E_ARG, "tp_dequant_matmul_gathered: bad dtype %d", out_dtype);
    return launch_tp_gemm_gathered((cudaStream_t)stream, peers, out, wq, scale, M, N, out_dtype, workspace, workspace_bytes);
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
