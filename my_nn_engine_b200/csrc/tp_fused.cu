// Tensor-parallel all-reduce fused with the operators that consume it, over NVLink peer memory.
//
// A row-parallel DequantMatMul (o_proj, down_proj) leaves an f32 partial sum [rows, hidden] on every rank.  The engine's
// schedule then needs: all-reduce(sum) -> round -> residual add -> RMSNorm -> (here) activation limbs for the next
// DequantMatMul.  Instead of a collective library call followed by separate kernels, ONE kernel per rank
//   1. tells every peer that its own partial sums are complete (a release store of the step number into the peer's
//      flag array) and waits, with a time limit, until every peer has said the same;
//   2. reads the partial sums of ALL ranks straight from their memory (plain peer loads over NVLink/NVSwitch, no
//      multicast) and adds them in rank order in f32 -- every rank computes the identical sum;
//   3. finishes the row: x = round(x + round(sum)), y = round(RMSNorm(x) * w), limbs of y.
// The messages are small (512 KB at batch 32), so the one-shot pattern (every rank reads everything) beats a
// reduce-scatter/all-gather pair, which would need a second cross-GPU barrier.
//
// Buffers: two partial-sum buffers are used alternately (attention block / MLP block).  A rank overwrites a buffer only
// after it has passed the barrier of the following reduction, which every peer reaches only after it has finished
// reading that buffer, so no reader can be overtaken.
// The wait is bounded (2 s): on expiry the kernel records status 21 and carries on, so the GPU never hangs on a lost
// peer; the host sees the status at its next check.
#include "common.cuh"
#include "i8_gemm.cuh"
#include "tcgen05.cuh"
#include "tp_fused.cuh"

namespace mynn {

MYNN_DEFINE_WAIT_BUDGET_SETTER(tp_fused)

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float *p) {  // system-scope load: never served from a stale L1 line
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long tp_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

constexpr int kTpThreads = 1024;

// grid = rows.  limbs / ascale / w may be null (then only x is updated: the reduction after the last layer).
template <typename T>
__global__ void __launch_bounds__(kTpThreads)
tp_reduce_norm_limbs_kernel(int8_t *limbs, float *ascale, T *x, const T *w, float eps, int D, int buf, const TpPeers peers) {
    extern __shared__ __align__(16) float row_s[];
    __shared__ float red[40];
    TpLocal *loc = peers.local;
    const uint32_t target = *(volatile uint32_t *)&loc->epoch + 1u;  // the epoch only changes when this kernel ends
    // 1. announce and wait
    if (blockIdx.x == 0 && threadIdx.x < peers.world)
        st_release_sys(&peers.remote[threadIdx.x]->flags[peers.rank], target);
    if (threadIdx.x < peers.world) {
        const unsigned long long t0 = tp_now_ns();
        while ((int)(ld_acquire_sys(&loc->flags[threadIdx.x]) - target) < 0) {
            __nanosleep(100);
            if (tp_now_ns() - t0 > d_wait_budget_ns) {
                atomicExch(&loc->status, 21);
                break;
            }
        }
    }
    __syncthreads();
    // 2. sum the partial rows of all ranks in rank order, 3. residual add
    const int m = blockIdx.x;
    const size_t base = (size_t)m * D;
    float ss = 0.f;
    for (int i = 4 * threadIdx.x; i < D; i += 4 * kTpThreads) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float4 part[8];
#pragma unroll
        for (int r = 0; r < 8; r++)
            if (r < peers.world) part[r] = ld_peer_f4(tp_part(peers.remote[r], peers.part_off[buf]) + base + i);
#pragma unroll
        for (int r = 0; r < 8; r++)
            if (r < peers.world) {
                acc.x += part[r].x;
                acc.y += part[r].y;
                acc.z += part[r].z;
                acc.w += part[r].w;
            }
        const float s4[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float v = round_store<T>(to_f32<T>(x[base + i + j]) + round_store<T>(s4[j]));
            x[base + i + j] = from_f32<T>(v);
            row_s[i + j] = v;
            ss += v * v;
        }
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
        uint32_t *l1 = reinterpret_cast<uint32_t *>(limbs + (size_t)(3 * m + 1) * D);
        uint32_t *l2 = reinterpret_cast<uint32_t *>(limbs + (size_t)(3 * m + 2) * D);
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
            l1[gi] = w1;
            l2[gi] = w2;
        }
    }
    // the last CTA to finish advances the epoch for the next reduction
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&loc->ticket, 1u) == gridDim.x - 1) {
            loc->ticket = 0u;
            __threadfence();
            *(volatile uint32_t *)&loc->epoch = target;
        }
    }
}

int launch_tp_reduce_norm_limbs(cudaStream_t st, int dtype, const TpPeers &peers, int buf, void *workspace,
                                size_t workspace_bytes, void *x, const void *w, float eps, int rows, int D) {
    if (rows < 1 || rows > kI8MaxRows || D % 16) return fail(MYNN_E_UNSUPPORTED, "tp reduce: rows=%d D=%d not supported", rows, D);
    if ((size_t)D * 4 > 200 * 1024) return fail(MYNN_E_UNSUPPORTED, "tp reduce: row of %d elements exceeds shared memory", D);
    int8_t *limbs = nullptr;
    float *ascale = nullptr;
    if (w != nullptr) {
        if (!workspace || workspace_bytes < i8_gemm_workspace_bytes(rows, D) || (uintptr_t)workspace % 256)
            return fail(MYNN_E_ARG, "tp reduce: workspace too small or misaligned");
        ascale = (float *)((char *)workspace + 256);
        limbs = (int8_t *)workspace + 512;
    }
    const size_t smem = (size_t)D * 4;
    MYNN_DISPATCH_DTYPE(dtype, T, {
        auto kern = tp_reduce_norm_limbs_kernel<T>;
        if (smem > 48 * 1024) MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<rows, kTpThreads, smem, st>>>(limbs, ascale, (T *)x, (const T *)w, eps, D, buf, peers);
    });
    MYNN_LAUNCH_OK("tp_reduce_norm_limbs_kernel");
    return MYNN_OK;
}

}  // namespace mynn
