// Shared helpers for the sm_100a decode-path kernels: status/error plumbing, storage-dtype
// conversions and small warp utilities.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/mynn_b200.h"

namespace mynn {

// ---- host-side status ----------------------------------------------------------------------
void set_error(const char *fmt, ...);
extern std::atomic<long long> g_launches;

inline int fail(int code, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
inline int fail(int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    set_error("%s", buf);
    return code;
}

#define MYNN_CUDA_OK(expr)                                                                                 \
    do {                                                                                                   \
        cudaError_t e__ = (expr);                                                                          \
        if (e__ != cudaSuccess)                                                                            \
            return mynn::fail(MYNN_E_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, \
                              __LINE__);                                                                   \
    } while (0)

// Call after every kernel launch: counts it and turns a launch error into a status code.
#define MYNN_LAUNCH_OK(name)                                                                          \
    do {                                                                                              \
        mynn::g_launches.fetch_add(1, std::memory_order_relaxed);                                     \
        cudaError_t e__ = cudaGetLastError();                                                         \
        if (e__ != cudaSuccess)                                                                       \
            return mynn::fail(MYNN_E_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e__)); \
    } while (0)

inline size_t dtype_size(int dt) { return dt == MYNN_F32 ? 4 : 2; }
inline bool dtype_ok(int dt) { return dt == MYNN_F32 || dt == MYNN_BF16 || dt == MYNN_F16; }

// ---- device-side storage conversions ---------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// One RoPE pair (xl, xh = the elements half a head apart) with the roundings of the engine's CPU kernel: two products and
// one sum, each rounded to f32, never contracted into a fused multiply-add.  Every kernel that rotates uses these, so the
// stand-alone RoPE kernel and the rotation inside the decode attention kernel give the same bits.
__device__ __forceinline__ float rope_low(float xl, float xh, float c, float s) { return __fsub_rn(__fmul_rn(xl, c), __fmul_rn(xh, s)); }
__device__ __forceinline__ float rope_high(float xl, float xh, float c, float s) { return __fadd_rn(__fmul_rn(xh, c), __fmul_rn(xl, s)); }

// One store point: round to storage dtype and come back to f32.
template <typename T>
__device__ __forceinline__ float round_store(float v) { return to_f32<T>(from_f32<T>(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---- programmatic dependent launch -----------------------------------------------------------------------------
// Only the DequantMatMul kernels are launched with the programmatic-stream-serialization attribute: they have work that
// does not depend on their predecessor (barrier set-up, streaming the first weight tiles) and order themselves with
// pdl_wait() before they touch anything an earlier kernel produces.  The other kernels of the decode chain are plain
// launches; their pdl_trigger() / pdl_wait() are no-ops there and only matter when such a kernel is the predecessor of a
// DequantMatMul (pdl_trigger() lets that kernel be scheduled early).  Giving every kernel of the chain the attribute was
// measured three times and rejected: without an early trigger in the GEMM it changed nothing; with a trigger at the GEMM's start
// the kernels two and three places ahead became resident early and took registers and shared memory from the running kernel
// (step 4.63 -> 5.31 ms); with a trigger after the GEMM's main loop the gaps stayed as they were (the glue kernels' own run
// time, not their launch, fills them) and the o_proj CTAs that became resident under the attention kernel slowed it by 5-40 %.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Library options (mynn_b200_set_option).
extern int g_ksplit_override;            // forced cluster K split of the DequantMatMul kernels, 0 = automatic
extern int g_prefill_attention_mode;     // see MYNN_OPT_PREFILL_ATTENTION
extern int g_fuse_rope;                  // see MYNN_OPT_FUSE_ROPE
extern int g_decode_ring;                // see MYNN_OPT_DECODE_RING
extern std::atomic<int> g_inject_stall;  // see MYNN_OPT_INJECT_STALL; consumed by the next launch it applies to

// A plain launch through cudaLaunchKernelEx (no attributes); the name says which kernels belong to the decode chain.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cfg.attrs = nullptr;
    cfg.numAttrs = 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Dispatch a launcher template over the three storage dtypes.
#define MYNN_DISPATCH_DTYPE(dt, T, ...)                       \
    switch (dt) {                                             \
        case MYNN_F32: { using T = float; __VA_ARGS__; } break;          \
        case MYNN_BF16: { using T = __nv_bfloat16; __VA_ARGS__; } break; \
        case MYNN_F16: { using T = __half; __VA_ARGS__; } break;         \
        default: return mynn::fail(MYNN_E_ARG, "bad dtype %d", dt);      \
    }

}  // namespace mynn
