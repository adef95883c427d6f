// W8A8 operators of the engine: DynamicQuantizeLinear (activations -> int8/uint8 + scale + zero point) and
// QuantizedMatMul (int8 x int8 with per-row / per-tensor lhs scale and per-channel rhs scale).
//
// DynamicQuantizeLinear follows the engine's arithmetic so that the bytes match it:
//   symmetric, per row    CPU kernel (src/codegen/cpu/kernels/dynquant_i8.rs:13-37): sc = amax / 127 (1 for an all-zero
//                         row), inv = 1 / sc, y = round-half-away(x * inv) clamped to [-127, 127];
//   the other variants    CUDA kernel (src/codegen/cuda/cpp/dynamic_quantize_linear.cuh), the only backend that has
//                         them: y = nearbyint(x / scale) + zero_point; symmetric scale = max|x| / 127; asymmetric
//                         (uint8) min/max widened to contain 0, scale = (max - min) / 255 (1 if 0),
//                         zero_point = clamp(nearbyint(-min / scale), 0, 255).
// One CTA per slice (row, or the whole tensor), as in the engine.
//
// QuantizedMatMul: out = (int32 dot) * lhs_scale * rhs_scale (src/codegen/cpu/kernels/qgemv_i8i8.rs:59-78).  The fast path
// is the persistent tcgen05 int8 kernel of i8_gemm_prefill.cu with one accumulator column per lhs row; shapes it does
// not take (K not a multiple of 16, unaligned operands) run on a plain one-warp-per-output kernel.
#include "common.cuh"
#include "i8_gemm.cuh"

namespace mynn {

constexpr int kDqThreads = 1024;

__device__ __forceinline__ float block_reduce(float v, float *buf, bool is_max) {
    // reduce over a 1024-thread block; result valid in every thread
    v = is_max ? warp_max(v) : -warp_max(-v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) buf[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = buf[0];
    for (int i = 1; i < kDqThreads / 32; i++) r = is_max ? fmaxf(r, buf[i]) : fminf(r, buf[i]);
    return r;
}

// MODE 0: symmetric, CPU rounding (per-row slices); 1: symmetric, CUDA rounding (per-tensor); 2: asymmetric (uint8)
template <typename T, int MODE>
__global__ void __launch_bounds__(kDqThreads) dyn_quantize_kernel(void *y_, T *y_scale, void *y_zp_, const T *x, long long inner) {
    __shared__ float buf[kDqThreads / 32];
    const long long slice = blockIdx.x;
    const T *xs = x + slice * inner;
    float amax = 0.f, mn = INFINITY, mx = -INFINITY;
    for (long long i = threadIdx.x; i < inner; i += kDqThreads) {
        const float v = to_f32<T>(xs[i]);
        if (MODE == 2) {
            mn = fminf(mn, v);
            mx = fmaxf(mx, v);
        } else {
            amax = fmaxf(amax, fabsf(v));
        }
    }
    if (MODE == 2) {
        mn = fminf(block_reduce(mn, buf, false), 0.f);
        mx = fmaxf(block_reduce(mx, buf, true), 0.f);
        float scale = __fdiv_rn(mx - mn, 255.0f);
        if (scale == 0.f) scale = 1.0f;
        const int zp = max(0, min(255, (int)nearbyintf(__fdiv_rn(-mn, scale))));
        if (threadIdx.x == 0) {
            y_scale[slice] = from_f32<T>(scale);
            reinterpret_cast<uint8_t *>(y_zp_)[slice] = (uint8_t)zp;
        }
        uint8_t *ys = reinterpret_cast<uint8_t *>(y_) + slice * inner;
        for (long long i = threadIdx.x; i < inner; i += kDqThreads) {
            const int q = (int)nearbyintf(__fdiv_rn(to_f32<T>(xs[i]), scale)) + zp;
            ys[i] = (uint8_t)max(0, min(255, q));
        }
    } else {
        amax = block_reduce(amax, buf, true);
        int8_t *ys = reinterpret_cast<int8_t *>(y_) + slice * inner;
        if (MODE == 0) {
            const float sc = amax > 0.f ? __fdiv_rn(amax, 127.0f) : 1.0f;
            const float inv = __fdiv_rn(1.0f, sc);
            if (threadIdx.x == 0) {
                y_scale[slice] = from_f32<T>(sc);
                reinterpret_cast<int8_t *>(y_zp_)[slice] = 0;
            }
            for (long long i = threadIdx.x; i < inner; i += kDqThreads)
                ys[i] = (int8_t)fmaxf(-127.f, fminf(127.f, roundf(__fmul_rn(to_f32<T>(xs[i]), inv))));
        } else {
            const float scale = __fdiv_rn(amax, 127.0f);
            if (threadIdx.x == 0) {
                y_scale[slice] = from_f32<T>(scale);
                reinterpret_cast<int8_t *>(y_zp_)[slice] = 0;
            }
            for (long long i = threadIdx.x; i < inner; i += kDqThreads) {
                // an all-zero tensor has scale 0: its bytes are 0 (the division would give NaN)
                const int q = scale > 0.f ? (int)nearbyintf(__fdiv_rn(to_f32<T>(xs[i]), scale)) : 0;
                ys[i] = (int8_t)max(-127, min(127, q));
            }
        }
    }
}

// one warp per output element group: warp (m, n-block of 32): lane handles n = n0 + lane, loops K bytes 4 at a time
template <typename T>
__global__ void quantized_matmul_generic_kernel(T *out, const int8_t *lhs, const T *lhs_scale, int ls_stride, const int8_t *rhs,
                                                const T *rhs_scale, int M, int N, int K) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x, m = blockIdx.y;
    if (n >= N) return;
    const int8_t *a = lhs + (size_t)m * K, *w = rhs + (size_t)n * K;
    int acc = 0;
    for (int k = 0; k < K; k++) acc += (int)a[k] * (int)w[k];
    const float v = __fmul_rn(__fmul_rn((float)acc, to_f32<T>(lhs_scale[(size_t)m * ls_stride])), to_f32<T>(rhs_scale[n]));
    out[(size_t)m * N + n] = from_f32<T>(v);
}

}  // namespace mynn

using namespace mynn;

extern "C" int mynn_b200_dynamic_quantize_linear(void *stream, void *y, void *y_scale, void *y_zero_point, const void *x,
                                                 long long slices, long long inner, int symmetric, int per_row, int dtype) {
    if (slices < 0 || inner < 0) return fail(MYNN_E_ARG, "dynamic_quantize_linear: bad shape");
    if (!dtype_ok(dtype)) return fail(MYNN_E_ARG, "dynamic_quantize_linear: bad dtype %d", dtype);
    if (slices == 0 || inner == 0) return MYNN_OK;
    if (!y || !y_scale || !y_zero_point || !x) return fail(MYNN_E_ARG, "dynamic_quantize_linear: null pointer");
    long long blocks = slices, len = inner;
    if (!per_row) {  // one slice covering the whole tensor
        blocks = 1;
        len = slices * inner;
    }
    if (blocks > 0x7fffffffLL) return fail(MYNN_E_UNSUPPORTED, "dynamic_quantize_linear: too many slices");
    cudaStream_t st = (cudaStream_t)stream;
    MYNN_DISPATCH_DTYPE(dtype, T, {
        if (!symmetric)
            dyn_quantize_kernel<T, 2><<<(unsigned)blocks, kDqThreads, 0, st>>>(y, (T *)y_scale, y_zero_point, (const T *)x, len);
        else if (per_row)
            dyn_quantize_kernel<T, 0><<<(unsigned)blocks, kDqThreads, 0, st>>>(y, (T *)y_scale, y_zero_point, (const T *)x, len);
        else
            dyn_quantize_kernel<T, 1><<<(unsigned)blocks, kDqThreads, 0, st>>>(y, (T *)y_scale, y_zero_point, (const T *)x, len);
    });
    MYNN_LAUNCH_OK("dyn_quantize_kernel");
    return MYNN_OK;
}

extern "C" size_t mynn_b200_quantized_matmul_workspace_bytes(int M, int N, int K) {
    (void)M;
    (void)N;
    (void)K;
    return 256;
}

extern "C" int mynn_b200_quantized_matmul(void *stream, void *out, const int8_t *lhs, const void *lhs_scale,
                                          int lhs_scale_per_row, const int8_t *rhs, const void *rhs_scale, int M, int N, int K,
                                          int dtype, void *workspace, size_t workspace_bytes) {
    if (M < 0 || N < 0 || K < 0) return fail(MYNN_E_ARG, "quantized_matmul: bad shape");
    if (!dtype_ok(dtype)) return fail(MYNN_E_ARG, "quantized_matmul: bad dtype %d", dtype);
    if (M == 0 || N == 0) return MYNN_OK;
    if (!out || !lhs_scale || !rhs_scale || (K > 0 && (!lhs || !rhs))) return fail(MYNN_E_ARG, "quantized_matmul: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    if (workspace && i8_w8a8_supported(M, N, K, lhs, rhs))
        return i8_w8a8_launch(st, out, lhs, lhs_scale, lhs_scale_per_row, rhs, rhs_scale, M, N, K, dtype, workspace, workspace_bytes);
    if (M > 65535) return fail(MYNN_E_UNSUPPORTED, "quantized_matmul: %d rows exceed the plain kernel's grid", M);
    MYNN_DISPATCH_DTYPE(dtype, T, {
        quantized_matmul_generic_kernel<T><<<dim3((N + 127) / 128, M), 128, 0, st>>>((T *)out, lhs, (const T *)lhs_scale, lhs_scale_per_row ? 1 : 0,
                                                                                   rhs, (const T *)rhs_scale, M, N, K);
    });
    MYNN_LAUNCH_OK("quantized_matmul_generic_kernel");
    return MYNN_OK;
}
