/*
 * CPU oracle in plain C: a restatement of the reference's CPU (LLVM) kernels for the LLM decode
 * path.  TEST INFRASTRUCTURE ONLY: it is the checker for tests, for the smoke test and for the
 * CPU-baseline leg of the benchmark.  Nothing the product ships links or calls it.
 *
 * Parity status: the reference (Rust + LLVM 18 + BLAS) cannot be built in this environment, so
 * these functions are pinned against the reference's own golden vectors through the Python
 * tests; M=1 int8 decode beyond the reference's 3x8 toy fixture is pinned by restatement only.
 *
 * Paths in comments are relative to the reference root.  bf16 tensors are uint16 bit patterns.
 * Build: see oracle/Makefile (gcc -O3 -fopenmp -shared).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* bits << 16 reinterpret (src/codegen/cpu/translator.rs:162-172) */
static inline float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round to nearest even, no NaN special case (src/codegen/cpu/translator.rs:174-204) */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    uint32_t bias = 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)((u + bias) >> 16);
}

enum { ORC_F32 = 0, ORC_BF16 = 1 };

static inline float load_elem(const void *p, int64_t i, int dtype) {
    return dtype == ORC_BF16 ? bf16_to_f32(((const uint16_t *)p)[i]) : ((const float *)p)[i];
}
static inline void store_elem(void *p, int64_t i, int dtype, float v) {
    if (dtype == ORC_BF16)
        ((uint16_t *)p)[i] = f32_to_bf16(v);
    else
        ((float *)p)[i] = v;
}

/*
 * DequantMatMul, fused decode form: out[m,n] = scale[n] * sum_k act[m,k] * f32(wq[n,k]).
 * The reference uses this loop nest for M == 1 (src/codegen/cpu/translator.rs:3208-3313) and
 * splits the N rows over OpenMP threads (omp_for_static, src/codegen/cpu/translator.rs:3122-3206).
 * The reference tags the multiply-add fast-math, so the summation order is free; this loop is
 * left to the compiler's vectoriser in the same spirit.  Storage dtype of act / scale+out given
 * separately, as the operator allows (out dtype == scale dtype, src/transform/shape.rs:326-345).
 */
void orc_dequant_matmul_fused(void *out, const void *act, const int8_t *wq, const void *scale,
                              int64_t M, int64_t N, int64_t K, int act_dtype, int out_dtype, int use_omp) {
    float *a = (float *)malloc(sizeof(float) * (size_t)(M * K));
    for (int64_t i = 0; i < M * K; i++) a[i] = load_elem(act, i, act_dtype);
#pragma omp parallel for schedule(static) if (use_omp)
    for (int64_t n = 0; n < N; n++) {
        const int8_t *w = wq + n * K;
        float s = load_elem(scale, n, out_dtype);
        for (int64_t m = 0; m < M; m++) {
            const float *am = a + m * K;
            float acc = 0.0f;
            for (int64_t k = 0; k < K; k++) acc += am[k] * (float)w[k];
            store_elem(out, m * N + n, out_dtype, acc * s);
        }
    }
    free(a);
}

/*
 * DequantMatMul, M > 1 form: W is first dequantised to an f32 workspace, ws[n,k] = scale[n]*f32(w)
 * (src/codegen/cpu/translator.rs:3073-3077 via build_dequantize_linear :206-282), then
 * C = A * ws^T in f32 (cblas_sgemm in the reference, :3085-3105), then the bf16 store.
 * The BLAS call is restated as a straightforward blocked loop (any summation order is allowed).
 */
void orc_dequant_matmul_workspace(void *out, const void *act, const int8_t *wq, const void *scale,
                                  int64_t M, int64_t N, int64_t K, int act_dtype, int out_dtype) {
    float *a = (float *)malloc(sizeof(float) * (size_t)(M * K));
    float *ws = (float *)malloc(sizeof(float) * (size_t)(N * K));
    for (int64_t i = 0; i < M * K; i++) a[i] = load_elem(act, i, act_dtype);
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; n++) {
        float s = load_elem(scale, n, out_dtype);
        for (int64_t k = 0; k < K; k++) ws[n * K + k] = (float)wq[n * K + k] * s;
    }
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; n++) {
        const float *w = ws + n * K;
        for (int64_t m = 0; m < M; m++) {
            const float *am = a + m * K;
            float acc = 0.0f;
            for (int64_t k = 0; k < K; k++) acc += am[k] * w[k];
            store_elem(out, m * N + n, out_dtype, acc);
        }
    }
    free(a);
    free(ws);
}

/*
 * Attention with streaming softmax, scalar and single-threaded exactly like the CPU kernel
 * (src/codegen/cpu/translator.rs:4440-5008).  q [B,Hq,Sq,D]; k,v [B,Hkv,Sk,D]; out like q.
 * k_bound = min(active, causal cap, Sk); kv head = q head / (Hq/Hkv).
 * parallel != 0 distributes the independent (b,h,sq) rows over OpenMP threads: that is NOT what the
 * reference does and is offered only as the "improved CPU" comparison.
 */
void orc_attention(void *out, const void *q, const void *k, const void *v, float scale, int64_t B,
                   int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Sk, int64_t D, int64_t active,
                   int is_causal, int dtype, int parallel) {
    int64_t group = Hq / Hkv;
    int64_t past = active - Sq;
#pragma omp parallel for schedule(static) if (parallel)
    for (int64_t row = 0; row < B * Hq * Sq; row++) {
        int64_t bh = row / Sq, sq = row % Sq;
        int64_t b = bh / Hq, h = bh % Hq;
        int64_t bhkv = b * Hkv + h / group;
        int64_t bound = active;
        if (is_causal) {
            int64_t cap = past + sq + 1;
            if (cap < bound) bound = cap;
        }
        if (Sk < bound) bound = Sk;
        float *o = (float *)malloc(sizeof(float) * (size_t)D);
        float *qf = (float *)malloc(sizeof(float) * (size_t)D);
        for (int64_t d = 0; d < D; d++) {
            o[d] = 0.0f;
            qf[d] = load_elem(q, row * D + d, dtype);
        }
        float m = -INFINITY, s = 0.0f;
        for (int64_t r = 0; r < bound; r++) {
            int64_t base = (bhkv * Sk + r) * D;
            float dot = 0.0f;
            for (int64_t d = 0; d < D; d++) dot += qf[d] * load_elem(k, base + d, dtype);
            float qk = dot * scale;
            float m_new = fmaxf(m, qk);
            float f = expf(m - m_new);
            float e = expf(qk - m_new);
            s = s * f + e;
            for (int64_t d = 0; d < D; d++) o[d] = o[d] * f + e * load_elem(v, base + d, dtype);
            m = m_new;
        }
        for (int64_t d = 0; d < D; d++) store_elem(out, row * D + d, dtype, o[d] / s);
        free(o);
        free(qf);
    }
}

/* The same recurrence over an int8 KV cache with one scale per cached row (the quant_kv_cache option):
 * qk = (q . k_int) * k_scale[r] * scale;  o = o * f + (e * v_scale[r]) * v_int
 * (src/codegen/cpu/translator.rs:4440-5008, the k_scale / v_scale operands).  q, out, scales: f32. */
void orc_attention_q8(float *out, const float *q, const int8_t *k, const int8_t *v, const float *k_scale,
                      const float *v_scale, float scale, int64_t B, int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Sk,
                      int64_t D, int64_t active, int is_causal, int parallel) {
    int64_t group = Hq / Hkv;
    int64_t past = active - Sq;
#pragma omp parallel for schedule(static) if (parallel)
    for (int64_t row = 0; row < B * Hq * Sq; row++) {
        int64_t bh = row / Sq, sq = row % Sq;
        int64_t b = bh / Hq, h = bh % Hq;
        int64_t bhkv = b * Hkv + h / group;
        int64_t bound = active;
        if (is_causal) {
            int64_t cap = past + sq + 1;
            if (cap < bound) bound = cap;
        }
        if (Sk < bound) bound = Sk;
        float *o = (float *)malloc(sizeof(float) * (size_t)D);
        for (int64_t d = 0; d < D; d++) o[d] = 0.0f;
        const float *qf = q + row * D;
        float m = -INFINITY, s = 0.0f;
        for (int64_t r = 0; r < bound; r++) {
            int64_t base = (bhkv * Sk + r) * D;
            float dot = 0.0f;
            for (int64_t d = 0; d < D; d++) dot += qf[d] * (float)k[base + d];
            float qk = dot * k_scale[bhkv * Sk + r];
            qk = qk * scale;
            float m_new = fmaxf(m, qk);
            float f = expf(m - m_new);
            float e = expf(qk - m_new);
            s = s * f + e;
            float ev = e * v_scale[bhkv * Sk + r];
            for (int64_t d = 0; d < D; d++) o[d] = o[d] * f + ev * (float)v[base + d];
            m = m_new;
        }
        for (int64_t d = 0; d < D; d++) out[row * D + d] = o[d] / s;
        free(o);
    }
}

/* cache[b,h,offset+t,:] = new[b,h,t,:], in place, no bounds check
 * (src/codegen/cpu/translator.rs:4374-4424).  elem_bytes = 2 or 4. */
void orc_kv_cache_update(void *cache, const void *newkv, int64_t BH, int64_t cache_seq, int64_t new_seq,
                         int64_t D, int64_t offset, int64_t elem_bytes) {
    for (int64_t bh = 0; bh < BH; bh++)
        memcpy((char *)cache + ((bh * cache_seq + offset) * D) * elem_bytes,
               (const char *)newkv + (bh * new_seq * D) * elem_bytes, (size_t)(new_seq * D * elem_bytes));
}

/* y = x * (1/sqrt(sum(x^2)/D + eps)) * w per row (src/codegen/cpu/translator.rs:5896-6027) */
void orc_rms_norm(void *out, const void *x, const void *w, float eps, int64_t rows, int64_t D, int dtype) {
    for (int64_t r = 0; r < rows; r++) {
        float ss = 0.0f;
        for (int64_t d = 0; d < D; d++) {
            float xv = load_elem(x, r * D + d, dtype);
            ss += xv * xv;
        }
        float inv = 1.0f / sqrtf(ss / (float)D + eps);
        for (int64_t d = 0; d < D; d++)
            store_elem(out, r * D + d, dtype, load_elem(x, r * D + d, dtype) * inv * load_elem(w, d, dtype));
    }
}

/* (g / (1 + exp(-g))) * u (src/codegen/cpu/translator.rs:459-476,994-1001) */
void orc_swish_mul(void *out, const void *gate, const void *up, int64_t n, int dtype) {
    for (int64_t i = 0; i < n; i++) {
        float g = load_elem(gate, i, dtype);
        store_elem(out, i, dtype, (g / (1.0f + expf(-g))) * load_elem(up, i, dtype));
    }
}

/* half-split RoPE with rows already gathered by position: x [rows_outer, S, D], cos/sin [S, D]
 * (crates/llm/src/builder.rs:402-438) */
void orc_rope(void *out, const void *x, const void *cosr, const void *sinr, int64_t outer, int64_t S,
              int64_t D, int dtype) {
    int64_t half = D / 2;
    for (int64_t o = 0; o < outer; o++)
        for (int64_t s = 0; s < S; s++)
            for (int64_t d = 0; d < D; d++) {
                int64_t base = (o * S + s) * D;
                float xv = load_elem(x, base + d, dtype);
                float rot = d < half ? -load_elem(x, base + d + half, dtype) : load_elem(x, base + d - half, dtype);
                float c = load_elem(cosr, s * D + d, dtype), sn = load_elem(sinr, s * D + d, dtype);
                store_elem(out, base + d, dtype, xv * c + rot * sn);
            }
}
