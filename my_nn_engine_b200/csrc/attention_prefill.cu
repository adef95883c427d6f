// Prefill attention (several query rows per sequence, causal or not, GQA) on the tensor cores.
//
// QK^T and PV of a prefill chunk are dense contractions, so the one-warp-per-query-row kernel of attention.cu (which
// walks the kv rows serially with scalar FMAs) is replaced by a tiled kernel in the FlashAttention-2 arrangement:
//   * one CTA per (64 query rows, query head, batch); 4 warps, each owning 16 query rows;
//   * K and V tiles of 64 kv rows arrive in shared memory with 16-byte cp.async copies, double buffered, in a layout whose
//     16-byte chunks are XOR-swizzled with the row index so that every ldmatrix is free of bank conflicts;
//   * S = Q K^T and O += P V run on mma.sync.m16n8k16 (bf16 / f16 inputs, f32 accumulation); the Q fragments stay in
//     registers for the whole kernel, the K fragments come from ldmatrix, the V fragments from ldmatrix.trans, and the
//     probabilities go from the S accumulators to the A operand of the second product without leaving registers;
//   * the softmax is the online form in f32 (running maximum and sum per query row, two rows per lane); the causal
//     bound of query row r is min(active, active - Sq + r + 1) as in the engine's kernel, and a CTA stops at the last
//     kv tile any of its rows can see.
// P is rounded to the 16-bit storage type before the second product (relative error 2^-9 per term, below the rounding of
// the output itself).  Shapes outside this kernel (f32, head dims other than 64/128, unaligned tensors) keep the plain
// kernel.  This is the legacy mma.sync path; chunks of 64 and more query rows run on the tcgen05 / tensor-memory kernels of
// attention_prefill_tc.cu, and this kernel serves the shorter chunks and the shapes those do not take.
#include "attention_internal.cuh"
#include "ops_internal.cuh"

namespace mynn {

constexpr int kPfaRows = 64;   // query rows per CTA
constexpr int kPfaCols = 64;   // kv rows per tile
constexpr int kPfaThreads = 128;

__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void *gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float x, float y) {
    const T a = from_f32<T>(x), b = from_f32<T>(y);
    return (uint32_t)reinterpret_cast<const uint16_t &>(a) | ((uint32_t)reinterpret_cast<const uint16_t &>(b) << 16);
}

struct PrefillAttnParams {
    void *out;
    const void *q, *k, *v;
    float scale;
    int Hq, Hkv, Sq, cache_seq;
    int active_host;
    const int32_t *active_dev;
    int is_causal, out_bshd;
};

// byte offset of 16-byte chunk c of row r in a tile whose rows hold D 16-bit elements
template <int D>
__device__ __forceinline__ uint32_t tile_off(int r, int c) {
    return (uint32_t)(r * (D * 2) + ((c ^ (r & 7)) << 4));
}

// grid (ceil(Sq / 64), Hq, B), block 128
template <typename T, int D>
__global__ void __launch_bounds__(kPfaThreads) attention_prefill_kernel(const PrefillAttnParams p) {
    constexpr int CH = D / 8;            // 16-byte chunks per row
    constexpr int KS = D / 16;           // k16 steps of QK^T
    constexpr int NT = kPfaCols / 8;     // 8-column tiles of S per warp (8)
    constexpr int DT = D / 8;            // 8-column tiles of O per warp
    constexpr uint32_t kTileBytes = kPfaCols * D * 2;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    // [Q tile][K buf0][K buf1][V buf0][V buf1]
    const uint32_t s_q = (uint32_t)__cvta_generic_to_shared(smem_raw), s_k = s_q + kPfaRows * D * 2, s_v = s_k + 2 * kTileBytes;

    const int qt = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;  // causal: the longest tiles are scheduled first
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int kvh = h / (p.Hq / p.Hkv);
    int active = p.active_dev ? *p.active_dev : p.active_host;
    active = max(0, min(active, p.cache_seq));
    const int q0 = qt * kPfaRows;
    const int past = active - p.Sq;
    // last kv row (exclusive) any query row of this CTA may see
    const int last_row = min(q0 + kPfaRows, p.Sq) - 1;
    const int kv_end = p.is_causal ? max(0, min(active, past + last_row + 1)) : active;

    const T *qg = reinterpret_cast<const T *>(p.q) + ((size_t)(b * p.Hq + h) * p.Sq) * D;
    const T *kg = reinterpret_cast<const T *>(p.k) + ((size_t)(b * p.Hkv + kvh) * p.cache_seq) * D;
    const T *vg = reinterpret_cast<const T *>(p.v) + ((size_t)(b * p.Hkv + kvh) * p.cache_seq) * D;

    auto load_kv_tile = [&](int kv0, int buf) {
        for (int i = threadIdx.x; i < kPfaCols * CH; i += kPfaThreads) {
            const int r = i / CH, c = i - r * CH;
            const int row = min(kv0 + r, active - 1);  // rows past the live ones are masked: read a live row instead, so that
                                                       // no stale NaN/Inf meets a zero probability in the second product
            cp_async16(s_k + buf * kTileBytes + tile_off<D>(r, c), kg + (size_t)row * D + c * 8);
            cp_async16(s_v + buf * kTileBytes + tile_off<D>(r, c), vg + (size_t)row * D + c * 8);
        }
    };

    // Q tile -> shared memory (rows past Sq are clamped; their results are never stored), first kv tile behind it
    for (int i = threadIdx.x; i < kPfaRows * CH; i += kPfaThreads) {
        const int r = i / CH, c = i - r * CH;
        cp_async16(s_q + tile_off<D>(r, c), qg + (size_t)min(q0 + r, p.Sq - 1) * D + c * 8);
    }
    cp_async_commit_group();
    if (kv_end > 0) load_kv_tile(0, 0);
    cp_async_commit_group();
    cp_async_wait_group<1>();
    __syncthreads();

    // Q fragments of this warp's 16 rows: a[ks][0..3]
    uint32_t qa[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
        const int r = 16 * warp + (lane & 7) + 8 * ((lane >> 3) & 1), c = 2 * ks + (lane >> 4);
        ldmatrix_x4(qa[ks], s_q + tile_off<D>(r, c));
    }

    float o[DT][4];
#pragma unroll
    for (int j = 0; j < DT; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int row_lo = q0 + 16 * warp + g, row_hi = row_lo + 8;  // the two query rows of this lane
    const int bound_lo = p.is_causal ? min(active, past + row_lo + 1) : active;
    const int bound_hi = p.is_causal ? min(active, past + row_hi + 1) : active;

    const int n_tiles = (kv_end + kPfaCols - 1) / kPfaCols;
    const float sl2 = p.scale * 1.4426950408889634f;
    for (int it = 0; it < n_tiles; it++) {
        const int buf = it & 1, kv0 = it * kPfaCols;
        if (it + 1 < n_tiles) load_kv_tile(kv0 + kPfaCols, buf ^ 1);  // the other buffer was released by the barrier below
        cp_async_commit_group();
        cp_async_wait_group<1>();  // tile `it` has landed
        __syncthreads();

        // ---- S = Q K^T : s[nt][c] ----
        float s[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        const uint32_t kb = s_k + buf * kTileBytes;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
#pragma unroll
            for (int np = 0; np < NT / 2; np++) {  // two 8-column tiles per ldmatrix.x4
                uint32_t bf[4];
                const int r = 16 * np + (lane & 7) + 8 * (lane >> 4), c = 2 * ks + ((lane >> 3) & 1);
                ldmatrix_x4(bf, kb + tile_off<D>(r, c));
                mma_kv<T>(s[2 * np], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], bf[0], bf[1]);
                mma_kv<T>(s[2 * np + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], bf[2], bf[3]);
            }
        }
        // ---- mask, online softmax (rows g and g + 8 of this warp's 16) ----
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int col = kv0 + 8 * nt + 2 * t + e;
                s[nt][e] = col < bound_lo ? s[nt][e] * sl2 : -INFINITY;  // scores in units of log2(e): exp() becomes exp2()
                s[nt][2 + e] = col < bound_hi ? s[nt][2 + e] * sl2 : -INFINITY;
                tmax[0] = fmaxf(tmax[0], s[nt][e]);
                tmax[1] = fmaxf(tmax[1], s[nt][2 + e]);
            }
        float alpha[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
            tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
            const float m_new = fmaxf(m_run[r], tmax[r]);
            m_use[r] = m_new == -INFINITY ? 0.f : m_new;  // a row with nothing visible yet (rows past Sq): keep exp() finite
            alpha[r] = exp2f(m_run[r] - m_use[r]);
            m_run[r] = m_new;
        }
        float psum[2] = {0.f, 0.f};
        uint32_t pa[NT / 2][4];  // P as A fragments of the second product: k16 step j covers S tiles 2j, 2j+1
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const float p0 = exp2f(s[nt][0] - m_use[0]), p1 = exp2f(s[nt][1] - m_use[0]);
            const float p2 = exp2f(s[nt][2] - m_use[1]), p3 = exp2f(s[nt][3] - m_use[1]);
            psum[0] += p0 + p1;
            psum[1] += p2 + p3;
            pa[nt >> 1][(nt & 1) * 2] = pack2<T>(p0, p1);      // row g:   a0 (k 2t..) for even nt, a2 (k 2t+8..) for odd nt
            pa[nt >> 1][(nt & 1) * 2 + 1] = pack2<T>(p2, p3);  // row g+8: a1 / a3
        }
#pragma unroll
        for (int r = 0; r < 2; r++) l_run[r] = l_run[r] * alpha[r] + psum[r];
#pragma unroll
        for (int j = 0; j < DT; j++) {
            o[j][0] *= alpha[0];
            o[j][1] *= alpha[0];
            o[j][2] *= alpha[1];
            o[j][3] *= alpha[1];
        }
        // ---- O += P V ----
        const uint32_t vb = s_v + buf * kTileBytes;
#pragma unroll
        for (int kk = 0; kk < kPfaCols / 16; kk++) {
#pragma unroll
            for (int dp = 0; dp < DT / 2; dp++) {  // two 8-column tiles of O per ldmatrix.x4.trans
                uint32_t bf[4];
                const int r = 16 * kk + (lane & 7) + 8 * ((lane >> 3) & 1), c = 2 * dp + (lane >> 4);
                ldmatrix_x4_trans(bf, vb + tile_off<D>(r, c));
                mma_kv<T>(o[2 * dp], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], bf[0], bf[1]);
                mma_kv<T>(o[2 * dp + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], bf[2], bf[3]);
            }
        }
        __syncthreads();  // everybody is done with buffer `buf` before the next iteration's prefetch overwrites it
    }

    // ---- finish: row sums over the 4 lanes of a row, normalise, store ----
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    T *out = reinterpret_cast<T *>(p.out);
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int row = r ? row_hi : row_lo;
        if (row >= p.Sq) continue;
        const float inv = 1.0f / l_run[r];
        const size_t orow = p.out_bshd ? ((size_t)b * p.Sq + row) * p.Hq + h : ((size_t)(b * p.Hq + h)) * p.Sq + row;
#pragma unroll
        for (int j = 0; j < DT; j++)
            *reinterpret_cast<uint32_t *>(out + orow * D + 8 * j + 2 * t) = pack2<T>(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
    }
}

template <typename T, int D>
static int launch_pfa(cudaStream_t st, const PrefillAttnParams &p, int B) {
    const size_t smem = (size_t)kPfaRows * D * 2 + 4 * (size_t)kPfaCols * D * 2;
    auto kern = attention_prefill_kernel<T, D>;
    static bool attr_set = false;
    if (!attr_set) {
        MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set = true;
    }
    kern<<<dim3((p.Sq + kPfaRows - 1) / kPfaRows, p.Hq, B), kPfaThreads, smem, st>>>(p);
    MYNN_LAUNCH_OK("attention_prefill_kernel");
    return MYNN_OK;
}

bool attention_prefill_supported(int Sq, int D, int dtype, const void *q, const void *k, const void *v, const void *out) {
    return Sq > 1 && (D == 64 || D == 128) && (dtype == MYNN_BF16 || dtype == MYNN_F16) &&
           ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) % 16) == 0) && ((uintptr_t)out % 4) == 0;
}

int launch_attention_prefill(cudaStream_t st, void *out, const void *q, const void *k, const void *v, float scale, int B, int Hq,
                             int Hkv, int Sq, int D, int cache_seq_len, int active_seq_kv, const int32_t *active_seq_kv_dev,
                             int is_causal, int dtype, int out_bshd) {
    PrefillAttnParams p;
    p.out = out;
    p.q = q;
    p.k = k;
    p.v = v;
    p.scale = scale;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.Sq = Sq;
    p.cache_seq = cache_seq_len;
    p.active_host = active_seq_kv;
    p.active_dev = active_seq_kv_dev;
    p.is_causal = is_causal;
    p.out_bshd = out_bshd;
    if (dtype == MYNN_BF16) return D == 64 ? launch_pfa<__nv_bfloat16, 64>(st, p, B) : launch_pfa<__nv_bfloat16, 128>(st, p, B);
    return D == 64 ? launch_pfa<__half, 64>(st, p, B) : launch_pfa<__half, 128>(st, p, B);
}

}  // namespace mynn
