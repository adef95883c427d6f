// Weight-streaming DequantMatMul on the 5th-generation tensor cores (tcgen05, kind::i8) for small batches.
//
//   out[m,n] = scale[n] * sum_k act[m,k] * wq[n,k],   M*3 <= 96 rows of activations (decode batches up to 32)
//
// Decode is bound by reading the int8 weights from HBM once.  Converting int8 to bf16 in registers and feeding
// mma.sync costs more issue slots and legacy-MMA throughput than the memory system leaves time for at batch 32, so
// this kernel removes all per-weight work from the SM's instruction stream:
//
//   * A tiny pre-pass rewrites each activation row as a fixed-point number with a per-row power-of-two scale and
//     splits it into three signed 8-bit digits ("limbs"): act = 2^(e-22) * (l0 + 256 l1 + 65536 l2) where the row
//     maximum is below 2^e.  A bf16 element within 2^-14 of its row maximum is represented EXACTLY; smaller ones are
//     rounded to 2^-23 of the maximum.
//   * The product then is three int8 x int8 dot products accumulated exactly in int32 (tcgen05.mma kind::i8): the
//     weight bytes go from HBM to shared memory by TMA (128-byte swizzled tiles, 3-stage mbarrier pipeline) and
//     from shared memory straight into the tensor core; no thread ever touches a weight.
//   * Accumulators live in TMEM (one lane per weight row, one column per (activation row, limb)); the epilogue reads
//     them with tcgen05.ld, recombines the limbs in f32, applies the activation-row and weight-row scales, the
//     optional residual add, and stores.
//   * K can be split over a thread-block cluster; the int32 partial sums are reduced through distributed shared
//     memory.  Integer addition is associative, so the result does not depend on the split.
//
// Roles inside a CTA (192 threads): warp 0 = TMA producer (one elected lane), warp 1 = MMA issuer (one elected
// lane) and TMEM allocator, warps 2-5 = epilogue (TMEM lane quadrant = warp index mod 4).
// Every mbarrier wait is bounded: on expiry the kernel records an error code in `status`, skips the remaining work,
// still releases TMEM and reaches every cluster barrier, and returns.
#include <cuda.h>

#include <cstring>

#include "common.cuh"
#include "i8_gemm.cuh"
#include "tcgen05.cuh"
#include "tp_fused.cuh"

namespace mynn {

MYNN_DEFINE_WAIT_BUDGET_SETTER(i8_gemm)

constexpr int kTileRows = 128;   // weight rows per CTA (UMMA M)
constexpr int kBlockK = 128;     // int8 k values per pipeline stage = one 128-byte swizzle row
constexpr int kStages = 3;      // pipeline depth when two CTAs share an SM
constexpr int kMaxStages = 7;   // depth when the grid has at most one CTA per SM (196 KB of tiles in flight)
constexpr int kGemmThreads = 320;  // TMA warp, MMA warp, eight epilogue warps

struct I8GemmParams {
    void *out;
    const void *scale, *resid;
    const float *ascale;  // [M] activation row scales 2^(e-22)
    int M, N, K;
    int *status;          // device int, set non-zero on a timed-out wait
    int stages;           // pipeline depth: kStages or kMaxStages
    I8Tp tp;              // tensor-parallel form: the outputs are delivered to every rank as partial sums (mode 0: off)
    int skip_last_stage;  // test aid (MYNN_OPT_INJECT_STALL): the producer leaves out the last k block, so a bounded wait expires
#ifdef MYNN_TUNING
    unsigned long long *timing;  // 8 timestamps (ns) of CTA (0,0), or null
#endif
};

#ifdef MYNN_TUNING
#define MYNN_STAMP(cond, slot) do { if (p.timing != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && (cond)) p.timing[slot] = global_ns(); } while (0)
#else
#define MYNN_STAMP(cond, slot) do { } while (0)
#endif
#ifdef MYNN_TUNING
// Tuning build: CTA 0 of a limb-producer kernel records {start, end, kernel id} in a ring (read with cudaMemcpyFromSymbol).
__device__ unsigned long long g_glue_t[3 * 1024];
__device__ unsigned g_glue_n;
#define MYNN_GLUE_BEGIN(id)                                                  \
    unsigned glue_slot = 0;                                                  \
    if (blockIdx.x == 0 && threadIdx.x == 0) {                               \
        glue_slot = atomicAdd(&g_glue_n, 1u) % 1024u;                        \
        g_glue_t[3 * glue_slot] = global_ns();                               \
        g_glue_t[3 * glue_slot + 2] = (id);                                  \
    }
#define MYNN_GLUE_END() do { if (blockIdx.x == 0 && threadIdx.x == 0) g_glue_t[3 * glue_slot + 1] = global_ns(); } while (0)
#define MYNN_GLUE_BEGIN_C(id)                                                \
    unsigned glue_slot = 0;                                                  \
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) {            \
        glue_slot = atomicAdd(&g_glue_n, 1u) % 1024u;                        \
        g_glue_t[3 * glue_slot] = global_ns();                               \
        g_glue_t[3 * glue_slot + 2] = (id);                                  \
    }
#define MYNN_GLUE_END_C() do { if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) g_glue_t[3 * glue_slot + 1] = global_ns(); } while (0)
#else
#define MYNN_GLUE_BEGIN_C(id) do { } while (0)
#define MYNN_GLUE_END_C() do { } while (0)
#define MYNN_GLUE_BEGIN(id) do { } while (0)
#define MYNN_GLUE_END() do { } while (0)
#endif

// grid (ceil(N/128), S), cluster (1, S, 1).  NC = activation columns (3 limbs x rows, padded to 16).
template <typename OutT, int NC>
__global__ void __launch_bounds__(kGemmThreads, 2)
i8_stream_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                      const I8GemmParams p) {
    constexpr uint32_t kWBytes = kTileRows * kBlockK, kABytes = NC * kBlockK;
    constexpr uint32_t kStageBytes = kWBytes + ((kABytes + 1023) / 1024) * 1024;
    constexpr uint32_t kTmemCols = NC <= 32 ? 32 : (NC <= 64 ? 64 : 128);
    static_assert(kStages * kStageBytes >= (NC / 3) * kTileRows * 8 + ((NC / 3 + 3) / 4) * (kGemmThreads - 64) * 4,
                  "the reduction buffer and the residual staging area alias the stage buffers");
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzled tiles need 1024-byte alignment
    __shared__ uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], accum_bar;
    const int stages = p.stages;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ float sh_ascale[32];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = gridDim.y;
    MYNN_STAMP(threadIdx.x == 0, 0);
    const int rank = S > 1 ? (int)cluster_ctarank() : 0;
    const int row0 = blockIdx.x * kTileRows;
    // this CTA's contiguous share of the k blocks
    const int kblocks = (p.K + kBlockK - 1) / kBlockK;
    const int q = kblocks / S, rem = kblocks - q * S;
    const int kb_beg = rank * q + min(rank, rem);
    const int nkb = q + (rank < rem ? 1 : 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&accum_bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    MYNN_STAMP(threadIdx.x == 0, 1);  // set-up done

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
            // The weights do not depend on the preceding kernel: start streaming them at once, and only then wait
            // (programmatic dependent launch) for the grid that writes the activation limbs.
            const int nload = nkb - ((p.skip_last_stage & 1) ? 1 : 0);  // normally every k block
            const int pre = min(nload, stages);
            for (int i = 0; i < pre; i++) {
                mbar_expect_tx(&full_bar[i], kWBytes + kABytes);
                tma_load_2d(smem + i * kStageBytes, &map_w, (kb_beg + i) * kBlockK, row0, &full_bar[i]);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            MYNN_STAMP(true, 2);  // predecessor grid complete
            for (int i = 0; i < pre; i++)
                tma_load_2d(smem + i * kStageBytes + kWBytes, &map_a, (kb_beg + i) * kBlockK, 0, &full_bar[i]);
            for (int i = pre; i < nload; i++) {
                const int s = i % stages, it = i / stages;
                if (!mbar_wait_spin(&empty_bar[s], (it - 1) & 1, &abort_flag)) {
                    atomicExch(&abort_flag, 1);
                    atomicExch(p.status, 1);
                    break;
                }
                uint8_t *st = smem + s * kStageBytes;
                mbar_expect_tx(&full_bar[s], kWBytes + kABytes);
                tma_load_2d(st, &map_w, (kb_beg + i) * kBlockK, row0, &full_bar[s]);
                tma_load_2d(st + kWBytes, &map_a, (kb_beg + i) * kBlockK, 0, &full_bar[s]);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // instruction descriptor: D = S32, A = B = signed int8, both K-major, N = NC, M = 128
            constexpr uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NC >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24);
            bool ok = true;
            for (int i = 0; i < nkb && ok; i++) {
                const int s = i % stages, it = i / stages;
                if (!mbar_wait_spin(&full_bar[s], it & 1, &abort_flag)) {
                    atomicExch(&abort_flag, 1);
                    atomicExch(p.status, 2);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + s * kStageBytes);
                const uint64_t adesc = make_kmajor_sw128_desc(a_addr), bdesc = make_kmajor_sw128_desc(a_addr + kWBytes);
#pragma unroll
                for (int k = 0; k < kBlockK / 32; k++)  // 32 bytes of k per instruction: advance the start address
                    umma_i8(tmem_base, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (i | k) ? 1u : 0u);
                umma_commit(&empty_bar[s]);  // the stage may be refilled once these MMAs have read it
            }
            umma_commit(&accum_bar);  // accumulators complete (also fires when nothing was issued)
        }
        __syncwarp();
    }

    // ---------------- epilogue: warps 2..9; a warp may read the TMEM lane quadrant (warp & 3) ----------------
    // Eight warps, two per lane quadrant: warps 2..5 take the first chunk of accumulator columns (48 = 16 activation rows
    // x 3 limbs), warps 6..9 the second.  The finish of an output is a chain of dependent instructions and every epilogue
    // warp sits alone on its scheduler, so the epilogue's length is the chain length times the outputs per thread: twice
    // the warps halve it.
    // S == 1: thread (quadrant, lane) finishes weight row quad * 32 + lane of the tile for the activation rows of its chunk.
    // S  > 1: every CTA first pushes its int64 partial sums (limbs already combined, still exact) into the shared
    //         memory of the CTA that owns the row (rows are dealt out in S contiguous groups), with remote stores
    //         that need no round trip; after a cluster barrier each CTA adds what it received and finishes its rows.
    //         The receive buffer aliases the stage buffers, so a first cluster barrier makes sure every CTA of the
    //         cluster is past its main loop before anybody writes into a peer.
    constexpr int kEpiThreads = kGemmThreads - 64;
    const int quad = warp & 3;
    const int r_local = quad * 32 + lane;
    const OutT *scale_p = reinterpret_cast<const OutT *>(p.scale);
    const OutT *resid_p = reinterpret_cast<const OutT *>(p.resid);
    OutT *out_p = reinterpret_cast<OutT *>(p.out);
    constexpr int MR = NC / 3;                        // activation rows this instantiation can hold
    constexpr int kChunk = NC < 48 ? NC : 48;         // accumulator columns per warp
    constexpr int RPC = kChunk / 3;                   // activation rows per chunk
    constexpr int kOwnMax = (MR + 3) / 4;             // outputs per thread with a K split (S >= 2)
    const int c0 = warp >= 6 ? kChunk : 0, m0 = warp >= 6 ? RPC : 0;  // this warp's chunk
    const bool has_chunk = warp >= 2 && c0 < NC;
    const int rows_per = kTileRows / S, mstep = kEpiThreads / rows_per;  // S > 1: this thread finishes row r_own for m = m_own + j * mstep
    const int et = threadIdx.x - 64;                  // epilogue thread index 0..255 (warps >= 2)
    const int r_own = S == 1 ? r_local : rank * rows_per + (et % rows_per);
    const int m_own = S == 1 ? 0 : et / rows_per;
    const int n_own = row0 + r_own;
    // The residuals are requested before the main loop ends and wait in registers with compile-time indices (a load per
    // output inside the finish loop cost 200-400 ns each): S == 1 those of this warp's chunk, S > 1 those of this thread's
    // outputs m_own + j * mstep.
    float wscale = 0.f, res_r[RPC > kOwnMax ? RPC : kOwnMax];  // one array: the two forms never run together
    bool have_acc = false;
    if (warp >= 2) {
        asm volatile("griddepcontrol.wait;" ::: "memory");  // row scales and the residual come from earlier grids
        // everything the finish needs from global memory is requested before waiting for the accumulators
        if (et < 32) sh_ascale[et] = et < p.M ? p.ascale[et] : 0.f;
        if (n_own < p.N) wscale = to_f32<OutT>(scale_p[n_own]);
        if (S == 1) {
#pragma unroll
            for (int i = 0; i < RPC; i++) {
                const int m = m0 + i;
                res_r[i] = (resid_p && n_own < p.N && m < MR && m < p.M) ? to_f32<OutT>(resid_p[(size_t)m * p.N + n_own]) : 0.f;
            }
        } else {
#pragma unroll
            for (int j = 0; j < kOwnMax; j++) {
                const int m = m_own + j * mstep;
                res_r[j] = (resid_p && n_own < p.N && m < p.M) ? to_f32<OutT>(resid_p[(size_t)m * p.N + n_own]) : 0.f;
            }
        }
        // one lane per warp polls the barrier (spinning threads would flood the shared-memory pipe that the
        // co-resident CTA needs); the outcome is broadcast to the warp
        int ok_i = 1;
        if (lane == 0) ok_i = mbar_wait_spin(&accum_bar, 0, &abort_flag) ? 1 : 0;
        const bool ok = __shfl_sync(0xffffffffu, ok_i, 0) != 0;
        MYNN_STAMP(threadIdx.x == 64, 3);  // accumulators complete
        // Delivering form: the kernel that sums the partial sums polls for them word by word and touches nothing else this
        // kernel still reads, so it may become resident now (if it was launched as a programmatic dependent) instead of
        // after this grid's slowest CTA has left.
        if (p.tp.mode == 1 && threadIdx.x == 64) pdl_trigger();
        if (!ok) {
            atomicExch(&abort_flag, 1);
            atomicExch(p.status, 3);
        }
        tc_fence_after();
        // warp-uniform, because tcgen05.ld below must be executed by whole warps
        have_acc = __all_sync(0xffffffffu, ok && nkb > 0 && !*(volatile int *)&abort_flag);
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");  // sh_ascale visible to the epilogue warps
        MYNN_STAMP(threadIdx.x == 64, 7);
    }
    // A warp reads its chunk in pieces of kSub columns (24 = 8 activation rows when the chunk has 48) to keep registers in check.
    constexpr int kSub = kChunk == 48 ? 24 : kChunk, kSubs = kChunk / kSub, RS = kSub / 3;
    auto load_sub = [&](int h, uint32_t (&acc)[kSub]) {
        const int cb = c0 + h * kSub;  // first column; columns at and past NC do not exist
        if (have_acc && cb < NC) {
            uint32_t v[16];
            tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + cb, v);
#pragma unroll
            for (int j = 0; j < 16; j++) acc[j] = v[j];
            if (kSub == 24) {
                if (cb + 16 < NC) tmem_ld8(tmem_base + ((uint32_t)(quad * 32) << 16) + cb + 16, &acc[16]);
            } else if (kSub == 32) {
                tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + cb + 16, v);
#pragma unroll
                for (int j = 0; j < 16; j++) acc[16 + j] = v[j];
            }
            tmem_ld_wait();
        } else {
#pragma unroll
            for (int c = 0; c < kSub; c++) acc[c] = 0u;
        }
    };
    auto combine = [](const uint32_t *a3) {
        return (long long)(int)a3[2] * 65536 + (long long)(int)a3[1] * 256 + (long long)(int)a3[0];
    };
    // An output in two steps, so that a caller can compute several values before it stores any: a store through the generic
    // `out` pointer may alias anything as far as the compiler knows, which would otherwise pin every finish behind the
    // previous one's store and expose its whole dependent chain (conversions, two products, the rounding) once per output.
    auto value = [&](long long sum, float asc, float resv) {
        // separate roundings (no fused multiply-add), so that every kernel of this operator gives the same bits
        float v = __fmul_rn(__fmul_rn((float)sum, asc), wscale);
        if (resid_p) v = __fadd_rn(round_store<OutT>(v), resv);
        return v;
    };
    auto deliver = [&](int m, float v) {
        if (p.tp.mode == 1) {
            // a partial sum goes to slot [this rank] of EVERY rank's buffer: one 4-byte store per destination, over NVLink
            // for the peers; the reader re-reads a word while it is EMPTY, so no fence or flag follows.  A NaN travels as the
            // canonical NaN, which is not the EMPTY pattern.
            const uint32_t word = v != v ? 0x7fc00000u : __float_as_uint(v);
            const size_t idx = ((size_t)p.tp.rank * p.tp.max_rows + m) * p.N + n_own;
            const int nr = p.tp.skip ? 0 : p.tp.world;
#pragma unroll 1
            for (int r = 0; r < nr; r++) p.tp.part[r][idx] = word;
        } else {
            out_p[(size_t)m * p.N + n_own] = from_f32<OutT>(v);
        }
    };

    if (S == 1) {
        if (has_chunk) {
#pragma unroll
            for (int h = 0; h < kSubs; h++) {
                uint32_t acc[kSub];
                load_sub(h, acc);
                MYNN_STAMP(threadIdx.x == 64 && h == 0, 4);
                float asc[RS], vv[RS];
#pragma unroll
                for (int i = 0; i < RS; i++) asc[i] = sh_ascale[min(m0 + h * RS + i, 31)];
#pragma unroll
                for (int i = 0; i < RS; i++) vv[i] = value(combine(&acc[3 * i]), asc[i], res_r[h * RS + i]);
#pragma unroll
                for (int i = 0; i < RS; i++) {
                    const int m = m0 + h * RS + i;
                    if (m < MR && m < p.M && n_own < p.N) deliver(m, vv[i]);
                }
            }
        }
    } else {
        long long *recv = reinterpret_cast<long long *>(smem);  // [S source ranks][MR][rows_per] int64 <= 32 KB
        cluster_sync_all();  // every CTA of the cluster is past its main loop: stage buffers are free everywhere
        if (has_chunk) {
            const uint32_t owner = (uint32_t)(r_local / rows_per);
            const int r_in = r_local % rows_per;
#pragma unroll
            for (int h = 0; h < kSubs; h++) {
                uint32_t acc[kSub];
                load_sub(h, acc);
#pragma unroll
                for (int i = 0; i < RS; i++) {
                    const int m = m0 + h * RS + i;
                    if (m < MR && m < p.M) {
                        const long long v = combine(&acc[3 * i]);
                        const uint32_t local = smem_u32(&recv[((size_t)rank * MR + m) * rows_per + r_in]);
                        uint32_t remote;
                        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(owner));
                        asm volatile("st.shared::cluster.b64 [%0], %1;" ::"r"(remote), "l"(v) : "memory");
                    }
                }
            }
        }
        // the rolled loop below takes its residuals from this thread's own column of a staging area behind the receive
        // buffer (nobody else touches it)
        float *res_stage = reinterpret_cast<float *>(smem + (size_t)MR * kTileRows * 8) + et;
        if (warp >= 2 && resid_p) {
#pragma unroll
            for (int j = 0; j < kOwnMax; j++) res_stage[j * kEpiThreads] = res_r[j];
        }
        cluster_sync_all();  // release/acquire: the partial sums pushed by every peer are visible
        MYNN_STAMP(threadIdx.x == 64, 4);
        if (warp >= 2 && n_own < p.N) {
            // a compact rolled loop: straight-line code that runs once per CTA pays an instruction-cache miss per line
            const int r_in = et % rows_per;
            int j = 0;
#pragma unroll 1
            for (int m = m_own; m < p.M; m += mstep, j++) {
                const float resv = resid_p ? res_stage[j * kEpiThreads] : 0.f;
                const long long *src = recv + (size_t)m * rows_per + r_in;
                long long sum = 0;
#pragma unroll
                for (int rr = 0; rr < 8; rr++)
                    if (rr < S) sum += src[(size_t)rr * MR * rows_per];
                deliver(m, value(sum, sh_ascale[m], resv));
            }
        }
    }

    MYNN_STAMP(threadIdx.x == 64, 5);  // outputs stored
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
    MYNN_STAMP(threadIdx.x == 0, 6);
}

// ---- activation pre-pass: rows -> three int8 limbs + power-of-two row scale -----------------------------------
// limbs [(3m + l)][K] int8 (row stride K); with max |row| < 2^e the row is scaled by 2^(22-e), so |A| < 2^22, and
// ascale[m] = 2^(e-22).
template <typename ActT>
__global__ void __launch_bounds__(256) act_to_limbs_kernel(int8_t *limbs, float *ascale, const ActT *act, int K) {
    constexpr int kMaxPer = 16;  // 4-element groups held per thread: rows up to 256 * 4 * 16 = 16384 stay in registers
    __shared__ float wmax[8];
    __shared__ float s_scale;
    pdl_trigger();  // the GEMM may begin streaming its weights
    pdl_wait();     // the activations come from the preceding kernel
    const int m = blockIdx.x;
    const ActT *row = act + (size_t)m * K;
    const int groups = K >> 2;  // K % 16 == 0
    float v[kMaxPer][4];
    float mx = 0.f;
    bool bad = false;
#pragma unroll
    for (int j = 0; j < kMaxPer; j++) {
        const int gi = threadIdx.x + j * 256;
        if (gi < groups) {
            if constexpr (sizeof(ActT) == 2) {
                const uint2 raw = *reinterpret_cast<const uint2 *>(row + 4 * gi);
                const ActT *e = reinterpret_cast<const ActT *>(&raw);
#pragma unroll
                for (int i = 0; i < 4; i++) v[j][i] = to_f32<ActT>(e[i]);
            } else {
                const float4 raw = *reinterpret_cast<const float4 *>(row + 4 * gi);
                v[j][0] = raw.x; v[j][1] = raw.y; v[j][2] = raw.z; v[j][3] = raw.w;
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                bad |= !(fabsf(v[j][i]) <= 3.0e38f);
                mx = fmaxf(mx, fabsf(v[j][i]));
            }
        }
    }
    for (int gi = threadIdx.x + kMaxPer * 256; gi < groups; gi += 256)  // rows longer than 16384: second read below
        for (int i = 0; i < 4; i++) {
            const float a = to_f32<ActT>(row[4 * gi + i]);
            bad |= !(fabsf(a) <= 3.0e38f);
            mx = fmaxf(mx, fabsf(a));
        }
    mx = warp_max(mx);
    const unsigned anybad = __syncthreads_or(bad);
    if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < 8; i++) t = fmaxf(t, wmax[i]);
        int e = 0;
        if (t > 0.f) frexpf(t, &e);  // t = f * 2^e, f in [0.5, 1): t < 2^e
        s_scale = t > 0.f ? ldexpf(1.0f, 22 - e) : 1.0f;  // |a| * s_scale < 2^22
    }
    __syncthreads();
    const float sc = s_scale;
    if (threadIdx.x == 0) ascale[m] = anybad ? __int_as_float(0x7fc00000) : 1.0f / sc;  // non-finite input -> NaN outputs
    int8_t *l0 = limbs + (size_t)(3 * m) * K, *l1 = l0 + K, *l2 = l1 + K;
    auto split4 = [&](const float (&x)[4], int gi) {
        uint32_t w0 = 0, w1 = 0, w2 = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int A = anybad ? 0 : __float2int_rn(x[i] * sc);
            const int d0 = (int)(int8_t)(A & 0xFF);
            A = (A - d0) >> 8;
            const int d1 = (int)(int8_t)(A & 0xFF);
            A = (A - d1) >> 8;
            w0 |= (uint32_t)(d0 & 0xFF) << (8 * i);
            w1 |= (uint32_t)(d1 & 0xFF) << (8 * i);
            w2 |= (uint32_t)(A & 0xFF) << (8 * i);
        }
        reinterpret_cast<uint32_t *>(l0)[gi] = w0;
        reinterpret_cast<uint32_t *>(l1)[gi] = w1;
        reinterpret_cast<uint32_t *>(l2)[gi] = w2;
    };
#pragma unroll
    for (int j = 0; j < kMaxPer; j++) {
        const int gi = threadIdx.x + j * 256;
        if (gi < groups) split4(v[j], gi);
    }
    for (int gi = threadIdx.x + kMaxPer * 256; gi < groups; gi += 256) {
        float x[4];
        for (int i = 0; i < 4; i++) x[i] = to_f32<ActT>(row[4 * gi + i]);
        split4(x, gi);
    }
}

// ---- fused producers: an operator's output row goes straight to limbs --------------------------------------------
// One CTA of 1024 threads per row.  The row (already rounded to the storage dtype, i.e. after the operator's store
// point) is kept in shared memory as f32; each thread tracks the maximum of what it produced, one block reduction
// gives the power-of-two scale, and the three int8 limbs per element are written 4 elements at a time.
constexpr int kRowThreads = 1024;

template <typename T>
__device__ __forceinline__ void load8(const T *p, float (&v)[8]) {
    if constexpr (sizeof(T) == 2) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(p);
        const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = to_f32<T>(e[i]);
    } else {
        const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
}
template <typename T>
__device__ __forceinline__ void store8(T *p, const float (&v)[8]) {
    if constexpr (sizeof(T) == 2) {
        uint4 raw;
        T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
        for (int i = 0; i < 8; i++) e[i] = from_f32<T>(v[i]);
        *reinterpret_cast<uint4 *>(p) = raw;
    } else {
        *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
}

// Block-wide maximum -> limb scale (broadcast through red[32]); writes the row scale; returns 0 for a bad row.
__device__ __forceinline__ float block_limb_scale(float mx, bool bad, float *ascale_m, float *red /* >= 34 floats */) {
    mx = warp_max(mx);
    const unsigned anybad = __syncthreads_or(bad);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < (int)(blockDim.x >> 5); i++) t = fmaxf(t, red[i]);
        int e = 0;
        if (t > 0.f) frexpf(t, &e);
        const float sc = t > 0.f ? ldexpf(1.0f, 22 - e) : 1.0f;
        red[32] = anybad ? 0.f : sc;
        *ascale_m = anybad ? __int_as_float(0x7fc00000) : 1.0f / sc;  // non-finite input -> NaN outputs
    }
    __syncthreads();
    return red[32];
}

// K elements of a row whose limb rows are `stride` bytes apart (stride == K for a whole row).
__device__ __forceinline__ void smem_row_to_limbs(const float *row_s, int K, int8_t *limb_row0, float sc, size_t stride) {
    uint32_t *l0 = reinterpret_cast<uint32_t *>(limb_row0);
    uint32_t *l1 = reinterpret_cast<uint32_t *>(limb_row0 + stride);
    uint32_t *l2 = reinterpret_cast<uint32_t *>(limb_row0 + 2 * stride);
    for (int gi = threadIdx.x; gi < (K >> 2); gi += blockDim.x) {
        const float4 x4 = reinterpret_cast<const float4 *>(row_s)[gi];
        const float x[4] = {x4.x, x4.y, x4.z, x4.w};
        uint32_t w0 = 0, w1 = 0, w2 = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int A = sc == 0.f ? 0 : __float2int_rn(x[i] * sc);
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

// RMSNorm whose output feeds only DequantMatMuls: y = round(x * rsqrt(mean x^2 + eps) * w) -> limbs.
// With `part`: first s = round(x + round(part)) is stored to sum_out (residual add of an all-reduced f32 partial sum).
// norm_out (optional) also receives y in the storage dtype.  D % 8 == 0, rows 16-byte aligned.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
rms_norm_limbs_kernel(int8_t *limbs, float *ascale, T *norm_out, T *sum_out, const T *x, const float *part, const T *w,
                      float eps, int D) {
    extern __shared__ __align__(16) float row_s[];
    __shared__ float red[40];
    MYNN_GLUE_BEGIN(1);
    pdl_trigger();
    pdl_wait();
    const int m = blockIdx.x;
    const size_t base = (size_t)m * D;
    float ss = 0.f;
    for (int i = 8 * threadIdx.x; i < D; i += 8 * kRowThreads) {
        float v[8];
        load8<T>(x + base + i, v);
        if (part != nullptr) {
            float pp[8];
            load8<float>(part + base + i, pp);
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = round_store<T>(v[j] + round_store<T>(pp[j]));
            store8<T>(sum_out + base + i, v);
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            row_s[i + j] = v[j];
            ss += v[j] * v[j];
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int i = 0; i < kRowThreads / 32; i++) tot += red[i];
        red[33] = 1.0f / sqrtf(tot / (float)D + eps);
    }
    __syncthreads();
    const float inv = red[33];
    float mx = 0.f;
    bool bad = false;
    for (int i = 8 * threadIdx.x; i < D; i += 8 * kRowThreads) {
        float wv[8], y[8];
        load8<T>(w + i, wv);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            y[j] = round_store<T>(row_s[i + j] * inv * wv[j]);
            row_s[i + j] = y[j];
            bad |= !(fabsf(y[j]) <= 3.0e38f);
            mx = fmaxf(mx, fabsf(y[j]));
        }
        if (norm_out != nullptr) store8<T>(norm_out + base + i, y);
    }
    const float sc = block_limb_scale(mx, bad, ascale + m, red);  // its barriers also publish row_s
    smem_row_to_limbs(row_s, D, limbs + (size_t)(3 * m) * D, sc, D);
    MYNN_GLUE_END();
}

// h = round(swish(gate) * up) -> limbs; gate/up rows are in_stride elements apart.  F % 8 == 0, 16-byte aligned rows.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
swiglu_limbs_kernel(int8_t *limbs, float *ascale, const T *gate, const T *up, int F, long long in_stride) {
    extern __shared__ __align__(16) float row_s[];
    __shared__ float red[40];
    MYNN_GLUE_BEGIN(2);
    pdl_trigger();
    pdl_wait();
    const int m = blockIdx.x;
    float mx = 0.f;
    bool bad = false;
    for (int i = 8 * threadIdx.x; i < F; i += 8 * kRowThreads) {
        float g[8], u[8];
        load8<T>(gate + (size_t)m * in_stride + i, g);
        load8<T>(up + (size_t)m * in_stride + i, u);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float h = round_store<T>((g[j] / (1.0f + expf(-g[j]))) * u[j]);
            row_s[i + j] = h;
            bad |= !(fabsf(h) <= 3.0e38f);
            mx = fmaxf(mx, fabsf(h));
        }
    }
    const float sc = block_limb_scale(mx, bad, ascale + m, red);
    smem_row_to_limbs(row_s, F, limbs + (size_t)(3 * m) * F, sc, F);
    MYNN_GLUE_END();
}

// The same with a row dealt out to a cluster of C CTAs (grid (C, rows), cluster (C, 1, 1), F % (8 C) == 0).  One SM needs
// about 2.5 us for the 14336 exponentials and divisions of a Llama-3-8B row; a quarter row per SM takes the operator off
// the step's critical path.  Every CTA pushes the maximum of its part into the shared memory of all CTAs of its cluster
// (remote stores, one cluster barrier), so each derives the same row scale and converts its own part.
constexpr int kSegThreads = 512;
template <typename T>
__global__ void __launch_bounds__(kSegThreads)
swiglu_limbs_cluster_kernel(int8_t *limbs, float *ascale, const T *gate, const T *up, int F, long long in_stride) {
    extern __shared__ __align__(16) float row_s[];
    __shared__ float red[40];
    __shared__ float peer_max[8];  // slot r: maximum of cluster rank r's part, negative when that part held a non-finite value
    MYNN_GLUE_BEGIN_C(2);
    pdl_trigger();
    pdl_wait();
    const int C = gridDim.x, rank = (int)cluster_ctarank(), m = blockIdx.y;
    const int seg = F / C, f0 = rank * seg;
    float mx = 0.f;
    bool bad = false;
    for (int i = 8 * threadIdx.x; i < seg; i += 8 * kSegThreads) {
        float g[8], u[8];
        load8<T>(gate + (size_t)m * in_stride + f0 + i, g);
        load8<T>(up + (size_t)m * in_stride + f0 + i, u);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float h = round_store<T>((g[j] / (1.0f + expf(-g[j]))) * u[j]);
            row_s[i + j] = h;
            bad |= !(fabsf(h) <= 3.0e38f);
            mx = fmaxf(mx, fabsf(h));
        }
    }
    mx = warp_max(mx);
    const unsigned anybad = __syncthreads_or(bad);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x < C) {  // thread r delivers this CTA's maximum to cluster rank r
        float t = 0.f;
        for (int i = 0; i < kSegThreads / 32; i++) t = fmaxf(t, red[i]);
        if (anybad) t = -1.f;
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(&peer_max[rank])), "r"((uint32_t)threadIdx.x));
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(t) : "memory");
    }
    cluster_sync_all();  // release / acquire: every part's maximum has arrived; also publishes row_s to the whole CTA
    float t = 0.f;
    bool rowbad = false;
    for (int r = 0; r < C; r++) {
        rowbad |= peer_max[r] < 0.f;
        t = fmaxf(t, peer_max[r]);
    }
    int e = 0;
    if (t > 0.f) frexpf(t, &e);
    const float sc1 = t > 0.f ? ldexpf(1.0f, 22 - e) : 1.0f;
    if (rank == 0 && threadIdx.x == 0) ascale[m] = rowbad ? __int_as_float(0x7fc00000) : 1.0f / sc1;  // non-finite input -> NaN outputs
    smem_row_to_limbs(row_s, seg, limbs + (size_t)(3 * m) * F + f0, rowbad ? 0.f : sc1, (size_t)F);
    MYNN_GLUE_END_C();
}

// Plain pre-pass in the same style (one 1024-thread CTA per row, 16-byte loads): act -> limbs.  K % 8 == 0.
template <typename T>
__global__ void __launch_bounds__(kRowThreads) act_limbs_row_kernel(int8_t *limbs, float *ascale, const T *act, int K) {
    extern __shared__ __align__(16) float row_s[];
    __shared__ float red[40];
    pdl_trigger();
    pdl_wait();
    const int m = blockIdx.x;
    float mx = 0.f;
    bool bad = false;
    for (int i = 8 * threadIdx.x; i < K; i += 8 * kRowThreads) {
        float v[8];
        load8<T>(act + (size_t)m * K + i, v);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            row_s[i + j] = v[j];
            bad |= !(fabsf(v[j]) <= 3.0e38f);
            mx = fmaxf(mx, fabsf(v[j]));
        }
    }
    const float sc = block_limb_scale(mx, bad, ascale + m, red);
    smem_row_to_limbs(row_s, K, limbs + (size_t)(3 * m) * K, sc, K);
}

// ---- host side --------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool tensor_map_api_available();
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

bool tensor_map_api_available() { return encode_fn() != nullptr; }

// 2D int8 tensor [rows][cols] (row stride = ld bytes), box = box_rows x 128 bytes, 128-byte swizzle, zero fill.
int make_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(MYNN_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld};
    cuuint32_t box[2] = {(cuuint32_t)kBlockK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MYNN_E_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return MYNN_OK;
}

static int nc_for(int M) {
    const int c = 3 * M;
    return c <= 16 ? 16 : c <= 32 ? 32 : c <= 48 ? 48 : c <= 64 ? 64 : 96;
}

int i8_gemm_limb_rows(int M) { return nc_for(M < 1 ? 1 : (M > kI8MaxRows ? kI8MaxRows : M)); }

size_t i8_gemm_workspace_bytes(int M, int K) {
    if (M <= 0 || M > kI8MaxRows || K <= 0) return 0;
    return 256 /* status word */ + 256 /* row scales */ + ((size_t)nc_for(M) * K + 255) / 256 * 256;
}

bool i8_gemm_supported(int M, int N, int K, const void *wq, int act_dtype, int out_dtype) {
    (void)act_dtype;
    return M >= 1 && M <= kI8MaxRows && K % 16 == 0 && K >= 16 && N >= 1 && ((uintptr_t)wq % 16) == 0 &&
           (out_dtype == MYNN_BF16 || out_dtype == MYNN_F16 || out_dtype == MYNN_F32) && encode_fn() != nullptr;
}

static int pick_split(int row_tiles, int kblocks) {
    // One SM ingests roughly 60-70 GB/s of tiles, so a GEMM with few row tiles cannot pull the full HBM bandwidth:
    // split K over a cluster of 2, 4 or 8 until there are about 120 CTAs, keeping at least 8 k blocks (128 KB of
    // weights) per CTA.  (Measured on the Llama-3-8B shapes at 32 rows: 4 is best for qkv, o and down.)
    int s = 1;
    while (s < 8 && row_tiles * s < 120 && kblocks / (s * 2) >= 8) s *= 2;
    return s;
}

#ifdef MYNN_TUNING
int glue_timing_read(unsigned long long *out, unsigned *n) {
    MYNN_CUDA_OK(cudaMemcpyFromSymbol(out, g_glue_t, sizeof(unsigned long long) * 3 * 1024));
    MYNN_CUDA_OK(cudaMemcpyFromSymbol(n, g_glue_n, sizeof(unsigned)));
    return MYNN_OK;
}
unsigned long long *g_i8_timing = nullptr;  // device buffer of 8 timestamps per slot, see I8GemmParams::timing
int g_i8_timing_slots = 1, g_i8_timing_next = 0;  // consecutive launches write consecutive slots (a captured graph keeps its slots)
int g_i8_stages_override = 0;
#endif

template <typename OutT, int NC>
static int launch_i8(cudaStream_t st, const CUtensorMap &mw, const CUtensorMap &ma, const I8GemmParams &p, int S) {
    constexpr uint32_t kStageBytes = kTileRows * kBlockK + ((NC * kBlockK + 1023) / 1024) * 1024;
    const size_t smem = (size_t)p.stages * kStageBytes + 1024;
    auto kern = i8_stream_gemm_kernel<OutT, NC>;
    static bool attr_set = false;
    if (!attr_set) {
        MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(kMaxStages * kStageBytes + 1024)));
        attr_set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.N + kTileRows - 1) / kTileRows, S, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = S;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may start while the limb pre-pass still runs
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    MYNN_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, mw, ma, p));
    MYNN_LAUNCH_OK("i8_stream_gemm_kernel");
    return MYNN_OK;
}

int i8_gemm_launch(cudaStream_t st, void *out, const void *act, const int8_t *wq, const void *scale, const void *resid,
                   int M, int N, int K, int act_dtype, int out_dtype, void *workspace, size_t workspace_bytes) {
    return i8_gemm_launch_tp(st, out, act, wq, scale, resid, M, N, K, act_dtype, out_dtype, workspace, workspace_bytes, nullptr, nullptr,
                             nullptr);
}

// tp: tensor-parallel form of the launch or null.  limbs_ext / ascale_ext: activation limbs that live outside the workspace
// (the workspace then only carries the status word).
int i8_gemm_launch_tp(cudaStream_t st, void *out, const void *act, const int8_t *wq, const void *scale, const void *resid,
                      int M, int N, int K, int act_dtype, int out_dtype, void *workspace, size_t workspace_bytes, const I8Tp *tp,
                      const int8_t *limbs_ext, const float *ascale_ext) {
    if (!tp && !limbs_ext && gemv_lean_supported(M, N, K, wq))  // a few rows over a small matrix: no tensor-core set-up to amortise
        return gemv_lean_launch(st, out, act, wq, scale, resid, M, N, K, act_dtype, out_dtype, workspace, workspace_bytes);
    const size_t need = limbs_ext ? 256 : i8_gemm_workspace_bytes(M, K);
    if (!workspace || workspace_bytes < need)
        return fail(MYNN_E_ARG, "dequant_matmul: workspace of %zu bytes needed, %zu given", need, workspace ? workspace_bytes : (size_t)0);
    if ((uintptr_t)workspace % 256) return fail(MYNN_E_ARG, "dequant_matmul: workspace must be 256-byte aligned");
    if (limbs_ext && (act != nullptr || !ascale_ext || (uintptr_t)limbs_ext % 16))
        return fail(MYNN_E_ARG, "dequant_matmul: external limbs need their row scales, 16-byte alignment and no activation tensor");
    const int NC = nc_for(M);
    int *status = (int *)workspace;
    float *ascale = limbs_ext ? const_cast<float *>(ascale_ext) : (float *)((char *)workspace + 256);
    int8_t *limbs = limbs_ext ? const_cast<int8_t *>(limbs_ext) : (int8_t *)workspace + 512;
    // limb rows 3M..NC-1 are padding: whatever they hold only reaches accumulator columns that are never read
    if (act != nullptr) {  // act == nullptr: a fused producer has already left limbs and row scales in the workspace
        const bool row_kernel = K % 8 == 0 && (size_t)K * 4 <= 200 * 1024 && ((uintptr_t)act % 16) == 0;
        const size_t smem = (size_t)K * 4;
#define PREP(T)                                                                                                          \
    if (row_kernel) {                                                                                                    \
        auto kern = act_limbs_row_kernel<T>;                                                                             \
        if (smem > 48 * 1024) MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        MYNN_CUDA_OK(launch_pdl(kern, dim3(M), dim3(kRowThreads), smem, st, limbs, ascale, (const T *)act, K));          \
    } else {                                                                                                             \
        MYNN_CUDA_OK(launch_pdl(act_to_limbs_kernel<T>, dim3(M), dim3(256), 0, st, limbs, ascale, (const T *)act, K));   \
    }
        switch (act_dtype) {
            case MYNN_BF16: PREP(__nv_bfloat16) break;
            case MYNN_F16: PREP(__half) break;
            case MYNN_F32: PREP(float) break;
            default: return fail(MYNN_E_ARG, "dequant_matmul: bad activation dtype %d", act_dtype);
        }
#undef PREP
        MYNN_LAUNCH_OK("act_to_limbs_kernel");
    }
    CUtensorMap mw, ma;
    int rc = make_map(&mw, wq, (uint64_t)N, (uint64_t)K, (uint64_t)K, kTileRows);
    if (rc) return rc;
    rc = make_map(&ma, limbs, (uint64_t)NC, (uint64_t)K, (uint64_t)K, (uint32_t)NC);
    if (rc) return rc;
    I8GemmParams p;
    p.out = out;
    p.scale = scale;
    p.resid = resid;
    p.ascale = ascale;
    p.M = M;
    p.N = N;
    p.K = K;
    p.status = status;
    if (tp) p.tp = *tp;
    else memset(&p.tp, 0, sizeof p.tp);
    p.skip_last_stage = 0;
    {
        int want = 1;
        if (g_inject_stall.compare_exchange_strong(want, 0)) p.skip_last_stage = 1;  // one launch only
    }
#ifdef MYNN_TUNING
    p.timing = g_i8_timing ? g_i8_timing + 32 * (size_t)(g_i8_timing_next++ % g_i8_timing_slots) : nullptr;
#endif
    const int row_tiles = (N + kTileRows - 1) / kTileRows, kblocks = (K + kBlockK - 1) / kBlockK;
    const int S = g_ksplit_override > 0 ? g_ksplit_override : pick_split(row_tiles, kblocks);
    // two CTAs per SM share 227 KB: three stages with 96 limb columns (28 KB per stage), up to five with fewer columns
    // (measured at 8 and 16 rows: a fourth stage gives 2 %, a fifth nothing)
    const int stage_bytes = kTileRows * kBlockK + ((NC * kBlockK + 1023) / 1024) * 1024;
    const int shared_stages = std::max(kStages, std::min(5, (111 * 1024) / stage_bytes));
    p.stages = (long long)row_tiles * S <= 148 ? kMaxStages : shared_stages;
#ifdef MYNN_TUNING
    if (g_i8_stages_override >= 2 && g_i8_stages_override <= kMaxStages) p.stages = g_i8_stages_override;
#endif
#define GO(OT, NCV) return launch_i8<OT, NCV>(st, mw, ma, p, S)
#define BY_NC(OT)                \
    switch (NC) {                \
        case 16: GO(OT, 16);     \
        case 32: GO(OT, 32);     \
        case 48: GO(OT, 48);     \
        case 64: GO(OT, 64);     \
        default: GO(OT, 96);     \
    }
    if (out_dtype == MYNN_BF16) BY_NC(__nv_bfloat16)
    if (out_dtype == MYNN_F16) BY_NC(__half)
    BY_NC(float)
#undef BY_NC
#undef GO
}

static int fused_ws(void *workspace, size_t workspace_bytes, int M, int K, int8_t **limbs, float **ascale) {
    if (M < 1 || M > kI8MaxRows || K % 16) return fail(MYNN_E_UNSUPPORTED, "fused limb producer: M=%d K=%d not supported", M, K);
    if (!workspace || workspace_bytes < i8_gemm_workspace_bytes(M, K) || (uintptr_t)workspace % 256)
        return fail(MYNN_E_ARG, "fused limb producer: workspace too small or misaligned");
    if ((size_t)K * 4 > 200 * 1024) return fail(MYNN_E_UNSUPPORTED, "fused limb producer: row of %d elements exceeds shared memory", K);
    *ascale = (float *)((char *)workspace + 256);
    *limbs = (int8_t *)workspace + 512;
    return MYNN_OK;
}

int launch_rms_norm_limbs(cudaStream_t st, int dtype, void *workspace, size_t workspace_bytes, void *norm_out, void *sum_out,
                          const void *x, const float *part, const void *w, float eps, int rows, int D) {
    int8_t *limbs;
    float *ascale;
    int rc = fused_ws(workspace, workspace_bytes, rows, D, &limbs, &ascale);
    if (rc) return rc;
    const size_t smem = (size_t)D * 4;
    MYNN_DISPATCH_DTYPE(dtype, T, {
        auto kern = rms_norm_limbs_kernel<T>;
        if (smem > 48 * 1024) MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        MYNN_CUDA_OK(launch_pdl(kern, dim3(rows), dim3(kRowThreads), smem, st, limbs, ascale, (T *)norm_out, (T *)sum_out, (const T *)x, part, (const T *)w, eps, D));
    });
    MYNN_LAUNCH_OK("rms_norm_limbs_kernel");
    return MYNN_OK;
}

int launch_swiglu_limbs(cudaStream_t st, int dtype, void *workspace, size_t workspace_bytes, const void *gate, const void *up,
                        int rows, int F, long long in_stride) {
    int8_t *limbs;
    float *ascale;
    int rc = fused_ws(workspace, workspace_bytes, rows, F, &limbs, &ascale);
    if (rc) return rc;
    // a cluster of C CTAs per row when the row is long enough to be worth a cluster barrier and the grid stays within one wave
    int C = 1;
    for (int c = 8; c >= 2; c >>= 1)
        if (F % (8 * c) == 0 && F / c >= 1024 && rows * c <= 148) {
            C = c;
            break;
        }
    if (C > 1) {
        const size_t smem = (size_t)(F / C) * 4;
        MYNN_DISPATCH_DTYPE(dtype, T, {
            auto kern = swiglu_limbs_cluster_kernel<T>;
            if (smem > 48 * 1024) MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(C, rows, 1);
            cfg.blockDim = dim3(kSegThreads, 1, 1);
            cfg.dynamicSmemBytes = smem;
            cfg.stream = st;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = C;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            MYNN_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, limbs, ascale, (const T *)gate, (const T *)up, F, in_stride));
        });
        MYNN_LAUNCH_OK("swiglu_limbs_cluster_kernel");
        return MYNN_OK;
    }
    const size_t smem = (size_t)F * 4;
    MYNN_DISPATCH_DTYPE(dtype, T, {
        auto kern = swiglu_limbs_kernel<T>;
        if (smem > 48 * 1024) MYNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        MYNN_CUDA_OK(launch_pdl(kern, dim3(rows), dim3(kRowThreads), smem, st, limbs, ascale, (const T *)gate, (const T *)up, F, in_stride));
    });
    MYNN_LAUNCH_OK("swiglu_limbs_kernel");
    return MYNN_OK;
}

}  // namespace mynn
