// Whole decoder step behind the engine's generated-library entry points (model_init / model / model_destroy).
//
// The engine generates one CUDA library per model and resolves those three symbols from it; the decoder DAG it
// generates for a Llama-family model is fixed (crates/llm/src/decoder.rs:203-537,731-865), so here it is written
// once and specialised by mynn_b200_model_configure().  Per layer the step launches
//     RMSNorm -> QKV DequantMatMul (one launch when the three weights are adjacent in memory) -> RoPE + KV append
//     -> GQA decode attention -> O DequantMatMul (+ residual) -> RMSNorm -> gate/up DequantMatMul -> Swish*Mul
//     -> down DequantMatMul (+ residual)
// on ONE stream (the DAG is a chain; the engine's 16-stream plan only adds event traffic) and captures the whole
// step in a CUDA graph that is replayed every token: sequence position, KV offset and active length live in
// device scalars, so the graph never changes.  Activations live in one arena sized at init; weights and KV
// caches belong to the host, as in the engine.  Every rounding point of the engine's schedule is kept (one
// rounding per kernel output), so greedy tokens can be compared with the CPU oracle.
//
// Tensor parallel (tp_world > 1): q/k/v/gate/up/lm_head shards are column-parallel (rows of wq), o/down are
// row-parallel (columns of wq) and produce f32 partial sums that are all-reduced and then rounded once and added
// to the residual, fused with the following RMSNorm.
#include <algorithm>
#include <cstring>
#include <vector>

#include "comm.cuh"
#include "common.cuh"
#include "i8_gemm.cuh"
#include "ops_internal.cuh"
#include "tp_fused.cuh"

extern "C" void model_destroy(void *state);

namespace mynn {

struct LayerW {
    const void *ln1, *ln2;
    const int8_t *wq, *wk, *wv, *wo, *wg, *wu, *wd;
    const void *sq, *sk, *sv, *so, *sg, *su, *sd;
    void *kc, *vc;
    void *ksc, *vsc;  // per-token scales of an int8 cache
    bool qkv_fused, gu_fused;
};

struct Model {
    mynn_b200_model_config c;
    int Hq, Hkv, ffn, vocab_l;  // per-rank sizes
    int max_rows;               // batch * max(1, max_prefill)
    std::vector<LayerW> layers;
    const int8_t *embed;
    const void *embed_scale, *final_norm, *lm_scale, *cos_t, *sin_t;
    const int8_t *lm_w;
    // device buffers
    char *arena = nullptr;
    // step inputs, contiguous so that one host-to-device copy delivers them: {past, active, pos0, ids[rows]}
    int32_t *past_dev, *active_dev;
    int64_t *pos0_dev, *ids_dev;
    int64_t *pos_dev;  // positions of a prefill chunk
    int32_t *tok_dev;
    char *h_in = nullptr;  // pinned mirror of the input block
    int *h_status = nullptr;  // pinned: status words of the GEMM workspace and of the tensor-parallel block, fetched with the result
    void *x, *n, *qkv, *q_rot, *attn, *gu, *h, *last_x, *logits, *logits_full;
    float *part, *pairs, *pairs_all;  // part = f32 partial sums of a row-parallel product (tp_world > 1, ncclAllReduce path)
    char *tp_block = nullptr;         // cudaMalloc'd block shared with the peers (fused reduction of decode steps, tp_fused.cuh)
    size_t tp_block_bytes = 0;
    TpPeers tp = {};
    bool tp_attached = false;
    bool weights_aligned = false;  // every projection weight is 16-byte aligned (the TMA-fed kernels can take all of them)
    void *attn_ws, *gemm_ws;
    size_t attn_ws_bytes, gemm_ws_bytes;
    // streaming (sink + ring) cache: per-slot key positions and the scratch that holds one layer's rotated keys
    int64_t *kvpos_dev = nullptr;
    void *k_rot = nullptr;
    void *k_deq = nullptr, *v_deq = nullptr;  // int8 cache: 16-bit copy of one layer's live rows for the tensor-core prefill attention
    cudaGraphExec_t stream_graph_exec = nullptr;
    bool tc_attention_ran = false;  // the step just enqueued went through the tcgen05 prefill attention (its status word is checked)
    cudaStream_t stream = nullptr;
    cudaGraphExec_t graph_exec = nullptr;
};

static mynn_b200_model_config g_cfg;
static bool g_cfg_set = false;
static int g_status = MYNN_OK;

static size_t up256(size_t x) { return (x + 255) / 256 * 256; }

#define RC(expr)            \
    do {                    \
        int rc__ = (expr);  \
        if (rc__) return rc__; \
    } while (0)

// DequantMatMul over any number of rows: the streaming kernel takes up to 32 rows per pass.
static int gemm(cudaStream_t st, const Model &m, void *out, const void *act, const int8_t *w, const void *scale,
                const void *resid, int M, int N, int K, int out_dtype) {
    const int dt = m.c.dtype;
    const size_t esz = dtype_size(dt), osz = dtype_size(out_dtype);
    if (M > 32 && m.gemm_ws && m.gemm_ws_bytes >= mynn_b200_dequant_matmul_workspace_bytes(M, N, K)) {
        // prefill: one launch of the large-tile tensor-core kernel over all rows
        if (resid) return mynn_b200_dequant_matmul_residual(st, out, act, w, scale, resid, M, N, K, dt, m.gemm_ws, m.gemm_ws_bytes);
        return mynn_b200_dequant_matmul(st, out, act, w, scale, M, N, K, dt, out_dtype, MYNN_W_NK, m.gemm_ws, m.gemm_ws_bytes);
    }
    for (int m0 = 0; m0 < M; m0 += 32) {
        const int mm = M - m0 < 32 ? M - m0 : 32;
        char *o = (char *)out + (size_t)m0 * N * osz;
        const char *a = (const char *)act + (size_t)m0 * K * esz;
        if (resid) {
            RC(mynn_b200_dequant_matmul_residual(st, o, a, w, scale, (const char *)resid + (size_t)m0 * N * osz, mm, N, K, dt,
                                                 m.gemm_ws, m.gemm_ws_bytes));
        } else {
            RC(mynn_b200_dequant_matmul(st, o, a, w, scale, mm, N, K, dt, out_dtype, MYNN_W_NK, m.gemm_ws, m.gemm_ws_bytes));
        }
    }
    return MYNN_OK;
}

// DequantMatMul whose activations a fused producer has already left as limbs in the GEMM workspace.
static int gemm_prequant(cudaStream_t st, const Model &m, void *out, const int8_t *w, const void *scale, const void *resid,
                         int M, int N, int K, int out_dtype) {
    return i8_gemm_launch(st, out, nullptr, w, scale, resid, M, N, K, m.c.dtype, out_dtype, m.gemm_ws, m.gemm_ws_bytes);
}

// The same for more than 32 rows: two limbs per element in the layout of the prefill kernel.
static int gemm_prequant2(cudaStream_t st, const Model &m, void *out, const int8_t *w, const void *scale, const void *resid,
                          int M, int N, int K, int out_dtype) {
    return i8_prefill_launch(st, out, nullptr, w, scale, resid, M, N, K, m.c.dtype, out_dtype, m.gemm_ws, m.gemm_ws_bytes);
}

// Enqueue one forward pass over S tokens per sequence (S == 1: decode).  Inputs are the device buffers
// ids_dev [B*S], pos0_dev / pos_dev [S], past_dev, active_dev.  Leaves logits (and token ids) in device buffers.
// When the step has at most 32 rows and the int8 tensor-core GEMM is enabled, RMSNorm and Swish*Mul write their
// (rounded) outputs directly as activation limbs into the GEMM workspace, so no separate pre-pass runs for the
// q/k/v, gate/up, down and lm_head products.
static int enqueue_forward(Model &m, cudaStream_t st, int S) {
    const mynn_b200_model_config &c = m.c;
    const int B = c.batch, H = c.hidden, D = c.head_dim, dt = c.dtype;
    const int M = B * S;
    const int tp = c.tp_world;
    const size_t esz = dtype_size(dt);
    const int Nq = m.Hq * D, Nkv = m.Hkv * D;
    const float attn_scale = 1.0f / sqrtf((float)D);
    const bool fused = m.gemm_ws != nullptr && M <= kI8MaxRows && H % 16 == 0 && m.ffn % 16 == 0 &&
                       (size_t)std::max(H, m.ffn) * 4 <= 200 * 1024;
    // decode steps of a tensor-parallel model: the reduction fused with its neighbours over peer memory (tp_fused.cuh)
    const bool tp_fused = tp > 1 && m.tp_attached && fused && S == 1 && M <= m.tp.lay.max_rows && Nq % 16 == 0 && m.weights_aligned;
    bool reduced_limbs = false;  // a fused reduction left the limbs of the next product in the workspace

    // prefill chunks (more than 32 rows): RMSNorm and Swish*Mul write the two limbs of the prefill kernel themselves
    if (S >= 64 && dt != MYNN_F32 && (D == 64 || D == 128)) m.tc_attention_ran = true;  // the attention launcher may pick the tcgen05 kernels
    const bool fused2 = m.gemm_ws != nullptr && M > kI8MaxRows && dt != MYNN_F32 && m.weights_aligned && tensor_map_api_available() &&
                        H % 16 == 0 && m.ffn % 16 == 0 && (size_t)std::max(H, m.ffn) * 4 <= 200 * 1024 &&
                        m.gemm_ws_bytes >= i8_prefill_workspace_bytes(M, std::max(H, m.ffn));
    bool n_limbs2 = false;  // the last norm left two-limb rows in the workspace instead of m.n

    // norm(x [+ part]) feeding a DequantMatMul: either limbs in the workspace (fused) or the bf16 tensor m.n
    auto push = [&](int buf, const void *act, const int8_t *w, const void *scale, int K) -> int {  // row-parallel product
        int skip = 0, want = 2;
        if (g_inject_stall.compare_exchange_strong(want, 0)) skip = 1;  // test aid: this launch delivers nothing
        return launch_tp_gemm_push(st, m.tp, buf, act, w, (const float *)scale, M, H, K, dt, m.gemm_ws, m.gemm_ws_bytes, skip);
    };
    auto reduce = [&](int buf, const void *w) -> int {  // fused reduction of the partial sums in buffer `buf`
        reduced_limbs = w != nullptr;
        return launch_tp_reduce_norm_limbs(st, dt, m.tp, buf, m.gemm_ws, m.gemm_ws_bytes, m.x, w, c.rms_eps, M, true);  // always right behind its push
    };
    auto norm = [&](const void *w, const float *part, int rows, const void *src) -> int {
        n_limbs2 = false;
        reduced_limbs = false;
        if (fused && rows <= kI8MaxRows)
            return launch_rms_norm_limbs(st, dt, m.gemm_ws, m.gemm_ws_bytes, nullptr, part ? m.x : nullptr, src, part, w,
                                         c.rms_eps, rows, H);
        if (part) return launch_add_f32_rms_norm(st, dt, m.x, m.n, m.x, part, w, c.rms_eps, rows, H);
        if (fused2 && rows == M && prefill_fused_supported(dt, H, src, w)) {
            n_limbs2 = true;
            return launch_rms_norm_limbs2(st, dt, m.gemm_ws, m.gemm_ws_bytes, src, w, c.rms_eps, rows, H);
        }
        return mynn_b200_rms_norm(st, m.n, src, w, c.rms_eps, rows, H, dt);
    };
    auto gemm_n = [&](void *out, const int8_t *w, const void *scale, int rows, int N, int out_dtype) -> int {
        if (reduced_limbs) return gemm_prequant(st, m, out, w, scale, nullptr, rows, N, H, out_dtype);
        if (fused && rows <= kI8MaxRows) return gemm_prequant(st, m, out, w, scale, nullptr, rows, N, H, out_dtype);
        if (n_limbs2) return gemm_prequant2(st, m, out, w, scale, nullptr, rows, N, H, out_dtype);
        return gemm(st, m, out, m.n, w, scale, nullptr, rows, N, H, out_dtype);
    };

    RC(mynn_b200_embed_gather_dequant(st, m.x, m.embed, m.embed_scale, m.ids_dev, M, H, c.vocab, dt));
    RC(norm(m.layers[0].ln1, nullptr, M, m.x));
    for (int l = 0; l < c.n_layers; l++) {
        const LayerW &L = m.layers[l];
        // --- attention block ---
        char *qb = (char *)m.qkv;
        bool attn_limbs = false;
        long long qs, ks, vs;
        const char *kb, *vb;
        if (L.qkv_fused) {
            const int Nt = Nq + 2 * Nkv;
            RC(gemm_n(qb, L.wq, L.sq, M, Nt, dt));
            qs = ks = vs = Nt;
            kb = qb + (size_t)Nq * esz;
            vb = qb + (size_t)(Nq + Nkv) * esz;
        } else {
            char *k_ = qb + (size_t)M * Nq * esz, *v_ = k_ + (size_t)M * Nkv * esz;
            RC(gemm_n(qb, L.wq, L.sq, M, Nq, dt));
            RC(gemm_n(k_, L.wk, L.sk, M, Nkv, dt));
            RC(gemm_n(v_, L.wv, L.sv, M, Nkv, dt));
            qs = Nq;
            ks = vs = Nkv;
            kb = k_;
            vb = v_;
        }
        if (c.kv_int8 && c.stream_window > 0) {
            // streaming int8 cache: K is quantized UNROTATED into its slot (past_dev holds the slot); the attention kernel
            // rotates every live key in f32 at the position the per-slot table gives (the engine's in-kernel RoPE operands,
            // crates/llm/src/decoder.rs:314-326).  The live rows are the slots [0, active): no ring remapping is needed, the
            // softmax does not depend on the order of the rows, and a chunk never evicts, so a causal bound by slot is the bound
            // by rank.
            RC(launch_rope_kv_append_q8(st, dt, m.q_rot, L.kc, L.vc, L.ksc, L.vsc, qb, kb, vb, qs, ks, vs, m.cos_t, m.sin_t,
                                        S == 1 ? m.pos0_dev : m.pos_dev, B, S, m.Hq, m.Hkv, D, c.max_seq_len, m.past_dev, 0));
            RC(launch_attention_streaming(st, m.attn, m.q_rot, L.kc, L.vc, L.ksc, L.vsc, attn_scale, B, m.Hq, m.Hkv, S, D, c.max_seq_len,
                                          c.max_seq_len, m.active_dev, S > 1, 0, 0, 0, m.cos_t, m.sin_t, m.kvpos_dev, dt, 1, 1));
        } else if (c.kv_int8) {
            RC(launch_rope_kv_append_q8(st, dt, m.q_rot, L.kc, L.vc, L.ksc, L.vsc, qb, kb, vb, qs, ks, vs, m.cos_t, m.sin_t,
                                        S == 1 ? m.pos0_dev : m.pos_dev, B, S, m.Hq, m.Hkv, D, c.max_seq_len, m.past_dev));
            if (S >= 64 && m.k_deq &&
                attention_prefill_tc_supported(B, m.Hq, m.Hkv, S, D, c.max_seq_len, dt, m.q_rot, m.k_deq, m.v_deq, m.attn)) {
                // a long prefill chunk: the tensor-core kernel over a 16-bit copy of the live rows (value * row scale, rounded
                // once, i.e. what a 16-bit cache would hold for these quantised rows)
                RC(launch_dequant_kv_rows(st, dt, m.k_deq, L.kc, L.ksc, B * m.Hkv, c.max_seq_len, D, 0, m.active_dev));
                RC(launch_dequant_kv_rows(st, dt, m.v_deq, L.vc, L.vsc, B * m.Hkv, c.max_seq_len, D, 0, m.active_dev));
                RC(launch_attention(st, m.attn, m.q_rot, m.k_deq, m.v_deq, attn_scale, B, m.Hq, m.Hkv, S, D, c.max_seq_len,
                                    c.max_seq_len, m.active_dev, 1, dt, m.attn_ws, m.attn_ws_bytes, 1));
            } else {
                RC(launch_attention_q8(st, m.attn, m.q_rot, L.kc, L.vc, L.ksc, L.vsc, attn_scale, B, m.Hq, m.Hkv, S, D,
                                       c.max_seq_len, c.max_seq_len, m.active_dev, S > 1, dt, m.attn_ws, m.attn_ws_bytes, 1));
            }
        } else if (c.stream_window > 0) {
            // streaming cache: K is appended unrotated at the slot in past_dev; the live rows are rotated at their
            // recency rank into the scratch copy that attention reads.  The live rows are the slots [0, active).
            RC(launch_rope_kv_append(st, dt, m.q_rot, L.kc, L.vc, qb, kb, vb, qs, ks, vs, m.cos_t, m.sin_t,
                                     S == 1 ? m.pos0_dev : m.pos_dev, B, S, m.Hq, m.Hkv, D, c.max_seq_len, m.past_dev, 0));
            RC(launch_rope_cache_rows(st, dt, m.k_rot, L.kc, m.cos_t, m.sin_t, m.kvpos_dev, B * m.Hkv, c.max_seq_len, D, 0, m.active_dev));
            RC(launch_attention(st, m.attn, m.q_rot, m.k_rot, L.vc, attn_scale, B, m.Hq, m.Hkv, S, D, c.max_seq_len,
                                c.max_seq_len, m.active_dev, S > 1, dt, m.attn_ws, m.attn_ws_bytes, 1));
        } else {
            // decode: the attention kernel also leaves its output rows as the activation limbs of o_proj
            attn_limbs = fused && S == 1 && Nq % 16 == 0 && (size_t)Nq * 4 <= 200 * 1024 &&
                         attention_decode_fast_path(S, D, m.Hq, m.Hkv, dt, qb, L.kc, L.vc);
            // ... and rotates q and the new key and appends the new key / value rows itself (one launch less per layer), when
            // the projection output is one block whose rows and heads are 16-byte aligned
            const bool fuse_rope = g_fuse_rope && attn_limbs && L.qkv_fused && qs % 8 == 0 && D % 32 == 0 &&
                                   (((uintptr_t)kb | (uintptr_t)vb) % 16) == 0;
            if (fuse_rope) {
                const AttentionFuse fz = {kb, vb, qs, m.cos_t, m.sin_t, m.pos0_dev, m.past_dev};
                RC(launch_attention(st, m.attn, qb, L.kc, L.vc, attn_scale, B, m.Hq, m.Hkv, S, D, c.max_seq_len, c.max_seq_len,
                                    m.active_dev, 0, dt, m.attn_ws, m.attn_ws_bytes, 1, (int8_t *)m.gemm_ws + 512,
                                    (float *)((char *)m.gemm_ws + 256), &fz, (int *)m.gemm_ws));
            } else {
                RC(launch_rope_kv_append(st, dt, m.q_rot, L.kc, L.vc, qb, kb, vb, qs, ks, vs, m.cos_t, m.sin_t,
                                         S == 1 ? m.pos0_dev : m.pos_dev, B, S, m.Hq, m.Hkv, D, c.max_seq_len, m.past_dev));
                attn_limbs = attn_limbs && attention_decode_fast_path(S, D, m.Hq, m.Hkv, dt, m.q_rot, L.kc, L.vc);
                RC(launch_attention(st, m.attn, m.q_rot, L.kc, L.vc, attn_scale, B, m.Hq, m.Hkv, S, D, c.max_seq_len,
                                    c.max_seq_len, m.active_dev, S > 1, dt, m.attn_ws, m.attn_ws_bytes, 1,
                                    attn_limbs ? (int8_t *)m.gemm_ws + 512 : nullptr, attn_limbs ? (float *)((char *)m.gemm_ws + 256) : nullptr,
                                    nullptr, (int *)m.gemm_ws));
            }
        }
        if (tp == 1) {
            // x = round(x + round(o))
            if (attn_limbs) {
                RC(gemm_prequant(st, m, m.x, L.wo, L.so, m.x, M, H, Nq, dt));
            } else if (fused2 && Nq <= 8192) {
                // a prefill chunk with a short reduction: the residual add inside the tensor-core kernel's epilogue (2-byte
                // accesses, one weight row per thread) takes longer than the main loop of such a tile; the product alone
                // into m.n (free here) and a 128-bit add cost less.  Same roundings: round(x + round(o)).
                RC(gemm(st, m, m.n, m.attn, L.wo, L.so, nullptr, M, H, Nq, dt));
                RC(mynn_b200_add(st, m.x, m.x, m.n, (int64_t)M * H, dt));
            } else {
                RC(gemm(st, m, m.x, m.attn, L.wo, L.so, m.x, M, H, Nq, dt));
            }
            RC(norm(L.ln2, nullptr, M, m.x));
        } else if (tp_fused) {
            // the partial sums go straight into every rank's memory; each rank then sums, adds, norms and writes the limbs
            RC(push(0, attn_limbs ? nullptr : m.attn, L.wo, L.so, Nq));
            RC(reduce(0, L.ln2));
        } else {
            if (attn_limbs) RC(gemm_prequant(st, m, m.part, L.wo, L.so, nullptr, M, H, Nq, MYNN_F32));
            else RC(gemm(st, m, m.part, m.attn, L.wo, L.so, nullptr, M, H, Nq, MYNN_F32));
            RC(comm_all_reduce(st, m.part, m.part, (size_t)M * H, MYNN_F32));
            RC(norm(L.ln2, m.part, M, m.x));  // x = round(x + round(sum of partials)), then the norm
        }
        // --- MLP block ---
        const bool fuse_mlp = fused && L.gu_fused;
        bool h_limbs2 = false;  // Swish*Mul left two-limb rows in the workspace instead of m.h
        if (L.gu_fused) {
            RC(gemm_n(m.gu, L.wg, L.sg, M, 2 * m.ffn, dt));
            const char *up_ = (char *)m.gu + (size_t)m.ffn * esz;
            if (fuse_mlp) {
                RC(launch_swiglu_limbs(st, dt, m.gemm_ws, m.gemm_ws_bytes, m.gu, up_, M, m.ffn, 2LL * m.ffn));
            } else if (fused2 && prefill_fused_supported(dt, m.ffn, m.gu, up_)) {
                RC(launch_swiglu_limbs2(st, dt, m.gemm_ws, m.gemm_ws_bytes, m.gu, up_, M, m.ffn, 2LL * m.ffn));
                h_limbs2 = true;
            } else {
                RC(launch_swiglu_strided(st, dt, m.h, m.gu, up_, M, m.ffn, 2LL * m.ffn));
            }
        } else {
            char *u_ = (char *)m.gu + (size_t)M * m.ffn * esz;
            RC(gemm_n(m.gu, L.wg, L.sg, M, m.ffn, dt));
            RC(gemm_n(u_, L.wu, L.su, M, m.ffn, dt));
            if (fused2 && prefill_fused_supported(dt, m.ffn, m.gu, u_)) {
                RC(launch_swiglu_limbs2(st, dt, m.gemm_ws, m.gemm_ws_bytes, m.gu, u_, M, m.ffn, m.ffn));
                h_limbs2 = true;
            } else {
                RC(launch_swiglu_strided(st, dt, m.h, m.gu, u_, M, m.ffn, m.ffn));
            }
        }
        const bool last = l + 1 == c.n_layers;
        const void *next_norm = last ? nullptr : m.layers[l + 1].ln1;
        if (tp == 1) {
            if (fuse_mlp) RC(gemm_prequant(st, m, m.x, L.wd, L.sd, m.x, M, H, m.ffn, dt));
            else if (h_limbs2) RC(gemm_prequant2(st, m, m.x, L.wd, L.sd, m.x, M, H, m.ffn, dt));
            else RC(gemm(st, m, m.x, m.h, L.wd, L.sd, m.x, M, H, m.ffn, dt));
            if (!last) RC(norm(next_norm, nullptr, M, m.x));
        } else if (tp_fused) {
            RC(push(1, fuse_mlp ? nullptr : m.h, L.wd, L.sd, m.ffn));
            RC(reduce(1, last ? m.final_norm : next_norm));  // after the last layer: the final norm, whose rows feed lm_head
        } else {
            if (fuse_mlp) RC(gemm_prequant(st, m, m.part, L.wd, L.sd, nullptr, M, H, m.ffn, MYNN_F32));
            else if (h_limbs2) RC(gemm_prequant2(st, m, m.part, L.wd, L.sd, nullptr, M, H, m.ffn, MYNN_F32));
            else RC(gemm(st, m, m.part, m.h, L.wd, L.sd, nullptr, M, H, m.ffn, MYNN_F32));
            RC(comm_all_reduce(st, m.part, m.part, (size_t)M * H, MYNN_F32));
            if (last) RC(launch_add_f32_rms_norm(st, dt, m.x, nullptr, m.x, m.part, nullptr, c.rms_eps, M, H));
            else RC(norm(next_norm, m.part, M, m.x));
        }
    }
    // --- head: only the last token of each sequence is needed ---
    const void *xl = m.x;
    if (S > 1) {
        MYNN_CUDA_OK(cudaMemcpy2DAsync(m.last_x, (size_t)H * esz, (const char *)m.x + (size_t)(S - 1) * H * esz,
                                       (size_t)S * H * esz, (size_t)H * esz, B, cudaMemcpyDeviceToDevice, st));
        xl = m.last_x;
    }
    const bool fused_head = m.gemm_ws != nullptr && B <= kI8MaxRows && H % 16 == 0 && (size_t)H * 4 <= 200 * 1024;
    if (reduced_limbs) {  // the last fused reduction applied the final norm and left its limbs
        RC(gemm_prequant(st, m, m.logits, m.lm_w, m.lm_scale, nullptr, B, m.vocab_l, H, dt));
    } else if (fused_head) {
        RC(launch_rms_norm_limbs(st, dt, m.gemm_ws, m.gemm_ws_bytes, nullptr, nullptr, xl, nullptr, m.final_norm, c.rms_eps, B, H));
        RC(gemm_prequant(st, m, m.logits, m.lm_w, m.lm_scale, nullptr, B, m.vocab_l, H, dt));
    } else {
        RC(mynn_b200_rms_norm(st, m.n, xl, m.final_norm, c.rms_eps, B, H, dt));
        RC(gemm(st, m, m.logits, m.n, m.lm_w, m.lm_scale, nullptr, B, m.vocab_l, H, dt));
    }
    if (c.output_mode == 1) {
        if (tp == 1) {
            if (m.vocab_l >= 16384) RC(launch_argmax_two_stage(st, dt, m.tok_dev, m.pairs_all, m.logits, B, m.vocab_l, 16));
            else RC(mynn_b200_argmax_last(st, m.tok_dev, m.logits, B, m.vocab_l, dt));
        } else {
            RC(launch_argmax_pairs(st, dt, m.pairs, m.logits, B, m.vocab_l, c.tp_rank * m.vocab_l));
            RC(comm_all_gather(st, m.pairs_all, m.pairs, (size_t)B * 2 * sizeof(float)));
            RC(launch_argmax_merge(st, m.tok_dev, m.pairs_all, B, tp));
        }
        if (S == 1) RC(launch_tok_feedback(st, m.ids_dev, m.tok_dev, B));  // next step may reuse the resident ids
    } else if (tp > 1) {
        RC(comm_all_gather(st, m.logits_full, m.logits, (size_t)B * m.vocab_l * esz));
    }
    return MYNN_OK;
}

static int model_create(Model **out, void **initializer, void **session_state) {
    if (!g_cfg_set) return fail(MYNN_E_STATE, "model_init: call mynn_b200_model_configure first");
    if (!initializer || !session_state) return fail(MYNN_E_ARG, "model_init: null pointer table");
    Model *m = new Model();
    m->c = g_cfg;
    const mynn_b200_model_config &c = m->c;
    const int tp = c.tp_world;
    m->Hq = c.n_heads / tp;
    m->Hkv = c.n_kv_heads / tp;
    m->ffn = c.ffn / tp;
    m->vocab_l = c.vocab / tp;
    const int prefill = c.max_prefill > 0 ? c.max_prefill : 1;
    m->max_rows = c.batch * prefill;
    const size_t esz = dtype_size(c.dtype);
    const int D = c.head_dim, H = c.hidden;

    int i = 0;
    m->embed = (const int8_t *)initializer[i++];
    m->embed_scale = initializer[i++];
    m->layers.resize(c.n_layers);
    for (int l = 0; l < c.n_layers; l++) {
        LayerW &L = m->layers[l];
        L.ln1 = initializer[i++];
        L.wq = (const int8_t *)initializer[i++]; L.sq = initializer[i++];
        L.wk = (const int8_t *)initializer[i++]; L.sk = initializer[i++];
        L.wv = (const int8_t *)initializer[i++]; L.sv = initializer[i++];
        L.wo = (const int8_t *)initializer[i++]; L.so = initializer[i++];
        L.ln2 = initializer[i++];
        L.wg = (const int8_t *)initializer[i++]; L.sg = initializer[i++];
        L.wu = (const int8_t *)initializer[i++]; L.su = initializer[i++];
        L.wd = (const int8_t *)initializer[i++]; L.sd = initializer[i++];
        const int per_layer = c.kv_int8 ? 4 : 2;
        L.kc = session_state[per_layer * l];
        L.vc = session_state[per_layer * l + 1];
        L.ksc = c.kv_int8 ? session_state[4 * l + 2] : nullptr;
        L.vsc = c.kv_int8 ? session_state[4 * l + 3] : nullptr;
        if (!L.kc || !L.vc || (c.kv_int8 && (!L.ksc || !L.vsc))) {
            delete m;
            return fail(MYNN_E_ARG, "model_init: a KV buffer of layer %d is null", l);
        }
        const size_t nq = (size_t)m->Hq * D, nkv = (size_t)m->Hkv * D;
        L.qkv_fused = L.wk == L.wq + nq * H && L.wv == L.wk + nkv * H &&
                      (const char *)L.sk == (const char *)L.sq + nq * esz &&
                      (const char *)L.sv == (const char *)L.sk + nkv * esz;
        L.gu_fused = L.wu == L.wg + (size_t)m->ffn * H && (const char *)L.su == (const char *)L.sg + (size_t)m->ffn * esz;
    }
    m->weights_aligned = true;
    for (const LayerW &L : m->layers)
        for (const int8_t *wp : {L.wq, L.wk, L.wv, L.wo, L.wg, L.wu, L.wd})
            if ((uintptr_t)wp % 16) m->weights_aligned = false;
    m->final_norm = initializer[i++];
    m->lm_w = (const int8_t *)initializer[i++];
    m->lm_scale = initializer[i++];
    m->cos_t = initializer[i++];
    m->sin_t = initializer[i++];
    for (int j = 0; j < i; j++)
        if (!initializer[j]) {
            delete m;
            return fail(MYNN_E_ARG, "model_init: initializer %d is null", j);
        }

    // ---- activation arena ----
    const size_t R = m->max_rows;
    const size_t nqkv = (size_t)(m->Hq + 2 * m->Hkv) * D;
    m->attn_ws_bytes = mynn_b200_attention_workspace_bytes(c.batch, m->Hq, m->Hkv, D, c.max_seq_len);
    {
        const int kmax = std::max(std::max(H, m->ffn), m->Hq * D);
        m->gemm_ws_bytes = c.use_tensor_gemm ? mynn_b200_dequant_matmul_workspace_bytes(32, 0, kmax) : 0;
        if (c.use_tensor_gemm && m->max_rows > 32)
            m->gemm_ws_bytes = std::max(m->gemm_ws_bytes, mynn_b200_dequant_matmul_workspace_bytes(m->max_rows, 0, kmax));
    }
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += up256(bytes); return o; };
    const size_t o_in = take(16 + R * 8), o_pos = take((size_t)prefill * 8), o_tok = take((size_t)c.batch * 4), o_x = take(R * H * esz), o_n = take(R * H * esz),
                 o_qkv = take(R * nqkv * esz), o_qrot = take(R * m->Hq * D * esz), o_attn = take(R * m->Hq * D * esz),
                 o_gu = take(R * 2 * m->ffn * esz), o_h = take(R * m->ffn * esz), o_last = take((size_t)c.batch * H * esz),
                 o_logits = take((size_t)c.batch * m->vocab_l * esz),
                 o_full = take(tp > 1 ? (size_t)c.batch * c.vocab * esz : 0), 
                 o_pairs = take((size_t)c.batch * 8), o_pairs_all = take((size_t)c.batch * 8 * std::max(tp, 16)),
                 o_ws = take(m->attn_ws_bytes), o_gws = take(m->gemm_ws_bytes), o_part = take(tp > 1 ? R * H * 4 : 0),
                 o_kvpos = take(c.stream_window > 0 ? (size_t)c.max_seq_len * 8 : 0),
                 o_krot = take(c.stream_window > 0 && !c.kv_int8 ? (size_t)c.batch * m->Hkv * c.max_seq_len * D * esz : 0);
    const bool want_deq = c.kv_int8 && prefill >= 64 && c.dtype != MYNN_F32 && (D == 64 || D == 128);
    const size_t deq_bytes = want_deq ? (size_t)c.batch * m->Hkv * c.max_seq_len * D * esz : 0;
    const size_t o_kdeq = take(deq_bytes), o_vdeq = take(deq_bytes);
    cudaError_t e = cudaMalloc(&m->arena, off);
    if (e != cudaSuccess) {
        delete m;
        return fail(MYNN_E_CUDA, "model_init: cudaMalloc(%zu) failed: %s", off, cudaGetErrorString(e));
    }
    cudaMemset(m->arena, 0, off);
    char *a = m->arena;
    m->past_dev = (int32_t *)(a + o_in);
    m->active_dev = (int32_t *)(a + o_in + 4);
    m->pos0_dev = (int64_t *)(a + o_in + 8);
    m->ids_dev = (int64_t *)(a + o_in + 16);
    m->pos_dev = (int64_t *)(a + o_pos);
    m->tok_dev = (int32_t *)(a + o_tok);
    m->x = a + o_x; m->n = a + o_n; m->qkv = a + o_qkv; m->q_rot = a + o_qrot; m->attn = a + o_attn;
    m->gu = a + o_gu; m->h = a + o_h; m->last_x = a + o_last; m->logits = a + o_logits;
    m->logits_full = a + o_full; m->pairs = (float *)(a + o_pairs);
    m->pairs_all = (float *)(a + o_pairs_all); m->attn_ws = a + o_ws;
    m->gemm_ws = m->gemm_ws_bytes ? a + o_gws : nullptr;
    m->kvpos_dev = (int64_t *)(a + o_kvpos);
    m->k_rot = a + o_krot;
    m->k_deq = want_deq ? a + o_kdeq : nullptr;
    m->v_deq = want_deq ? a + o_vdeq : nullptr;
    m->part = tp > 1 ? (float *)(a + o_part) : nullptr;
    if (tp > 1 && c.use_tensor_gemm && c.batch <= kI8MaxRows && H % 16 == 0) {
        // the block the fused reduction of decode steps shares with the peers (tp_fused.cuh); without it the step uses NCCL
        m->tp.lay = tp_layout(c.batch, H, tp);
        m->tp_block_bytes = m->tp.lay.bytes;
        e = cudaMalloc(&m->tp_block, m->tp_block_bytes);
        if (e != cudaSuccess) {
            cudaFree(m->arena);
            delete m;
            return fail(MYNN_E_CUDA, "model_init: cudaMalloc of the peer-shared block failed: %s", cudaGetErrorString(e));
        }
        tp_block_init(nullptr, m->tp_block, m->tp_block_bytes);  // header zero, partial sums EMPTY; ordered by the synchronise below
        m->tp.rank = c.tp_rank;
        m->tp.world = tp;
        m->tp.blocks[c.tp_rank] = m->tp_block;
    }
    e = cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMallocHost((void **)&m->h_in, 16 + R * 8);
    if (e == cudaSuccess) e = cudaMallocHost((void **)&m->h_status, 2 * sizeof(int));
    if (e != cudaSuccess) {
        cudaFree(m->arena);
        delete m;
        return fail(MYNN_E_CUDA, "model_init: stream / pinned buffer creation failed: %s", cudaGetErrorString(e));
    }
    // the zero fills above ran on the legacy stream, the model's stream does not wait for it implicitly: finish them before the
    // first step and before a peer can map the shared block
    e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        model_destroy(m);
        return fail(MYNN_E_CUDA, "model_init: %s", cudaGetErrorString(e));
    }
    *out = m;
    return MYNN_OK;
}

// Run the decode step from device-resident inputs already in ids_dev/pos_dev/past_dev/active_dev.
static int run_decode(Model &m, cudaStream_t st) {
    if (!m.c.use_graph) return enqueue_forward(m, st, 1);
    if (!m.graph_exec) {
        cudaGraph_t graph = nullptr;
        MYNN_CUDA_OK(cudaStreamBeginCapture(m.stream, cudaStreamCaptureModeThreadLocal));
        int rc = enqueue_forward(m, m.stream, 1);
        cudaError_t e = cudaStreamEndCapture(m.stream, &graph);
        if (rc) {
            if (graph) cudaGraphDestroy(graph);
            return rc;
        }
        if (e != cudaSuccess) return fail(MYNN_E_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
        e = cudaGraphInstantiate(&m.graph_exec, graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) return fail(MYNN_E_CUDA, "graph instantiation failed: %s", cudaGetErrorString(e));
    }
    MYNN_CUDA_OK(cudaGraphLaunch(m.graph_exec, st));
    return MYNN_OK;
}

static const void *result_ptr(const Model &m, size_t *bytes) {
    if (m.c.output_mode == 1) {
        *bytes = (size_t)m.c.batch * 4;
        return m.tok_dev;
    }
    *bytes = (size_t)m.c.batch * m.c.vocab * dtype_size(m.c.dtype);
    return m.c.tp_world > 1 ? m.logits_full : m.logits;
}

// tp > 1 logits arrive as [rank][batch][vocab/tp]; reorder on the host side of the copy.
static int copy_result_to_host(Model &m, void *dst) {
    size_t bytes;
    const void *src = result_ptr(m, &bytes);
    if (m.c.output_mode == 0 && m.c.tp_world > 1) {
        const size_t row = (size_t)m.vocab_l * dtype_size(m.c.dtype);
        for (int r = 0; r < m.c.tp_world; r++)
            MYNN_CUDA_OK(cudaMemcpy2DAsync((char *)dst + r * row, row * m.c.tp_world, (const char *)src + (size_t)r * m.c.batch * row,
                                           row, row, m.c.batch, cudaMemcpyDeviceToHost, m.stream));
    } else {
        MYNN_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, m.stream));
    }
    // the status words of the bounded waits travel with the result: one synchronisation per step, not one per word
    int *hs = m.h_status;
    hs[0] = hs[1] = 0;
    if (m.gemm_ws) MYNN_CUDA_OK(cudaMemcpyAsync(&hs[0], m.gemm_ws, sizeof(int), cudaMemcpyDeviceToHost, m.stream));
    if (m.tp_attached)
        MYNN_CUDA_OK(cudaMemcpyAsync(&hs[1], &tp_header(m.tp_block)->status, sizeof(int), cudaMemcpyDeviceToHost, m.stream));
    MYNN_CUDA_OK(cudaStreamSynchronize(m.stream));
    if (hs[0]) RC(mynn_b200_dequant_matmul_check(m.stream, m.gemm_ws));  // reports the code and clears the word
    if (m.tc_attention_ran) {  // prefill chunks of 64 and more rows: the tcgen05 attention has bounded waits of its own
        m.tc_attention_ran = false;
        int pfa = 0;
        RC(attention_prefill_tc_take_status(&pfa));
        if (pfa) return fail(MYNN_E_CUDA, "model: pipeline wait %d timed out inside the tcgen05 prefill attention", pfa);
    }
    if (hs[1]) {
        int *word = &tp_header(m.tp_block)->status;
        const int st_ = hs[1];
        {
            MYNN_CUDA_OK(cudaMemset(word, 0, sizeof st_));
            return fail(MYNN_E_COMM, "tensor-parallel reduction: a wait for a peer ran out of time (status %d)", st_);
        }
    }
    return MYNN_OK;
}

static int model_run(Model &m, void **output, void **input) {
    if (!output || !input || !output[0] || !input[0] || !input[1] || !input[2] || !input[3])
        return fail(MYNN_E_ARG, "model: null input/output pointer");
    if (m.c.stream_window > 0) return fail(MYNN_E_STATE, "model: this model has a streaming cache; step it with mynn_b200_model_stream");
    const int64_t past = *(const int64_t *)input[2], active = *(const int64_t *)input[3];
    if (past < 0 || past >= m.c.max_seq_len || active < 0 || active > m.c.max_seq_len)
        return fail(MYNN_E_ARG, "model: past_len %lld / active_seq_kv %lld outside the %d-row cache", (long long)past,
                    (long long)active, m.c.max_seq_len);
    cudaStream_t st = m.stream;
    // one pinned block, one copy: {past, active, position, ids}
    ((int32_t *)m.h_in)[0] = (int32_t)past;
    ((int32_t *)m.h_in)[1] = (int32_t)active;
    memcpy(m.h_in + 8, input[1], 8);
    memcpy(m.h_in + 16, input[0], (size_t)m.c.batch * 8);
    MYNN_CUDA_OK(cudaMemcpyAsync(m.past_dev, m.h_in, 16 + (size_t)m.c.batch * 8, cudaMemcpyHostToDevice, st));
    RC(run_decode(m, st));
    return copy_result_to_host(m, output[0]);
}

}  // namespace mynn

using namespace mynn;

extern "C" int mynn_b200_model_configure(const mynn_b200_model_config *cfg) {
    if (!cfg) return fail(MYNN_E_ARG, "model_configure: null config");
    const mynn_b200_model_config &c = *cfg;
    if (c.n_layers <= 0 || c.hidden <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.head_dim <= 0 || c.ffn <= 0 ||
        c.vocab <= 0 || c.max_seq_len <= 0 || c.batch <= 0)
        return fail(MYNN_E_ARG, "model_configure: non-positive dimension");
    if (c.dtype != MYNN_BF16 && c.dtype != MYNN_F16 && c.dtype != MYNN_F32) return fail(MYNN_E_ARG, "model_configure: bad dtype %d", c.dtype);
    if (c.tp_world < 1 || c.tp_rank < 0 || c.tp_rank >= c.tp_world) return fail(MYNN_E_ARG, "model_configure: bad tp rank %d/%d", c.tp_rank, c.tp_world);
    if (c.tp_world > kTpMaxRanks) return fail(MYNN_E_UNSUPPORTED, "model_configure: tp_world %d exceeds the %d ranks of one NVLink domain", c.tp_world, kTpMaxRanks);
    if (c.n_heads % c.n_kv_heads) return fail(MYNN_E_ARG, "model_configure: heads %d not a multiple of kv heads %d", c.n_heads, c.n_kv_heads);
    if (c.n_kv_heads % c.tp_world || c.ffn % c.tp_world || c.vocab % c.tp_world)
        return fail(MYNN_E_ARG, "model_configure: kv heads / ffn / vocab must divide by tp_world=%d", c.tp_world);
    if (c.tp_world > 1 && (comm_world() != c.tp_world || comm_rank() != c.tp_rank))
        return fail(MYNN_E_STATE, "model_configure: communicator is rank %d of %d, config says %d of %d", comm_rank(), comm_world(), c.tp_rank, c.tp_world);
    if (c.head_dim & 1) return fail(MYNN_E_ARG, "model_configure: odd head_dim");
    if (c.stream_window < 0 || c.stream_sink < 0 || (c.stream_window == 0 && c.stream_sink != 0))
        return fail(MYNN_E_ARG, "model_configure: bad streaming cache (sink %d, window %d)", c.stream_sink, c.stream_window);
    if (c.stream_window > 0 && c.stream_sink + c.stream_window > c.max_seq_len)
        return fail(MYNN_E_ARG, "model_configure: sink %d + window %d exceed max_seq_len %d", c.stream_sink, c.stream_window, c.max_seq_len);
    g_cfg = c;
    g_cfg_set = true;
    return MYNN_OK;
}

extern "C" void *model_init(void **initializer, void **session_state) {
    Model *m = nullptr;
    g_status = model_create(&m, initializer, session_state);
    return m;
}

extern "C" void model(void *state, void **output, void **input) {
    if (!state) {
        g_status = fail(MYNN_E_STATE, "model: null state");
        return;
    }
    g_status = model_run(*(Model *)state, output, input);
}

extern "C" void model_destroy(void *state) {
    if (!state) return;
    Model *m = (Model *)state;
    if (m->stream) cudaStreamSynchronize(m->stream);
    if (m->graph_exec) cudaGraphExecDestroy(m->graph_exec);
    if (m->stream_graph_exec) cudaGraphExecDestroy(m->stream_graph_exec);
    if (m->stream) cudaStreamDestroy(m->stream);
    if (m->arena) cudaFree(m->arena);
    if (m->h_in) cudaFreeHost(m->h_in);
    if (m->h_status) cudaFreeHost(m->h_status);
    for (int r = 0; r < m->tp.world; r++)
        if (m->tp_attached && r != m->tp.rank && m->tp.blocks[r]) cudaIpcCloseMemHandle(m->tp.blocks[r]);
    if (m->tp_block) cudaFree(m->tp_block);
    delete m;
}

extern "C" int mynn_b200_model_status(void) { return g_status; }

extern "C" int mynn_b200_model_step_device(void *state, void *stream, const int64_t *ids_dev, int past_len, void *out_dev) {
    if (!state) return fail(MYNN_E_STATE, "model_step_device: null state");
    Model &m = *(Model *)state;
    if (m.c.stream_window > 0) return fail(MYNN_E_STATE, "model_step_device: this model has a streaming cache; step it with mynn_b200_model_stream");
    if (past_len < 0 || past_len >= m.c.max_seq_len) return fail(MYNN_E_ARG, "model_step_device: past_len %d outside the cache", past_len);
    cudaStream_t st = stream ? (cudaStream_t)stream : m.stream;
    // The 16-byte header is passed by value through a pageable copy (staged by the runtime before it returns).
    struct { int32_t past, active; int64_t pos; } hdr = {past_len, past_len + 1, (int64_t)past_len};
    if (ids_dev) MYNN_CUDA_OK(cudaMemcpyAsync(m.ids_dev, ids_dev, (size_t)m.c.batch * 8, cudaMemcpyDeviceToDevice, st));
    MYNN_CUDA_OK(cudaMemcpyAsync(m.past_dev, &hdr, 16, cudaMemcpyHostToDevice, st));
    RC(run_decode(m, st));
    if (out_dev) {
        size_t bytes;
        const void *src = result_ptr(m, &bytes);
        MYNN_CUDA_OK(cudaMemcpyAsync(out_dev, src, bytes, cudaMemcpyDeviceToDevice, st));
    }
    return MYNN_OK;
}

// Prefill of T tokens per sequence starting at cache row past_len (the engine's prefill graph,
// crates/llm/src/session.rs:426-480, without the padding rows): ids_host int64 [batch, T]; out_host receives the
// logits / token ids of the last position, as model() does.  T <= max_prefill.
extern "C" int mynn_b200_model_prefill(void *state, const int64_t *ids_host, int T, int past_len, void *out_host) {
    if (!state) return fail(MYNN_E_STATE, "model_prefill: null state");
    Model &m = *(Model *)state;
    if (m.c.stream_window > 0) return fail(MYNN_E_STATE, "model_prefill: this model has a streaming cache; step it with mynn_b200_model_stream");
    const int cap = m.c.max_prefill > 0 ? m.c.max_prefill : 1;
    if (T <= 0 || T > cap) return fail(MYNN_E_ARG, "model_prefill: %d tokens, capacity %d", T, cap);
    if (past_len < 0 || past_len + T > m.c.max_seq_len) return fail(MYNN_E_ARG, "model_prefill: rows [%d, %d) outside the %d-row cache", past_len, past_len + T, m.c.max_seq_len);
    if (!ids_host || !out_host) return fail(MYNN_E_ARG, "model_prefill: null pointer");
    cudaStream_t st = m.stream;
    std::vector<int64_t> pos(T);
    for (int i = 0; i < T; i++) pos[i] = past_len + i;
    struct { int32_t past, active; int64_t pos; } hdr = {past_len, past_len + T, (int64_t)past_len};
    MYNN_CUDA_OK(cudaMemcpyAsync(m.ids_dev, ids_host, (size_t)m.c.batch * T * 8, cudaMemcpyHostToDevice, st));
    MYNN_CUDA_OK(cudaMemcpyAsync(m.pos_dev, pos.data(), (size_t)T * 8, cudaMemcpyHostToDevice, st));
    MYNN_CUDA_OK(cudaMemcpyAsync(m.past_dev, &hdr, 16, cudaMemcpyHostToDevice, st));
    MYNN_CUDA_OK(cudaStreamSynchronize(st));  // the sources above are short-lived host memory
    RC(enqueue_forward(m, st, T));
    return copy_result_to_host(m, out_host);
}

// Streaming step.  Token P of the stream lives in slot P (P < sink) or sink + (P - sink) % window.  After the append
// `active` = min(stream_pos + T, sink + window) slots are live, the oldest ring entry sits at ring offset ring_start, a
// cached key rotates at its recency rank and the query of token P at min(P, sink + window - 1).  While nothing has been
// evicted this is the engine's own host math (crates/llm/src/session.rs:539-635); afterwards it keeps the layout that
// code documents (the engine derives the write slot and the rank table from the position before the append, which do
// not agree with each other once the ring has wrapped).
extern "C" int mynn_b200_model_stream(void *state, const int64_t *ids_host, int T, long long stream_pos, void *out_host) {
    if (!state) return fail(MYNN_E_STATE, "model_stream: null state");
    Model &m = *(Model *)state;
    const mynn_b200_model_config &c = m.c;
    if (c.stream_window <= 0) return fail(MYNN_E_STATE, "model_stream: the model was not configured with a streaming cache");
    const int sink = c.stream_sink, window = c.stream_window, max_active = sink + window;
    const int cap = c.max_prefill > 0 ? c.max_prefill : 1;
    if (T <= 0 || T > cap) return fail(MYNN_E_ARG, "model_stream: %d tokens, capacity %d", T, cap);
    if (stream_pos < 0 || !ids_host || !out_host) return fail(MYNN_E_ARG, "model_stream: bad argument");
    if (T > 1 && stream_pos + T > max_active)
        return fail(MYNN_E_ARG, "model_stream: a chunk of %d tokens at position %lld would evict (sink + window = %d); feed those tokens one at a time", T, stream_pos, max_active);
    const long long after = stream_pos + T;
    const int slot0 = stream_pos < sink ? (int)stream_pos : sink + (int)((stream_pos - sink) % window);
    const int active = (int)std::min<long long>(after, max_active);
    const int ring_start = after <= max_active ? 0 : (int)((after - sink) % window);
    std::vector<int64_t> kvpos(c.max_seq_len), qpos(T);
    for (int s = 0; s < c.max_seq_len; s++) {
        kvpos[s] = s;
        if (s >= sink && s < max_active) {
            const int rank = sink + ((s - sink) - ring_start + window) % window;
            if (rank < active) kvpos[s] = rank;
        }
    }
    for (int i = 0; i < T; i++) qpos[i] = std::min<long long>(stream_pos + i, max_active - 1);
    cudaStream_t st = m.stream;
    struct { int32_t past, active; int64_t pos; } hdr = {slot0, active, qpos[0]};
    MYNN_CUDA_OK(cudaMemcpyAsync(m.ids_dev, ids_host, (size_t)c.batch * T * 8, cudaMemcpyHostToDevice, st));
    MYNN_CUDA_OK(cudaMemcpyAsync(m.pos_dev, qpos.data(), (size_t)T * 8, cudaMemcpyHostToDevice, st));
    MYNN_CUDA_OK(cudaMemcpyAsync(m.kvpos_dev, kvpos.data(), (size_t)c.max_seq_len * 8, cudaMemcpyHostToDevice, st));
    MYNN_CUDA_OK(cudaMemcpyAsync(m.past_dev, &hdr, 16, cudaMemcpyHostToDevice, st));
    MYNN_CUDA_OK(cudaStreamSynchronize(st));  // the sources above are short-lived host memory
    if (T == 1 && c.use_graph) {
        if (!m.stream_graph_exec) {
            cudaGraph_t graph = nullptr;
            MYNN_CUDA_OK(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
            int rc = enqueue_forward(m, st, 1);
            cudaError_t e = cudaStreamEndCapture(st, &graph);
            if (rc) {
                if (graph) cudaGraphDestroy(graph);
                return rc;
            }
            if (e != cudaSuccess) return fail(MYNN_E_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
            e = cudaGraphInstantiate(&m.stream_graph_exec, graph, 0);
            cudaGraphDestroy(graph);
            if (e != cudaSuccess) return fail(MYNN_E_CUDA, "graph instantiation failed: %s", cudaGetErrorString(e));
        }
        MYNN_CUDA_OK(cudaGraphLaunch(m.stream_graph_exec, st));
    } else {
        RC(enqueue_forward(m, st, T));
    }
    return copy_result_to_host(m, out_host);
}

// Peer-memory set-up of the fused tensor-parallel reduction.  Each rank exports a 64-byte handle of its shared block
// (cudaIpcGetMemHandle); after the host has gathered the handles of all ranks in rank order, attach maps the peers'
// blocks.  Call both before the first step (the captured graph holds the mapped addresses).  Without attach the
// step uses ncclAllReduce followed by separate kernels.
extern "C" int mynn_b200_model_tp_export(void *state, void *handle_out_64_bytes) {
    if (!state || !handle_out_64_bytes) return fail(MYNN_E_ARG, "model_tp_export: null pointer");
    Model &m = *(Model *)state;
    if (!m.tp_block) return fail(MYNN_E_STATE, "model_tp_export: the model has no peer-shared block (not tensor parallel, more than 32 sequences, or no tensor-core GEMM)");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
    MYNN_CUDA_OK(cudaIpcGetMemHandle((cudaIpcMemHandle_t *)handle_out_64_bytes, m.tp_block));
    return MYNN_OK;
}

extern "C" int mynn_b200_model_tp_attach(void *state, const void *handles_world_x_64_bytes) {
    if (!state || !handles_world_x_64_bytes) return fail(MYNN_E_ARG, "model_tp_attach: null pointer");
    Model &m = *(Model *)state;
    if (!m.tp_block) return fail(MYNN_E_STATE, "model_tp_attach: the model has no peer-shared block");
    if (m.tp_attached) return fail(MYNN_E_STATE, "model_tp_attach: already attached");
    if (m.graph_exec) return fail(MYNN_E_STATE, "model_tp_attach: call before the first step");
    for (int r = 0; r < m.tp.world; r++) {
        if (r == m.tp.rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char *)handles_world_x_64_bytes + (size_t)r * 64, 64);
        void *p = nullptr;
        MYNN_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        m.tp.blocks[r] = (char *)p;
    }
    m.tp_attached = true;
    return MYNN_OK;
}
