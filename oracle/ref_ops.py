"""CPU oracle: numpy restatement of the reference's CPU (LLVM) backend for the LLM decode path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this module; it is
the checker used by ``tests/``, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.

Parity status: the reference itself (Rust + LLVM 18 + OpenBLAS) cannot be built in this
environment, so the restatement is pinned against the reference's own golden vectors
(``models/test/single_op/*`` of the reference, converted by ``tests/golden/make_golden.py``)
and against the ``tiny-llama-random`` greedy ids of
``crates/llm/tests/tinyllama_random.rs:23-24``.  M=1 int8 decode beyond the 3x8 toy fixture
is pinned by restatement only.

Every function names the reference code it follows (paths relative to the reference root).
All arithmetic is float32 unless stated; bf16 values travel as uint16 bit patterns or as
float32 arrays that are exactly representable in bf16.
"""
from __future__ import annotations

import math

import numpy as np

# --------------------------------------------------------------------------------------
# storage conversions
# --------------------------------------------------------------------------------------


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """bf16 bit pattern -> f32 by a 16-bit left shift (src/codegen/cpu/translator.rs:162-172)."""
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits_rne(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bits, round to nearest even, no NaN special case
    (src/codegen/cpu/translator.rs:174-204: bias = 0x7FFF + ((bits >> 16) & 1))."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    bias = ((bits >> 16) & 1) + np.uint32(0x7FFF)
    return ((bits + bias) >> 16).astype(np.uint16)


def f32_to_bf16_bits_trunc(x: np.ndarray) -> np.ndarray:
    """f64/f32 host tensor -> bf16 bits by truncation, the conversion applied to graph inputs
    and initializers (src/session.rs:171-175: ``(x as f32).to_bits() >> 16``)."""
    bits = np.asarray(x, dtype=np.float64).astype(np.float32).view(np.uint32)
    return (bits >> 16).astype(np.uint16)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """f32 -> nearest bf16, returned as f32 (a kernel's bf16 store followed by a reload)."""
    return bf16_bits_to_f32(f32_to_bf16_bits_rne(x))


def round_f16(x: np.ndarray) -> np.ndarray:
    """f32 -> nearest fp16 -> f32.  fp16 is an extension: the reference has no fp16 tensor type
    (src/tensor/types.rs:278-282); store points are the same as for bf16."""
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def store_round(x: np.ndarray, dtype: str) -> np.ndarray:
    """Model one kernel's output store in storage dtype ``dtype`` ('f32' | 'bf16' | 'f16')."""
    x = np.asarray(x, dtype=np.float32)
    if dtype == "f32":
        return x
    if dtype == "bf16":
        return round_bf16(x)
    if dtype == "f16":
        return round_f16(x)
    raise ValueError(dtype)


# --------------------------------------------------------------------------------------
# DequantizeLinear / DequantMatMul
# --------------------------------------------------------------------------------------


def dequantize_linear(x: np.ndarray, scale: np.ndarray, axis: int = 0) -> np.ndarray:
    """out = f32(x) * scale[axis_idx]  (src/codegen/cpu/translator.rs:206-282)."""
    shape = [1] * x.ndim
    shape[axis] = x.shape[axis]
    return x.astype(np.float32) * np.asarray(scale, dtype=np.float32).reshape(shape)


def dequant_matmul_variant_a(act: np.ndarray, wq: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """M=1 fused decode loop: out[n] = scale[n] * sum_k f32(act[k]) * f32(wq[n,k])
    (src/codegen/cpu/translator.rs:3208-3313; same formula as the CUDA GEMV,
    src/codegen/cuda/cpp/dequant_gemv.cuh:11-59).  act [M,K] f32, wq [N,K] int8, scale [N]."""
    acc = act.astype(np.float32) @ wq.astype(np.float32).T
    return acc * np.asarray(scale, dtype=np.float32)[None, :]


def dequant_matmul_variant_b(act: np.ndarray, wq: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """Tensor-core tile of the reference: the weight is dequantised and ROUNDED TO BF16 before
    the product, f32 accumulate (src/codegen/cuda/cpp/dequant_matmul_wmma.cuh:65-76,87-192).
    The reference's dequant_matmul_MxNxK golden outputs equal this variant after the bf16 store."""
    w = round_bf16(wq.astype(np.float32) * np.asarray(scale, dtype=np.float32)[:, None])
    return act.astype(np.float32) @ w.T


def dequant_matmul_variant_c(act: np.ndarray, wq: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """CPU M>1 path: dequantise W to an f32 workspace (scale[n]*f32(w)), then sgemm(A, B^T)
    (src/codegen/cpu/translator.rs:3042-3111).  The BLAS summation order is unspecified."""
    w = dequantize_linear(wq, scale, 0)
    return act.astype(np.float32) @ w.T


def dequant_matmul(act: np.ndarray, wq: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """Reference CPU dispatch (src/codegen/cpu/translator.rs:3045-3049): M == 1 -> variant A,
    otherwise variant C.  ``act`` may have leading dims; they are flattened to M."""
    k = wq.shape[1]
    a2 = act.reshape(-1, k)
    out = dequant_matmul_variant_a(a2, wq, scale) if a2.shape[0] == 1 else dequant_matmul_variant_c(a2, wq, scale)
    return out.reshape(act.shape[:-1] + (wq.shape[0],))


def _round_half_away(x):
    """f32::round: half away from zero.  x - trunc(x) is exact, so no value just below one half rounds up."""
    t = np.trunc(x)
    return t + np.sign(x) * (np.abs(x - t) >= np.float32(0.5))


def dynamic_quantize_linear(x: np.ndarray, symmetric: bool, per_row: bool, dtype: str = "bf16"):
    """DynamicQuantizeLinear, the engine's extension of the ONNX operator (src/graph/operator.rs:265-285).
    Returns (y, scale stored in ``dtype``, zero_point).  x [rows, inner] f32 values.

    symmetric per-row follows the CPU kernel mynn_dynquant_i8 (src/codegen/cpu/kernels/dynquant_i8.rs:13-37):
    sc = amax / 127 (1 for an all-zero row), inv = 1 / sc, y = round-half-away(x * inv) clamped to [-127, 127].
    The other three variants exist only in the CUDA backend (src/codegen/cuda/cpp/dynamic_quantize_linear.cuh:41-151):
    y = nearbyint(x / scale) + zp with scale = max|x| / 127, zp = 0 (symmetric, int8) or, asymmetric (uint8), the
    range widened to contain 0, scale = (max - min) / 255 (1 if 0), zp = clamp(nearbyint(-min / scale), 0, 255)."""
    x = np.asarray(x, dtype=np.float32)
    rows = x if per_row else x.reshape(1, -1)
    f32 = np.float32
    if symmetric and per_row:
        amax = np.abs(rows).max(axis=1)
        sc = np.where(amax > 0, amax / f32(127.0), f32(1.0)).astype(f32)
        inv = (f32(1.0) / sc).astype(f32)
        y = np.clip(_round_half_away((rows * inv[:, None]).astype(f32)), -127, 127).astype(np.int8)
        zp = np.zeros(len(sc), np.int8)
    elif symmetric:
        amax = np.abs(rows).max(axis=1)
        sc = (amax / f32(127.0)).astype(f32)
        with np.errstate(divide="ignore", invalid="ignore"):
            q = np.where(sc[:, None] > 0, np.rint((rows / sc[:, None]).astype(f32)), 0)
        y = np.clip(q, -127, 127).astype(np.int8)
        zp = np.zeros(len(sc), np.int8)
    else:
        mn = np.minimum(rows.min(axis=1), f32(0.0))
        mx = np.maximum(rows.max(axis=1), f32(0.0))
        sc = ((mx - mn) / f32(255.0)).astype(f32)
        sc = np.where(sc == 0, f32(1.0), sc).astype(f32)
        zp = np.clip(np.rint((-mn / sc).astype(f32)), 0, 255).astype(np.int64)
        q = np.rint((rows / sc[:, None]).astype(f32)).astype(np.int64) + zp[:, None]
        y = np.clip(q, 0, 255).astype(np.uint8)
        zp = zp.astype(np.uint8)
    scale = store_round(sc, dtype)
    if not per_row:
        return y.reshape(x.shape), scale.reshape(()), zp.reshape(())
    return y, scale, zp


def quantized_matmul(lhs: np.ndarray, lhs_scale: np.ndarray, rhs: np.ndarray, rhs_scale: np.ndarray) -> np.ndarray:
    """QuantizedMatMul: out[m,n] = (int32 sum_k lhs[m,k] * rhs[n,k]) * lhs_scale[m] * rhs_scale[n], products taken left
    to right in f32 (src/codegen/cpu/kernels/qgemv_i8i8.rs:59-78).  lhs_scale [M] or a scalar; the caller rounds the
    result to the storage dtype."""
    acc = lhs.astype(np.int64) @ rhs.astype(np.int64).T
    ls = np.asarray(lhs_scale, dtype=np.float32).reshape(-1, 1) if np.ndim(lhs_scale) else np.float32(lhs_scale)
    return (acc.astype(np.float32) * ls).astype(np.float32) * np.asarray(rhs_scale, dtype=np.float32)[None, :]


# --------------------------------------------------------------------------------------
# Attention / KV cache
# --------------------------------------------------------------------------------------


def attention(q, k, v, scale, active_seq_kv=None, is_causal=False, mask=None, k_scale=None, v_scale=None):
    """Streaming-softmax attention exactly as the CPU kernel orders it
    (src/codegen/cpu/translator.rs:4440-5008).

    q [B,Hq,Sq,D], k/v [B,Hkv,Sk,D] (float, or int8 with per-token scales [B,Hkv,Sk]).
    kv head = q head // (Hq/Hkv).  k_bound = min(active, causal cap, Sk) where the causal cap of
    query row sq is (active - Sq) + sq + 1.  Per kv row: qk = (q.k)[*k_scale]*scale [+mask];
    m' = max(m, qk); f = exp(m-m'); e = exp(qk-m'); s = s*f+e; o = o*f + e[*v_scale]*v; out = o/s.
    The loop over kv rows is vectorised over (b, h, sq) here; the recurrence itself is kept.
    """
    q = np.asarray(q, dtype=np.float32)
    b, hq, sq, d = q.shape
    hkv, sk = k.shape[1], k.shape[2]
    group = hq // hkv
    active = sk if active_seq_kv is None else int(active_seq_kv)
    kf = np.repeat(np.asarray(k).astype(np.float32), group, axis=1)
    vf = np.repeat(np.asarray(v).astype(np.float32), group, axis=1)
    ks = None if k_scale is None else np.repeat(np.asarray(k_scale, dtype=np.float32), group, axis=1)
    vs = None if v_scale is None else np.repeat(np.asarray(v_scale, dtype=np.float32), group, axis=1)
    bounds = np.full((sq,), active, dtype=np.int64)
    if is_causal:
        past = active - sq
        bounds = np.minimum(bounds, past + np.arange(sq) + 1)
    bounds = np.minimum(bounds, sk)
    m = np.full((b, hq, sq), -np.inf, dtype=np.float32)
    s = np.zeros((b, hq, sq), dtype=np.float32)
    o = np.zeros((b, hq, sq, d), dtype=np.float32)
    fscale = np.float32(scale)
    for r in range(int(bounds.max()) if sq else 0):
        live = (r < bounds)[None, None, :]
        qk = np.einsum("bhsd,bhd->bhs", q, kf[:, :, r, :]).astype(np.float32)
        if ks is not None:
            qk = qk * ks[:, :, r][:, :, None]
        qk = qk * fscale
        if mask is not None:
            qk = qk + np.broadcast_to(mask, (b, hq, sq, sk))[..., r].astype(np.float32)
        m_new = np.where(live, np.maximum(m, qk), m)
        with np.errstate(invalid="ignore"):
            f = np.where(live, np.exp(m - m_new), np.float32(1)).astype(np.float32)
            e = np.where(live, np.exp(qk - m_new), np.float32(0)).astype(np.float32)
        s = s * f + e
        e_eff = e if vs is None else e * vs[:, :, r][:, :, None]
        o = o * f[..., None] + e_eff[..., None] * vf[:, :, r, :][:, :, None, :]
        m = m_new
    with np.errstate(invalid="ignore", divide="ignore"):
        return (o / s[..., None]).astype(np.float32)


def attention_softmax_f64(q, k, v, scale, active):
    """Plain two-pass softmax attention in float64: the in-test reference the engine's own KV
    session test uses (tests/session_state.rs:122-150)."""
    q = np.asarray(q, dtype=np.float64)
    b, hq, sq, d = q.shape
    group = hq // k.shape[1]
    kf = np.repeat(np.asarray(k, dtype=np.float64), group, axis=1)[:, :, :active]
    vf = np.repeat(np.asarray(v, dtype=np.float64), group, axis=1)[:, :, :active]
    logits = np.einsum("bhsd,bhkd->bhsk", q, kf) * scale
    logits -= logits.max(axis=-1, keepdims=True)
    p = np.exp(logits)
    p /= p.sum(axis=-1, keepdims=True)
    return np.einsum("bhsk,bhkd->bhsd", p, vf)


def kv_cache_update(cache: np.ndarray, new: np.ndarray, offset: int) -> np.ndarray:
    """In place: cache[b,h,offset+t,:] = new[b,h,t,:] (src/codegen/cpu/translator.rs:4374-4424;
    CUDA src/codegen/cuda/cpp/kvcache_update.cuh:6-26).  No bounds check in the reference."""
    t = new.shape[2]
    cache[:, :, offset:offset + t, :] = new
    return cache


def ring_phys_index(rank: int, ring_sink: int, ring_window: int, ring_start: int) -> int:
    """Logical row -> physical cache slot of the sink + ring layout (src/codegen/cuda/cpp/common.cuh:55-60).  The first
    ``ring_sink`` rows stay in place; later rows live in a ring of ``ring_window`` slots whose oldest entry is at ring
    offset ``ring_start``.  ring_window == 0 switches the mapping off.  Only the CUDA backend of the reference has it (the
    CPU backend ignores the ring operands), so everything built on it here restates the CUDA kernels."""
    if ring_window == 0 or rank < ring_sink:
        return rank
    return ring_sink + (ring_start + (rank - ring_sink)) % ring_window


def kv_cache_update_ring(cache: np.ndarray, new: np.ndarray, offset: int, ring_sink: int, ring_window: int, ring_start: int):
    """KVCacheUpdate with ring operands: cache[b,h,phys(offset+t),:] = new[b,h,t,:]
    (src/codegen/cuda/cpp/kvcache_update.cuh:6-26)."""
    for t in range(new.shape[2]):
        cache[:, :, ring_phys_index(offset + t, ring_sink, ring_window, ring_start), :] = new[:, :, t, :]
    return cache


def attention_ring(q, k, v, scale, active_seq_kv, ring_sink, ring_window, ring_start, is_causal=False):
    """Attention over a sink + ring cache: logical rows 0..active-1 are visited in order, each read from its physical
    slot (src/codegen/cuda/cpp/attention.cuh:546-600).  Implemented as a gather into logical order followed by the plain
    recurrence, which is the same arithmetic in the same order."""
    active = int(active_seq_kv)
    idx = [ring_phys_index(r, ring_sink, ring_window, ring_start) for r in range(active)]
    kg, vg = np.asarray(k)[:, :, idx, :], np.asarray(v)[:, :, idx, :]
    return attention(q, kg, vg, scale, active, is_causal=is_causal)


def streaming_state(stream_pos: int, n_new: int, sink: int, window: int, max_seq_len: int, engine_literal: bool = False):
    """Host-side index math of a streaming (sink + ring) step that appends tokens stream_pos .. stream_pos+n_new-1.

    Token P lives in slot P while P < sink + window... precisely: slot(P) = P for P < sink, else sink + (P - sink) % window.
    After the append ``active`` rows are live; the oldest ring entry sits at ring offset ``ring_start``; the RoPE
    position of a cached row is its logical (recency) rank and the query of token P rotates at min(P, sink+window-1).
    Returns dict(slots, q_positions, active, ring_start, kv_position[max_seq_len]).

    While nothing has been evicted (stream_pos + n_new <= sink + window) this is exactly what the engine computes
    (crates/llm/src/session.rs:539-635: identity slots, ring_start 0, kv_position = slot).  After that point the
    engine's host code derives ring_start and kv_position from the position BEFORE the append and reuses ring_start for
    the write slot, which sends the new row to slot sink + 2*((P-sink) % window) % window and rotates the newest key as if
    it were the oldest; that regime is not covered by any test of the engine.  By default this function follows the layout
    the engine documents (sink rows fixed, ring holds the last ``window`` tokens in age order) consistently instead;
    ``engine_literal=True`` reproduces the engine's host code line by line (streaming_decode_inputs / streaming_prefill_inputs /
    streaming_kv_position, and the write slot its KVCacheUpdate derives from them), so that the two can be compared."""
    max_active = sink + window
    after = stream_pos + n_new
    if engine_literal:
        if n_new == 1:  # streaming_decode_inputs (crates/llm/src/session.rs:571-598)
            ring_start = 0 if stream_pos < max_active else (stream_pos - sink) % window
            table_pos = stream_pos  # streaming_kv_position is called with the position BEFORE the append
        else:           # streaming_prefill_inputs (:539-569)
            ring_start = 0 if after <= max_active else (after - sink) % window
            table_pos = after
        active = min(after, max_active)
        q_positions = np.minimum(np.arange(stream_pos, after), max_active - 1).astype(np.int64)
        # KVCacheUpdate writes logical row offset + t = stream_pos + t through ring_phys_index with THIS ring_start
        slots = [ring_phys_index(stream_pos + t, sink, window, ring_start) for t in range(n_new)]
        # streaming_kv_position (:606-635)
        rs = 0 if table_pos < max_active else (table_pos - sink) % window
        active_in_ring = min(max(table_pos - sink, 0), window)
        kv_position = np.arange(max_seq_len, dtype=np.int64)
        for slot in range(sink, min(max_active, max_seq_len)):
            rel_age = ((slot - sink) + window - rs) % window
            if rel_age < active_in_ring:
                kv_position[slot] = sink + rel_age
        return dict(slots=slots, q_positions=q_positions, active=active, ring_start=ring_start, kv_position=kv_position)
    slots = [p if p < sink else sink + (p - sink) % window for p in range(stream_pos, after)]
    active = min(after, max_active)
    ring_start = 0 if after <= max_active else (after - sink) % window
    kv_position = np.arange(max_seq_len, dtype=np.int64)
    for slot in range(sink, min(max_active, max_seq_len)):
        rank = sink + ((slot - sink) - ring_start + window) % window
        if rank < active:
            kv_position[slot] = rank
    q_positions = np.minimum(np.arange(stream_pos, after), max_active - 1).astype(np.int64)
    if after > max_active:  # a chunk that evicts: every query row sits at the end of what it can see
        q_positions = np.minimum(q_positions, max_active - 1)
    return dict(slots=slots, q_positions=q_positions, active=active, ring_start=ring_start, kv_position=kv_position)


def attention_streaming(q, k, v, scale, active_seq_kv, ring_sink=0, ring_window=0, ring_start=0, is_causal=False, k_scale=None,
                        v_scale=None, cos_table=None, sin_table=None, kv_position=None):
    """The CUDA backend's attention with all its streaming operands, restated literally (src/codegen/cuda/cpp/attention.cuh:
    495-606 for one query row, :319-489 for several): logical rows 0..bound-1 are visited in order; row r is read from slot
    ring_phys_index(r); with an int8 cache the row is multiplied by its k_scale first; with kv_position given the key is then
    rotated in f32 at table row kv_position[r] -- indexed by the LOGICAL row r, as the kernel does --
    k_rot[i] = k[i] * cos[pos, i] + sign * k[pair(i)] * sin[pos, i] (sign -1 for the first half), and never rounded; the
    softmax weight of a row is multiplied by its v_scale before it meets v.  The only CPU-side restatement of these operands:
    the engine's CPU backend ignores them (crates/llm/tests/run_llm.rs:76-78)."""
    q = np.asarray(q, dtype=np.float32)
    b, hq, sq, d = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    half = d // 2
    active = int(active_seq_kv)
    out = np.zeros_like(q)
    for row_q in range(sq):
        bound = min(active, active - sq + row_q + 1) if is_causal else active
        m = np.full((b, hq), -np.inf, np.float32)
        ssum = np.zeros((b, hq), np.float32)
        o = np.zeros((b, hq, d), np.float32)
        for r in range(bound):
            phys = ring_phys_index(r, ring_sink, ring_window, ring_start)
            kr = np.repeat(np.asarray(k[:, :, phys, :]).astype(np.float32), group, axis=1)
            vr = np.repeat(np.asarray(v[:, :, phys, :]).astype(np.float32), group, axis=1)
            if k_scale is not None:
                kr = kr * np.repeat(np.asarray(k_scale[:, :, phys], dtype=np.float32), group, axis=1)[..., None]
            if kv_position is not None:
                pos = int(kv_position[r])
                c, s_ = np.asarray(cos_table[pos], np.float32), np.asarray(sin_table[pos], np.float32)
                pair = np.concatenate([-kr[..., half:], kr[..., :half]], axis=-1)
                kr = kr * c + pair * s_
            qk = (q[:, :, row_q, :] * kr).sum(axis=-1, dtype=np.float32) * np.float32(scale)
            m_new = np.maximum(m, qk)
            score = np.exp(qk - m_new).astype(np.float32)
            coeff = np.exp(m - m_new).astype(np.float32)
            ssum = ssum * coeff + score
            if v_scale is not None:
                score = score * np.repeat(np.asarray(v_scale[:, :, phys], dtype=np.float32), group, axis=1)
            o = o * coeff[..., None] + score[..., None] * vr
            m = m_new
        with np.errstate(invalid="ignore", divide="ignore"):
            out[:, :, row_q, :] = o / ssum[..., None]
    return out


def quantizing_kv_cache_update(cache: np.ndarray, scale: np.ndarray, new: np.ndarray, offset: int, scale_dtype: str = "bf16"):
    """INT8 KV cache append with one scale per token (src/codegen/cpu/translator.rs:4090-4372):
    s = max_d |new| * (1/127) in f32; inv = 127 / max (0 for an all-zero row); q = trunc(v * inv +- 0.5) clamped to
    [-128, 127]; cache[b,h,offset+t,:] = q, scale[b,h,offset+t] = s stored in the scale dtype.  In place.
    cache int8 [B,H,S,D]; scale f32 values [B,H,S]; new f32 values [B,H,T,D]."""
    new = np.asarray(new, dtype=np.float32)
    t = new.shape[2]
    max_abs = np.abs(new).max(axis=-1)
    s = (max_abs * np.float32(1.0 / 127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(max_abs == 0, np.float32(0), np.float32(127.0) / max_abs).astype(np.float32)
    scaled = (new * inv[..., None]).astype(np.float32)
    biased = scaled + np.where(scaled >= 0, np.float32(0.5), np.float32(-0.5))
    q = np.clip(np.trunc(biased).astype(np.int64), -128, 127).astype(np.int8)
    cache[:, :, offset:offset + t, :] = q
    scale[:, :, offset:offset + t] = store_round(s, scale_dtype)
    return cache, scale


# --------------------------------------------------------------------------------------
# glue ops
# --------------------------------------------------------------------------------------


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """y = x * (1/sqrt(mean(x^2)+eps)) * w over the last axis, f32
    (src/codegen/cpu/translator.rs:5896-6027; src/codegen/cuda/cpp/rms_norm.cuh:9-59)."""
    x = np.asarray(x, dtype=np.float32)
    ms = (x * x).sum(axis=-1, keepdims=True, dtype=np.float32) / np.float32(x.shape[-1])
    inv = np.float32(1.0) / np.sqrt(ms + np.float32(eps), dtype=np.float32)
    return (x * inv) * np.asarray(w, dtype=np.float32)


def rope_table(max_seq: int, head_dim: int, base: float, dtype: str):
    """cos/sin tables [max_seq, head_dim]: angle = p * inv_freq[j % (D/2)],
    inv_freq[i] = 1/base^(2i/D), computed in f64 (crates/llm/src/builder.rs:359-393, ``base`` is
    an f32 widened to f64) and then converted like any initializer: f64 -> f32 (nearest) ->
    bf16 by TRUNCATION (src/session.rs:171-175).  For 'f32' storage only the f64->f32 step applies;
    'f16' (extension) rounds to nearest."""
    half = head_dim // 2
    base64 = float(np.float32(base))
    inv_freq = np.array([1.0 / math.pow(base64, 2.0 * i / head_dim) for i in range(half)], dtype=np.float64)
    ang = np.arange(max_seq, dtype=np.float64)[:, None] * inv_freq[np.arange(head_dim) % half][None, :]
    cos, sin = np.cos(ang), np.sin(ang)
    if dtype == "bf16":
        return bf16_bits_to_f32(f32_to_bf16_bits_trunc(cos)), bf16_bits_to_f32(f32_to_bf16_bits_trunc(sin))
    if dtype == "f16":
        return round_f16(cos.astype(np.float32)), round_f16(sin.astype(np.float32))
    return cos.astype(np.float32), sin.astype(np.float32)


def rope(x: np.ndarray, cos_rows: np.ndarray, sin_rows: np.ndarray) -> np.ndarray:
    """Half-split rotation out = x*cos + concat(-x_high, x_low)*sin
    (crates/llm/src/builder.rs:402-438; fused form src/codegen/cuda/cpp/rope.cuh:19-46).
    x [..., S, D]; cos_rows/sin_rows [S, D] are the table rows already gathered by position."""
    x = np.asarray(x, dtype=np.float32)
    half = x.shape[-1] // 2
    rot = np.concatenate([-x[..., half:], x[..., :half]], axis=-1)
    return x * cos_rows.astype(np.float32) + rot * sin_rows.astype(np.float32)


def swish_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """SwiGLU inner product: (g / (1 + exp(-g))) * u in f32
    (src/codegen/cuda/kernel.rs:763; CPU src/codegen/cpu/translator.rs:459-476,994-1001)."""
    g = np.asarray(gate, dtype=np.float32)
    with np.errstate(over="ignore"):
        return (g / (np.float32(1) + np.exp(-g, dtype=np.float32))) * np.asarray(up, dtype=np.float32)


def argmax_last(logits: np.ndarray) -> int:
    """Greedy pick with the reference's tie rule: ``max_by(partial_cmp)`` returns the LAST index
    among equal maxima (crates/llm/src/session.rs:683-690)."""
    logits = np.asarray(logits).ravel()
    return int(len(logits) - 1 - np.argmax(logits[::-1]))


# --------------------------------------------------------------------------------------
# quantizer
# --------------------------------------------------------------------------------------


def quantize_per_channel(w: np.ndarray):
    """int8 per-output-channel quantizer (crates/llm/src/quantize.rs:124-169): scale = max|row|/127
    (zero row -> 1.0); q = clamp(round_half_away(x / scale), -128, 127) using the f32 scale; the
    stored scale is then rounded to bf16 (RNE, NaN -> 0x7FC0).  Returns (int8 [N,K], bf16 bits [N])."""
    w = np.asarray(w, dtype=np.float32)
    rows = w.reshape(w.shape[0], -1)
    max_abs = np.abs(rows).max(axis=1)
    scale = np.where(max_abs == 0, np.float32(1.0), max_abs / np.float32(127.0)).astype(np.float32)
    ratio = rows / scale[:, None]
    t = np.trunc(ratio)  # f32::round = half away from zero; r - trunc(r) is exact, |r| + 0.5 is not (0.5 - 2^-25 would round up)
    rounded = t + np.sign(ratio) * (np.abs(ratio - t) >= np.float32(0.5))
    q = np.clip(rounded, -128, 127).astype(np.int8).reshape(w.shape)
    bits = f32_to_bf16_bits_rne(scale)
    bits = np.where(np.isnan(scale), np.uint16(0x7FC0), bits)
    return q, bits
