"""Pins the CPU oracle (numpy and C) against the reference's own golden vectors (CPU only)."""
import numpy as np
import pytest

from conftest import eq_with_epsilon
from oracle import c_oracle, ref_ops as R
from oracle.ref_model import LlamaConfig, OracleLlama

DQMM = ["dequant_matmul", "dequant_matmul_16x16x16", "dequant_matmul_16x32x32", "dequant_matmul_32x32x64",
        "dequant_matmul_64x64x128", "dequant_matmul_128x128x64", "dequant_matmul_24x48x40",
        "dequant_matmul_17x17x17", "dequant_matmul_50x50x50", "dequant_matmul_80x96x96"]


@pytest.mark.parametrize("name", DQMM)
def test_dequant_matmul_goldens(single_op, name):
    """Reference tolerance for these fixtures is 1e-1 'Either' (tests/single_op.rs:1201-1231).  The CPU
    dispatch (variants A/C) must meet it; the tensor-core variant B reproduces the stored bf16 bits."""
    fx = single_op(name)
    act, wq, scale = fx.inputs
    k = wq.shape[1]
    a = R.bf16_bits_to_f32(act).reshape(-1, k)
    s = R.bf16_bits_to_f32(scale)
    want = R.bf16_bits_to_f32(fx.outputs[0]).reshape(a.shape[0], -1)
    for fn in (R.dequant_matmul_variant_a, R.dequant_matmul_variant_c, R.dequant_matmul):
        ok, md = eq_with_epsilon(R.round_bf16(fn(a, wq, s)), want, 1e-1)
        assert ok, (fn.__name__, md)
    got_b = R.f32_to_bf16_bits_rne(R.dequant_matmul_variant_b(a, wq, s))
    mism = int((got_b != fx.outputs[0].reshape(got_b.shape)).sum())
    assert mism <= max(1, got_b.size // 200), f"variant B differs from golden bits in {mism}/{got_b.size}"
    # C oracle, bf16 storage in/out
    c_out = c_oracle.dequant_matmul_fused(act.reshape(-1, k), wq, scale)
    ok, md = eq_with_epsilon(R.bf16_bits_to_f32(c_out), want, 1e-1)
    assert ok, md
    c_out = c_oracle.dequant_matmul_workspace(act.reshape(-1, k), wq, scale)
    ok, md = eq_with_epsilon(R.bf16_bits_to_f32(c_out), want, 1e-1)
    assert ok, md


@pytest.mark.parametrize("name,n_in", [("attention_decode", 3), ("attention_decode_gqa", 3),
                                       ("attention_decode_runtime_kv", 4), ("attention_causal", 3),
                                       ("attention_no_causal", 3), ("attention_causal_large", 3)])
def test_attention_goldens(single_op, name, n_in):
    """Reference tolerance 1e-4 'Either' (tests/single_op.rs:906-985)."""
    fx = single_op(name)
    q, k, v = fx.inputs[:3]
    active = int(fx.inputs[3]) if n_in == 4 else None
    causal = bool(fx.attr("is_causal", 0))
    scale = fx.attr("scale")
    got = R.attention(q, k, v, scale, active, causal)
    ok, md = eq_with_epsilon(got, fx.outputs[0], 1e-4)
    assert ok, md
    got_c = c_oracle.attention(q, k, v, scale, active, causal)
    ok, md = eq_with_epsilon(got_c, fx.outputs[0], 1e-4)
    assert ok, md


def test_kv_cache_update_golden(single_op):
    """Fixture graph is KVCacheUpdate followed by Sigmoid (tests/single_op.rs:951-957, eps 1e-5)."""
    fx = single_op("kv_cache_update")
    cache, new, offset = fx.inputs
    upd = R.kv_cache_update(cache.copy(), new, int(offset))
    ok, md = eq_with_epsilon(1.0 / (1.0 + np.exp(-upd.astype(np.float64))), fx.outputs[0], 1e-5)
    assert ok, md
    upd_c = c_oracle.kv_cache_update(cache.copy(), new, int(offset))
    assert np.array_equal(upd, upd_c)


def test_quantizing_kvcache_update_golden(single_op):
    """Exact int8 match required by the reference (tests/single_op.rs:1233-1244)."""
    fx = single_op("quantizing_kvcache_update")
    cache, scale, new, offset = fx.inputs
    c, s = R.quantizing_kv_cache_update(cache.copy(), R.bf16_bits_to_f32(scale).copy(), R.bf16_bits_to_f32(new), int(offset))
    assert np.array_equal(c, fx.outputs[0])
    assert s[:, :, int(offset):int(offset) + new.shape[2]].all() and not s[:, :, :int(offset)].any()


def test_attention_with_int8_kv_matches_dequantised_attention():
    """Attention over an int8 cache with per-token scales == attention over the dequantised cache (the scales enter
    as qk * k_scale and e * v_scale, src/codegen/cpu/translator.rs:4440-5008)."""
    rng = np.random.default_rng(2)
    k = rng.standard_normal((2, 2, 12, 16)).astype(np.float32)
    v = rng.standard_normal((2, 2, 12, 16)).astype(np.float32)
    q = rng.standard_normal((2, 4, 1, 16)).astype(np.float32)
    kc, ks = np.zeros((2, 2, 12, 16), np.int8), np.zeros((2, 2, 12), np.float32)
    vc, vs = np.zeros((2, 2, 12, 16), np.int8), np.zeros((2, 2, 12), np.float32)
    R.quantizing_kv_cache_update(kc, ks, k, 0)
    R.quantizing_kv_cache_update(vc, vs, v, 0)
    got = R.attention(q, kc, vc, 0.25, 9, k_scale=ks, v_scale=vs)
    want = R.attention(q, kc.astype(np.float32) * ks[..., None], vc.astype(np.float32) * vs[..., None], 0.25, 9)
    assert np.abs(got - want).max() < 1e-5


@pytest.mark.parametrize("name,symmetric,per_row", [("dyn_quantize_linear_sym_per_row", True, True),
                                                    ("dyn_quantize_linear_sym_per_tensor", True, False),
                                                    ("dyn_quantize_linear_asym_per_row", False, True),
                                                    ("dyn_quantize_linear_asym_per_tensor", False, False)])
def test_dynamic_quantize_linear_goldens(single_op, name, symmetric, per_row):
    """The reference's rule (tests/single_op.rs:1140-1180): y and zero_point exact, scale within 1e-3."""
    fx = single_op(name)
    assert bool(fx.attr("symmetric", 0)) == symmetric and (fx.attr("axis", None) is not None) == per_row
    y, scale, zp = R.dynamic_quantize_linear(R.bf16_bits_to_f32(fx.inputs[0]), symmetric, per_row, "bf16")
    assert y.dtype == fx.outputs[0].dtype and np.array_equal(y, fx.outputs[0])
    ok, md = eq_with_epsilon(scale, R.bf16_bits_to_f32(fx.outputs[1]), 1e-3)
    assert ok, md
    assert np.array_equal(zp, fx.outputs[2])


@pytest.mark.parametrize("name", ["quantized_matmul_64x64x64", "quantized_matmul_128x128x128", "quantized_matmul_256x128x128",
                                  "quantized_matmul_128x256x64", "quantized_matmul_1x128x128"])
def test_quantized_matmul_goldens(single_op, name):
    """tests/single_op.rs:1182-1199: tolerance 1e-1 (either rule); the restatement is far inside it."""
    fx = single_op(name)
    lhs, ls, rhs, rs = fx.inputs
    out = R.round_bf16(R.quantized_matmul(lhs, R.bf16_bits_to_f32(ls), rhs, R.bf16_bits_to_f32(rs)))
    want = R.bf16_bits_to_f32(fx.outputs[0])
    ok, md = eq_with_epsilon(out, want, 1e-1)
    assert ok, md
    assert np.abs(out - want).max() <= np.abs(want).max() * 2.0 ** -7  # in fact within one bf16 ulp of the output scale


def test_ring_index_and_streaming_state_properties():
    """ring_phys_index is the engine's formula; streaming_state keeps sink rows in place, the last `window` tokens in the
    ring, ranks equal to recency order, and reduces to the engine's host math while nothing has been evicted."""
    assert [R.ring_phys_index(r, 2, 3, 1) for r in range(5)] == [0, 1, 3, 4, 2]
    assert [R.ring_phys_index(r, 2, 0, 1) for r in range(5)] == [0, 1, 2, 3, 4]
    sink, window, ms = 3, 5, 12
    owner = {}
    for p in range(40):
        st = R.streaming_state(p, 1, sink, window, ms)
        owner[st["slots"][0]] = p
        live = sorted(owner.values())
        assert live == list(range(min(sink, p + 1))) + list(range(max(sink, p + 1 - window), p + 1))
        assert st["active"] == len(live) and st["q_positions"][0] == st["active"] - 1
        for rank, tok in enumerate(live):  # logical rank -> slot -> token, and the slot's RoPE position is its rank
            slot = R.ring_phys_index(rank, sink, window, st["ring_start"])
            assert owner[slot] == tok and st["kv_position"][slot] == rank
        if p + 1 <= sink + window:
            assert st["ring_start"] == 0 and st["slots"] == [p] and list(st["kv_position"]) == list(range(ms))


def test_attention_ring_equals_plain_attention_over_the_gathered_rows():
    rng = np.random.default_rng(4)
    k = rng.standard_normal((2, 2, 10, 8)).astype(np.float32)
    v = rng.standard_normal((2, 2, 10, 8)).astype(np.float32)
    q = rng.standard_normal((2, 4, 1, 8)).astype(np.float32)
    order = [0, 1, 5, 6, 7, 2, 3, 4]  # sink 2, window 6, ring_start 3
    got = R.attention_ring(q, k, v, 0.3, 8, 2, 6, 3)
    want = R.attention(q, k[:, :, order], v[:, :, order], 0.3, 8)
    assert np.array_equal(got, want)
    cache = np.zeros((1, 1, 10, 2), np.float32)
    R.kv_cache_update_ring(cache, np.arange(1, 7, dtype=np.float32).reshape(1, 1, 3, 2), 6, 2, 6, 3)
    assert [int(cache[0, 0, s, 0]) for s in range(10)] == [0, 0, 0, 1, 3, 5, 0, 0, 0, 0]  # ranks 6, 7, 8 -> slots 3, 4, 5


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_tiny_llama_streaming_reproduces_expected_ids(tiny_llama, dtype):
    """crates/llm/tests/tinyllama_random.rs:23-49: the golden ids are produced in streaming mode, sink 4 + window 28."""
    cfg, weights, prompt, _, expected = tiny_llama
    m = OracleLlama(LlamaConfig.from_hf(cfg), weights, dtype, 32, streaming=(4, 28))
    assert m.generate(prompt[None, :], len(expected))[0].tolist() == expected.tolist()


def test_streaming_oracle_matches_plain_oracle_until_eviction_and_differs_after(tiny_llama):
    cfg, weights, prompt, _, _ = tiny_llama
    c = LlamaConfig.from_hf(cfg)
    plain = OracleLlama(c, weights, "f32", 64)
    stream = OracleLlama(c, weights, "f32", 64, streaming=(2, 6))
    toks = np.array([[int(prompt[0])]])
    same = []
    for step in range(14):
        a = plain.decode_step(toks[:, 0])
        b = stream.decode_step(toks[:, 0])
        same.append(np.abs(plain.last_logits - stream.last_logits).max() < 1e-5)
        toks = a[:, None]
    assert all(same[:8]) and not all(same[8:])  # 8 = sink + window tokens fit; the 9th evicts one


def test_dequantize_linear_golden(single_op):
    fx = single_op("dequantize_linear")
    x, scale = fx.inputs
    got = R.round_bf16(R.dequantize_linear(x, R.bf16_bits_to_f32(scale), fx.attr("axis", 0)))
    ok, md = eq_with_epsilon(got, R.bf16_bits_to_f32(fx.outputs[0]), 1e-2)
    assert ok, md


def test_swish_golden(single_op):
    fx = single_op("swish")
    x = fx.inputs[0].astype(np.float32)
    got = R.swish_mul(x, np.ones_like(x))
    ok, md = eq_with_epsilon(got, fx.outputs[0], 1e-5)
    assert ok, md


def test_session_state_attention_reference():
    """Streaming softmax == the two-pass f64 softmax the reference's KV session test checks against
    (tests/session_state.rs:122-229): 3 decode steps appending to a zero-initialised cache."""
    B, H, S_MAX, D = 1, 2, 8, 4
    kc = np.zeros((B, H, S_MAX, D), np.float32)
    vc = np.zeros((B, H, S_MAX, D), np.float32)

    def data(step, kind):
        i = np.arange(B * H * D, dtype=np.float64)
        return np.clip(np.sin(i * 0.31 + step * 1.7 + kind * 2.4) * 0.5, -1, 1).astype(np.float32).reshape(B, H, 1, D)

    for step in range(3):
        q, k, v = data(step, 0), data(step, 1), data(step, 2)
        R.kv_cache_update(kc, k, step)
        R.kv_cache_update(vc, v, step)
        got = R.attention(q, kc, vc, 1.0 / np.sqrt(D), step + 1)
        want = R.attention_softmax_f64(q, kc, vc, 1.0 / np.sqrt(D), step + 1)
        ok, md = eq_with_epsilon(got, want, 1e-4)
        assert ok, md
    assert not kc[:, :, 3:].any()


def test_quantizer_known_answers():
    """crates/llm/tests/quantize.rs:101-166 of the reference."""
    w = np.array([[127.0, -127.0, 0.0, 64.0], [2.0, -1.0, 0.0, 0.5], [0, 0, 0, 0]], dtype=np.float32)
    q, sbits = R.quantize_per_channel(w)
    s = R.bf16_bits_to_f32(sbits)
    assert np.allclose(s, [1.0, 2.0 / 127.0, 1.0], atol=1e-3)
    assert q[0].tolist() == [127, -127, 0, 64]
    assert q[1].tolist() == [127, -64, 0, 32]     # -63.5 and 31.75 round half away / to nearest
    assert q[2].tolist() == [0, 0, 0, 0]
    assert np.abs(q.astype(np.float32) * s[:, None] - w).max() < 0.02


def test_argmax_takes_last_maximum():
    assert R.argmax_last(np.array([1.0, 5.0, 5.0, 2.0])) == 2
    assert R.argmax_last(np.array([7.0])) == 0


def test_rope_table_truncates_to_bf16():
    cos, sin = R.rope_table(8, 4, 10000.0, "bf16")
    exact = np.cos(np.arange(8.0)[:, None] * np.array([1.0, 0.01, 1.0, 0.01])[None, :]).astype(np.float32)
    bits = exact.view(np.uint32) >> 16
    assert np.array_equal(R.f32_to_bf16_bits_rne(cos), bits.astype(np.uint16))


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("prefill_len", [None, 4])
def test_tiny_llama_random_greedy_ids(tiny_llama, dtype, prefill_len):
    """End-to-end pin: prompt "Hello" -> the 8 greedy ids of crates/llm/tests/tinyllama_random.rs:23-24,
    for f32 and bf16 storage, token-by-token and through chunked prefill (:79-147)."""
    cfg, weights, prompt, _, expected = tiny_llama
    model = OracleLlama(LlamaConfig.from_hf(cfg), weights, dtype, max_seq_len=32)
    got = model.generate(prompt, len(expected), prefill_len)
    assert got[0].tolist() == expected.tolist()


def test_tiny_llama_prefill_matches_decode_only_multi_turn(tiny_llama):
    """crates/llm/tests/tinyllama_random.rs:84-142: two turns, prefill(4) vs decode-only give the same ids."""
    cfg, weights, p1, p2, _ = tiny_llama
    c = LlamaConfig.from_hf(cfg)
    a = OracleLlama(c, weights, "f32", 32)
    ref = a.generate(p1, 1)[0].tolist() + a.generate(p2, 3)[0].tolist()
    b = OracleLlama(c, weights, "f32", 32)
    got = b.generate(p1, 1, 4)[0].tolist() + b.generate(p2, 3, 4)[0].tolist()
    assert ref == got


def test_c_oracle_int8_attention_equals_the_numpy_restatement():
    """The C form of the attention recurrence over an int8 cache (used for long contexts) against ref_ops.attention."""
    from oracle import c_oracle
    rng = np.random.default_rng(1)
    q = rng.standard_normal((2, 4, 3, 16)).astype(np.float32)
    k = rng.integers(-127, 128, (2, 2, 20, 16), dtype=np.int8)
    v = rng.integers(-127, 128, (2, 2, 20, 16), dtype=np.int8)
    ks = rng.uniform(0.01, 0.02, (2, 2, 20)).astype(np.float32)
    vs = rng.uniform(0.01, 0.02, (2, 2, 20)).astype(np.float32)
    for causal in (False, True):
        want = R.attention(q, k, v, 0.25, 17, is_causal=causal, k_scale=ks, v_scale=vs)
        got = c_oracle.attention_q8(q, k, v, ks, vs, 0.25, 17, causal, parallel=True)
        assert np.abs(got - want).max() <= 1e-6
