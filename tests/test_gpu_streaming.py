"""GPU parity tests for the streaming (sink + ring) KV cache: ring append, key re-rotation, ring attention and the whole
decoder in streaming mode against the oracle, before and after the ring wraps."""
import numpy as np
import pytest
import torch

from oracle import ref_ops as R
from oracle.ref_model import LlamaConfig, OracleLlama

pytestmark = pytest.mark.gpu

ops = None
NAME = {torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32"}


@pytest.fixture(scope="module", autouse=True)
def _load():
    global ops
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from my_nn_engine_b200 import ops as _ops
    ops = _ops


def rel_err(got, want):
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_kv_cache_update_ring_vs_oracle(dtype):
    rng = np.random.default_rng(1)
    cache = rng.standard_normal((2, 3, 12, 8)).astype(np.float32)
    c = torch.from_numpy(cache).to(dtype).cuda()
    ref = c.float().cpu().numpy()
    for offset, t, ring in [(0, 3, (2, 6, 0)), (6, 3, (2, 6, 3)), (9, 1, (2, 6, 5)), (4, 2, (0, 0, 0)), (11, 4, (4, 8, 7))]:
        new = torch.from_numpy(rng.standard_normal((2, 3, t, 8)).astype(np.float32)).to(dtype)
        ops.kv_cache_update_ring(c, new.cuda(), offset, *ring)
        R.kv_cache_update_ring(ref, new.float().numpy(), offset, *ring)
        assert np.array_equal(c.float().cpu().numpy(), ref)
    from my_nn_engine_b200 import ffi
    with pytest.raises(ffi.MynnError):
        ops.kv_cache_update_ring(c, c[:, :, :1].contiguous(), 0, 8, 8, 0)  # sink + window > cache rows


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("d", [8, 64, 128])
def test_rope_cache_rows_vs_oracle(dtype, d):
    rng = np.random.default_rng(d)
    s, active = 24, 17
    cos, sin = R.rope_table(32, d, 10000.0, NAME[dtype])
    x = torch.from_numpy(rng.standard_normal((2, 2, s, d)).astype(np.float32)).to(dtype)
    kvpos = rng.permutation(s).astype(np.int64)
    out = ops.rope_cache_rows(x.cuda(), torch.from_numpy(cos).to(dtype).cuda(), torch.from_numpy(sin).to(dtype).cuda(),
                              torch.from_numpy(kvpos).cuda(), active)
    want = R.store_round(R.rope(x.float().numpy(), cos[kvpos], sin[kvpos]), NAME[dtype])
    got = out.float().cpu().numpy()
    ulp = {"bf16": 2.0 ** -7, "f16": 2.0 ** -10, "f32": 2.0 ** -22}[NAME[dtype]]
    assert np.abs(got[:, :, :active] - want[:, :, :active]).max() <= ulp * np.abs(want).max()  # fused multiply-add vs two roundings
    assert not got[:, :, active:].any()  # rows past the live ones are not touched


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("b,hq,hkv,sq,d,cache,active,ring,causal", [
    (2, 8, 2, 1, 128, 96, 40, (4, 60, 0), False),    # not wrapped: tuned decode kernel
    (2, 8, 2, 1, 128, 96, 64, (4, 60, 37), False),   # full ring: tuned decode kernel on the physical rows
    (1, 8, 2, 1, 128, 96, 30, (4, 60, 11), False),   # partly filled, rotated ring: ring walk
    (1, 4, 4, 5, 64, 40, 22, (2, 30, 7), True),      # several query rows: causal bound per logical rank
    (1, 6, 2, 3, 32, 16, 16, (0, 16, 5), True),
])
def test_attention_ring_vs_oracle(dtype, b, hq, hkv, sq, d, cache, active, ring, causal):
    rng = np.random.default_rng(active + d)
    q = torch.from_numpy(rng.standard_normal((b, hq, sq, d)).astype(np.float32)).to(dtype)
    k = torch.from_numpy(rng.standard_normal((b, hkv, cache, d)).astype(np.float32)).to(dtype)
    v = torch.from_numpy(rng.standard_normal((b, hkv, cache, d)).astype(np.float32)).to(dtype)
    want = R.attention_ring(q.float().numpy(), k.float().numpy(), v.float().numpy(), 0.2, active, *ring, is_causal=causal)
    out = ops.attention_ring(q.cuda(), k.cuda(), v.cuda(), 0.2, active, *ring, is_causal=causal)
    assert rel_err(out.float().cpu().numpy(), want) <= (1e-2 if dtype != torch.float32 else 1e-5)


def to_oracle_weights(state, dtype):
    out = {}
    for k, v in state.items():
        if v.dtype == torch.int8:
            out[k] = v.cpu().numpy()
        elif k.endswith(".scale"):
            out[k] = R.store_round(v.float().cpu().numpy(), dtype)
        else:
            out[k] = v.float().cpu().numpy()
    return out


MID = dict(hidden_size=512, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
           intermediate_size=1408, vocab_size=2048, rms_norm_eps=1e-5, rope_theta=10000.0)


@pytest.mark.parametrize("dtype,batch,prefill,use_graph", [("bf16", 1, 0, True), ("f32", 2, 0, False), ("bf16", 3, 6, True)])
def test_streaming_decoder_matches_oracle_across_eviction(dtype, batch, prefill, use_graph):
    """sink 3 + window 9 = 12 live rows, 30 tokens: the ring wraps one and a half times.  Teacher-forced logits within the
    end-to-end bound of the model tests at every step."""
    from my_nn_engine_b200.decoder import DecoderModel
    from my_nn_engine_b200.quantize import random_llama_state
    state = random_llama_state(MID, seed=11)
    sink, window = 3, 9
    oracle = OracleLlama(LlamaConfig.from_hf(MID), to_oracle_weights(state, dtype), dtype, 16, batch, streaming=(sink, window))
    model = DecoderModel(MID, state, dtype=dtype, max_seq_len=16, batch=batch, output="logits", use_graph=use_graph,
                         max_prefill=prefill, streaming=(sink, window))
    rng = np.random.default_rng(batch)
    toks = rng.integers(0, MID["vocab_size"], size=(batch, 30))
    tol = {"bf16": 3e-2, "f16": 1e-2, "f32": 1e-4}[dtype]
    pos = 0
    if prefill:
        oracle.prefill(toks[:, :prefill], prefill)
        out = model.stream(toks[:, :prefill], 0)
        assert rel_err(out.float().numpy(), oracle.last_logits) <= tol
        pos = prefill
    for p in range(pos, 30):
        oracle.decode_step(toks[:, p])
        out = model.stream(toks[:, p], p)
        assert rel_err(out.float().numpy(), oracle.last_logits) <= tol, p
    kc = model.k_cache[0].float().cpu().numpy()  # unrotated keys, in their ring slots
    assert np.abs(kc[:, :, :12] - oracle.k_cache[0][:, :, :12]).max() <= 2.0 ** -5 * np.abs(oracle.k_cache[0]).max()
    assert not kc[:, :, 12:].any()
    from my_nn_engine_b200 import ffi
    with pytest.raises(ffi.MynnError):
        model.step(toks[:, 0], 0)  # a streaming model is stepped through stream()
    model.close()


@pytest.mark.parametrize("dtype,batch,prefill,use_graph", [("bf16", 1, 0, True), ("f32", 2, 0, False), ("bf16", 3, 6, True), ("f16", 2, 5, True)])
def test_streaming_decoder_with_int8_cache_matches_oracle_across_eviction(dtype, batch, prefill, use_graph):
    """The engine's (streaming, quant_kv_cache) graph branch: keys quantized unrotated into the int8 ring and rotated inside the
    attention kernel at their recency rank.  sink 3 + window 9, 30 tokens (one and a half wraps)."""
    from my_nn_engine_b200.decoder import DecoderModel
    from my_nn_engine_b200.quantize import random_llama_state
    state = random_llama_state(MID, seed=11)
    sink, window = 3, 9
    oracle = OracleLlama(LlamaConfig.from_hf(MID), to_oracle_weights(state, dtype), dtype, 16, batch, streaming=(sink, window), kv_int8=True)
    model = DecoderModel(MID, state, dtype=dtype, max_seq_len=16, batch=batch, output="logits", use_graph=use_graph,
                         max_prefill=prefill, streaming=(sink, window), kv_int8=True)
    rng = np.random.default_rng(batch + 7)
    toks = rng.integers(0, MID["vocab_size"], size=(batch, 30))
    tol = {"bf16": 3e-2, "f16": 1e-2, "f32": 2e-3}[dtype]  # f32: the int8 rows flip by one step where the inputs differ in the last bit
    pos = 0
    if prefill:
        oracle.prefill(toks[:, :prefill], prefill)
        out = model.stream(toks[:, :prefill], 0)
        assert rel_err(out.float().numpy(), oracle.last_logits) <= tol
        pos = prefill
    for p in range(pos, 30):
        oracle.decode_step(toks[:, p])
        out = model.stream(toks[:, p], p)
        assert rel_err(out.float().numpy(), oracle.last_logits) <= tol, p
    kc = model.k_cache[0].cpu().numpy().astype(np.int32)  # unrotated int8 keys in their ring slots
    assert np.abs(kc[:, :, :12] - oracle.k_cache[0][:, :, :12].astype(np.int32)).max() <= 2
    assert not kc[:, :, 12:].any()
    model.close()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("quant", [False, True])
@pytest.mark.parametrize("b,hq,hkv,sq,d,sink,window,start,active,rope,causal", [
    (2, 4, 2, 1, 64, 3, 9, 4, 12, True, False), (1, 8, 2, 1, 128, 0, 0, 0, 20, True, False), (2, 4, 4, 1, 8, 2, 6, 0, 5, False, False),
    (1, 4, 2, 5, 64, 0, 0, 0, 14, True, True), (1, 2, 1, 3, 32, 4, 12, 7, 16, True, True)])
def test_attention_streaming_operator_vs_literal_oracle(dtype, quant, b, hq, hkv, sq, d, sink, window, start, active, rope, causal):
    """Every operand of the engine's Attention node at once: ring mapping, int8 cache with per-row scales, keys rotated inside
    the kernel at kv_position[logical row], one and several query rows, against the literal restatement of the engine's
    kernels."""
    from my_nn_engine_b200 import ops
    rng = np.random.default_rng(b * 100 + sq * 10 + d + active)
    cache = 24
    name = "f32" if dtype == torch.float32 else "bf16"
    q = torch.from_numpy(rng.standard_normal((b, hq, sq, d)).astype(np.float32)).to(dtype)
    if quant:
        k = torch.from_numpy(rng.integers(-127, 128, (b, hkv, cache, d), dtype=np.int8))
        v = torch.from_numpy(rng.integers(-127, 128, (b, hkv, cache, d), dtype=np.int8))
        ks = torch.from_numpy(rng.uniform(0.005, 0.02, (b, hkv, cache)).astype(np.float32)).to(dtype)
        vs = torch.from_numpy(rng.uniform(0.005, 0.02, (b, hkv, cache)).astype(np.float32)).to(dtype)
    else:
        k = torch.from_numpy(rng.standard_normal((b, hkv, cache, d)).astype(np.float32)).to(dtype)
        v = torch.from_numpy(rng.standard_normal((b, hkv, cache, d)).astype(np.float32)).to(dtype)
        ks = vs = None
    cos, sin = R.rope_table(32, d, 10000.0, name)
    kvpos = rng.permutation(32)[:cache].astype(np.int64)  # any table: the kernel must index it by logical row
    want = R.attention_streaming(q.float().numpy(), k.numpy() if quant else k.float().numpy(), v.numpy() if quant else v.float().numpy(),
                                 0.2, active, sink, window, start, is_causal=causal,
                                 k_scale=None if ks is None else ks.float().numpy(), v_scale=None if vs is None else vs.float().numpy(),
                                 cos_table=cos if rope else None, sin_table=sin if rope else None, kv_position=kvpos if rope else None)
    out = ops.attention_streaming(q.cuda(), k.cuda(), v.cuda(), 0.2, active, causal, (sink, window, start),
                                  None if ks is None else ks.cuda(), None if vs is None else vs.cuda(),
                                  torch.from_numpy(cos).to(dtype).cuda() if rope else None, torch.from_numpy(sin).to(dtype).cuda() if rope else None,
                                  torch.from_numpy(kvpos).cuda() if rope else None)
    got = out.float().cpu().numpy()
    assert np.abs(got - want).max() <= (1e-4 if dtype == torch.float32 else 1e-2) * max(np.abs(want).max(), 1e-6)


def test_streaming_decoder_long_prefill_chunks_then_eviction():
    """sink 4 + window 156 = 160 live rows; two prefill chunks of 70 tokens (long enough for the tcgen05 attention over the
    rotated copy of the keys), then 40 decode steps, of which the last 20 evict."""
    from my_nn_engine_b200 import ops
    from my_nn_engine_b200.decoder import DecoderModel
    from my_nn_engine_b200.quantize import random_llama_state
    state = random_llama_state(MID, seed=11)
    sink, window, batch, chunk = 4, 156, 2, 70
    oracle = OracleLlama(LlamaConfig.from_hf(MID), to_oracle_weights(state, "bf16"), "bf16", 160, batch, streaming=(sink, window))
    model = DecoderModel(MID, state, dtype="bf16", max_seq_len=160, batch=batch, output="logits", max_prefill=chunk,
                         streaming=(sink, window))
    rng = np.random.default_rng(5)
    toks = rng.integers(0, MID["vocab_size"], size=(batch, 180))
    oracle.prefill(toks[:, :2 * chunk], chunk)
    model.stream(toks[:, :chunk], 0)
    out = model.stream(toks[:, chunk:2 * chunk], chunk)
    ops.attention_check()
    assert rel_err(out.float().numpy(), oracle.last_logits) <= 3e-2
    for p in range(2 * chunk, 180):
        oracle.decode_step(toks[:, p])
        out = model.stream(toks[:, p], p)
        assert rel_err(out.float().numpy(), oracle.last_logits) <= 3e-2, p
    model.close()


def test_tiny_llama_streaming_session_reproduces_expected_ids(tiny_llama):
    """crates/llm/tests/tinyllama_random.rs:23-49 with the float weights quantised: the int8 model is not pinned by the
    float ids, so the device model is compared with the oracle on the same int8 weights; the f32 oracle on the float
    weights reproduces the reference ids in the CPU suite."""
    from my_nn_engine_b200 import LlmSession
    from my_nn_engine_b200.decoder import DecoderModel
    from my_nn_engine_b200.quantize import quantize_state_dict
    cfg, weights, prompt, _, _ = tiny_llama
    state = quantize_state_dict({k: torch.from_numpy(v) for k, v in weights.items()})
    oracle = OracleLlama(LlamaConfig.from_hf(cfg), to_oracle_weights(state, "f32"), "f32", 32, streaming=(4, 28))
    want = oracle.generate(prompt[None, :], 8)[0].tolist()
    model = DecoderModel(cfg, state, dtype="f32", max_seq_len=32, streaming=(4, 28), output="ids")
    sess = LlmSession.for_llama_streaming(model, eos_token_id=-1)
    assert sess.generate_ids(prompt.tolist(), 8) == want
    model.close()
