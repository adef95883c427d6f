"""GPU parity tests, model level: the whole decoder step behind model_init / model / model_destroy against the CPU
oracle on the same seeded int8 checkpoints.  Greedy tokens are compared teacher-forced (the device model is fed the
oracle's token each step, so one flipped near-tie cannot cascade): every step must pick the oracle's token unless the
oracle's own top-2 logits are closer than the storage dtype can resolve.  Each kernel meets the 1e-2 bound on its
own (operator tests); the logits at the end of the stack carry the rounding noise of every bf16/fp16 store in between
(the two sides round differently whenever their f32 sums differ in the last bit), so the end-to-end bound is a few
storage ulps of the logit scale: 3e-2 for bf16, 1e-2 for fp16, 1e-4 for f32."""
import numpy as np
import pytest
import torch

from oracle import ref_ops as R
from oracle.ref_model import LlamaConfig, OracleLlama

pytestmark = pytest.mark.gpu


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


def run_parity(cfg, state, dtype, batch, steps, max_seq, prompt_len, prefill_len, seed, use_graph=True, kv_int8=False):
    from my_nn_engine_b200.decoder import DecoderModel
    rng = np.random.default_rng(seed)
    oracle = OracleLlama(LlamaConfig.from_hf(cfg), to_oracle_weights(state, dtype), dtype, max_seq, batch, kv_int8=kv_int8)
    model = DecoderModel(cfg, state, dtype=dtype, max_seq_len=max_seq, batch=batch, output="logits",
                         use_graph=use_graph, max_prefill=prefill_len or 0, kv_int8=kv_int8)
    prompt = rng.integers(0, cfg["vocab_size"], size=(batch, prompt_len))
    ulp = {"bf16": 2.0 ** -7, "f16": 2.0 ** -10, "f32": 2.0 ** -20}[dtype]
    worst, flips = 0.0, 0

    def compare(gpu_logits, ora_logits):
        nonlocal worst, flips
        g = gpu_logits.float().numpy()
        worst = max(worst, float(np.abs(g - ora_logits).max() / np.abs(ora_logits).max()))
        for b in range(batch):
            want, got = R.argmax_last(ora_logits[b]), R.argmax_last(g[b])
            if want != got:
                gap = ora_logits[b][want] - ora_logits[b][got]
                assert gap <= 4 * ulp * abs(ora_logits[b][want]), f"token {got} != {want}, logit gap {gap}"
                flips += 1

    if prefill_len:
        tok = oracle.prefill(prompt, prefill_len)
        past = 0
        for p0 in range(0, prompt_len, prefill_len):
            out = model.prefill(prompt[:, p0:p0 + prefill_len], past)
            past += min(prefill_len, prompt_len - p0)
        compare(out, oracle.last_logits)
    else:
        past = 0
        for j in range(prompt_len):
            tok = oracle.decode_step(prompt[:, j])
            out = model.step(prompt[:, j], past)
            past += 1
        compare(out, oracle.last_logits)
    for _ in range(steps):
        nxt = oracle.decode_step(tok)
        out = model.step(tok, past)  # teacher forcing: the oracle's previous token
        past += 1
        compare(out, oracle.last_logits)
        tok = nxt
    # KV caches: the device rows equal the oracle's (rounded) rows, rows past the sequence are still zero
    kc = model.k_cache[0].float().cpu().numpy()
    if kv_int8:
        # int8 rows with their scales: equal to the oracle's up to one quantisation step where the inputs differed by an ulp
        ks = model.k_scale[0].float().cpu().numpy()
        assert np.abs(ks[:, :, :past] - oracle.k_scale[0][:, :, :past]).max() <= 8 * ulp * oracle.k_scale[0].max()
        deq, want = kc * ks[..., None], oracle.k_cache[0].astype(np.float32) * oracle.k_scale[0][..., None]
        assert np.abs(deq[:, :, :past] - want[:, :, :past]).max() <= 1.5 * oracle.k_scale[0].max() + 8 * ulp * np.abs(want).max()
        assert not ks[:, :, past:].any()
    else:
        assert np.abs(kc[:, :, :past] - oracle.k_cache[0][:, :, :past]).max() <= 8 * ulp * np.abs(oracle.k_cache[0]).max()
    assert not kc[:, :, past:].any()
    model.close()
    assert worst <= {"bf16": 3e-2, "f16": 1e-2, "f32": 1e-4}[dtype], worst
    return worst, flips


@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
def test_tiny_llama_random_int8_matches_oracle(tiny_llama, dtype):
    """The reference's checked-in 2-layer model (hidden 16, head_dim 4: exercises the generic kernels), quantised
    with the reference's quantizer; prompt "Hello", 8 greedy steps as in crates/llm/tests/tinyllama_random.rs."""
    from my_nn_engine_b200.quantize import quantize_state_dict
    cfg, weights, prompt, _, expected = tiny_llama
    state = quantize_state_dict({k: torch.from_numpy(v) for k, v in weights.items()})
    run_parity(cfg, state, dtype, batch=1, steps=8, max_seq=32, prompt_len=1, prefill_len=None, seed=0)
    run_parity(cfg, state, dtype, batch=1, steps=4, max_seq=32, prompt_len=6, prefill_len=4, seed=1)


MID = dict(hidden_size=512, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
           intermediate_size=1408, vocab_size=2048, rms_norm_eps=1e-5, rope_theta=10000.0)


@pytest.mark.parametrize("dtype,batch,prefill_len,use_graph", [("bf16", 1, None, True), ("bf16", 4, 8, True),
                                                                ("f16", 2, None, False), ("bf16", 32, 16, True)])
def test_mid_size_model_32_greedy_steps(dtype, batch, prefill_len, use_graph):
    from my_nn_engine_b200.quantize import random_llama_state
    state = random_llama_state(MID, seed=3)
    worst, flips = run_parity(MID, state, dtype, batch, steps=32, max_seq=96, prompt_len=24, prefill_len=prefill_len,
                              seed=batch, use_graph=use_graph)
    # every flip was checked above to be a near tie of the oracle's own top two (4 storage ulps); with 2048 random logits
    # about 3 % of the picks are that close, and which side of a tie a pick falls on changes with any change of summation order
    assert flips <= max(batch, (33 * batch) // 20)


def test_mid_size_model_long_prefill_chunks_use_the_tensor_core_attention():
    """Prefill chunks of 70 tokens (two chunks, the second over a past of 70 rows): attention of 64 or more query rows runs
    on the tcgen05 kernel and writes [B, S, Hq, D] rows for o_proj."""
    from my_nn_engine_b200 import ops
    from my_nn_engine_b200.quantize import random_llama_state
    state = random_llama_state(MID, seed=3)
    worst, flips = run_parity(MID, state, "bf16", batch=2, steps=4, max_seq=160, prompt_len=140, prefill_len=70, seed=11)
    ops.attention_check()
    assert flips <= 2


def test_int8_kv_cache_long_prefill_chunks_use_the_tensor_core_attention():
    """quant_kv_cache with prefill chunks of 70 tokens: attention runs on the tcgen05 kernel over a 16-bit copy of the
    quantised rows (value * row scale, rounded once)."""
    from my_nn_engine_b200 import ops
    from my_nn_engine_b200.quantize import random_llama_state
    state = random_llama_state(MID, seed=3)
    worst, flips = run_parity(MID, state, "bf16", batch=2, steps=4, max_seq=160, prompt_len=140, prefill_len=70, seed=11, kv_int8=True)
    ops.attention_check()
    assert flips <= 2


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_int8_kv_cache_tiny_model(tiny_llama, dtype):
    """quant_kv_cache on the 2-layer fixture model (head_dim 4: generic attention over the int8 cache)."""
    from my_nn_engine_b200.quantize import quantize_state_dict
    cfg, weights, _, _, _ = tiny_llama
    state = quantize_state_dict({k: torch.from_numpy(v) for k, v in weights.items()})
    run_parity(cfg, state, dtype, batch=1, steps=8, max_seq=32, prompt_len=1, prefill_len=None, seed=0, kv_int8=True)
    run_parity(cfg, state, dtype, batch=2, steps=4, max_seq=32, prompt_len=6, prefill_len=4, seed=1, kv_int8=True)


@pytest.mark.parametrize("dtype,batch,prefill_len,use_graph", [("bf16", 1, None, True), ("bf16", 4, 8, True), ("f16", 2, None, False)])
def test_int8_kv_cache_mid_size_model(dtype, batch, prefill_len, use_graph):
    from my_nn_engine_b200.quantize import random_llama_state
    state = random_llama_state(MID, seed=3)
    worst, flips = run_parity(MID, state, dtype, batch, steps=32, max_seq=96, prompt_len=24, prefill_len=prefill_len,
                              seed=batch, use_graph=use_graph, kv_int8=True)
    assert flips <= batch


def test_int8_kv_cache_llama3_8b_shapes_batch32():
    from my_nn_engine_b200.quantize import random_llama_state
    cfg = dict(hidden_size=4096, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=14336, vocab_size=4096, rms_norm_eps=1e-5, rope_theta=500000.0)
    state = random_llama_state(cfg, seed=5)
    run_parity(cfg, state, "bf16", batch=32, steps=3, max_seq=96, prompt_len=70, prefill_len=35, seed=9, kv_int8=True)


def test_llama3_8b_shapes_two_layer_slice_batch32():
    """Llama-3-8B dimensions (hidden 4096, 32 q / 8 kv heads, head_dim 128, FFN 14336, theta 5e5) on a 2-layer slice
    with a reduced vocabulary so the CPU oracle finishes in seconds; batch 32, a 40-token context, 3 decode steps."""
    from my_nn_engine_b200.quantize import random_llama_state
    cfg = dict(hidden_size=4096, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=14336, vocab_size=4096, rms_norm_eps=1e-5, rope_theta=500000.0)
    state = random_llama_state(cfg, seed=5)
    run_parity(cfg, state, "bf16", batch=32, steps=3, max_seq=64, prompt_len=40, prefill_len=20, seed=9)


@pytest.mark.parametrize("vocab", [2048, 32768])
def test_device_argmax_output_and_step_device(vocab):
    """output='ids' returns the last-maximum argmax of the logits the 'logits' model returns (one-stage kernel for the
    small vocabulary, two-stage for the large one); the device-resident step gives the same tokens as the host-buffer
    step."""
    from my_nn_engine_b200.decoder import DecoderModel
    from my_nn_engine_b200.quantize import random_llama_state
    cfg = dict(MID, vocab_size=vocab)
    state = random_llama_state(cfg, seed=4)
    a = DecoderModel(cfg, state, batch=3, max_seq_len=32, output="logits")
    b = DecoderModel(cfg, state, batch=3, max_seq_len=32, output="ids")
    c = DecoderModel(cfg, state, batch=3, max_seq_len=32, output="ids")
    tok = np.array([5, 6, 7])
    ids_dev = torch.tensor(tok, device="cuda")
    out_dev = torch.zeros(3, dtype=torch.int32, device="cuda")
    for past in range(6):
        la = a.step(tok, past).float().numpy()
        ib = b.step(tok, past).numpy().copy()
        c.step_device(ids_dev, past, out_dev)
        torch.cuda.synchronize()
        assert ib.tolist() == [R.argmax_last(r) for r in la] == out_dev.cpu().tolist()
        tok = ib
        ids_dev = out_dev.to(torch.int64)
    for m in (a, b, c):
        m.close()


def test_from_pretrained_directory_matches_in_memory_model(tmp_path, tiny_llama):
    """config.json + model.safetensors -> quantize_int8 command -> model.int8.safetensors -> DecoderModel: the same logits
    as the model built from the in-memory quantized state."""
    import json
    from my_nn_engine_b200 import checkpoint as C
    from my_nn_engine_b200.decoder import DecoderModel
    from my_nn_engine_b200.quantize import quantize_state_dict
    cfg, weights, prompt, _, _ = tiny_llama
    state = {k: torch.from_numpy(v) for k, v in weights.items()}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    C.write_safetensors(str(tmp_path / "model.safetensors"), state)
    assert C.main([str(tmp_path / "model.safetensors"), str(tmp_path / C.QUANTIZED_SAFETENSORS)]) == 0
    a = DecoderModel.from_pretrained(str(tmp_path), dtype="bf16", max_seq_len=32)
    b = DecoderModel(cfg, quantize_state_dict(state), dtype="bf16", max_seq_len=32)
    ids = np.asarray([[int(prompt[0])]])
    assert torch.equal(a.step(ids[:, 0], 0), b.step(ids[:, 0], 0))
    a.close()
    b.close()


def test_llm_session_on_device_model():
    from my_nn_engine_b200 import LlmSession
    from my_nn_engine_b200.decoder import DecoderModel
    from my_nn_engine_b200.quantize import random_llama_state
    state = random_llama_state(MID, seed=6)
    m1 = DecoderModel(MID, state, batch=1, max_seq_len=48, output="ids", max_prefill=8)
    m2 = DecoderModel(MID, state, batch=1, max_seq_len=48, output="logits")
    s1 = LlmSession.for_llama(m1, eos_token_id=-1, prefill_len=8)
    s2 = LlmSession.for_llama(m2, eos_token_id=-1)
    prompt = list(range(100, 111))
    a, b = s1.generate_ids(prompt, 12), s2.generate_ids(prompt, 12)
    assert a == b and len(a) == 12 and s1.past_len() == s2.past_len() == 11 + 11
    m1.close()
    m2.close()


@pytest.mark.parametrize("dtype,heads,kv_heads,head_dim,batch", [("bf16", 8, 2, 64, 4), ("f16", 16, 2, 64, 1), ("bf16", 8, 2, 128, 32),
                                                                 ("f16", 4, 4, 128, 3)])
def test_rope_and_append_inside_the_attention_kernel(dtype, heads, kv_heads, head_dim, batch):
    """MYNN_OPT_FUSE_ROPE: the decode attention kernel that rotates q and the new key and appends the new rows itself against
    the stand-alone RoPE + append kernel in front of it (group sizes 1, 4 and 8, both head dims, context lengths that put
    the new row first, last and in the middle of a split)."""
    from my_nn_engine_b200 import ffi
    from my_nn_engine_b200.decoder import DecoderModel
    from my_nn_engine_b200.quantize import random_llama_state
    cfg = dict(MID, num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim, hidden_size=512)
    state = random_llama_state(cfg, seed=5)
    rng = np.random.default_rng(7)
    prompt = rng.integers(0, cfg["vocab_size"], size=(batch, 13))
    toks = [rng.integers(0, cfg["vocab_size"], size=batch) for _ in range(40)]
    runs = []
    try:
        for fuse in (0, 1):
            ffi.set_option(ffi.OPT_FUSE_ROPE, fuse)
            m = DecoderModel(cfg, state, dtype=dtype, max_seq_len=80, batch=batch, output="logits", max_prefill=13)
            outs = [m.prefill(prompt, 0).clone()]
            for i, t in enumerate(toks):
                outs.append(m.step(t, 13 + i).clone())
            runs.append((torch.stack(outs), [k.clone() for k in m.k_cache], [v.clone() for v in m.v_cache]))
            m.close()
    finally:
        ffi.set_option(ffi.OPT_FUSE_ROPE, 1)
    # layer 0 sees the same inputs in both runs (embedding rows): its appended rows are identical bit for bit
    assert torch.equal(runs[0][1][0], runs[1][1][0]) and torch.equal(runs[0][2][0], runs[1][2][0])
    assert runs[1][1][0][:, :, :53].float().abs().sum() > 0 and not runs[1][1][0][:, :, 53:].any()
    # the softmax takes the new row in a tile of its own in one kernel and inside the last tile in the other: same sums in a
    # different order, so the later layers agree to a few storage ulps, not to the bit
    ulp = 2.0 ** -7 if dtype == "bf16" else 2.0 ** -10
    a, b = runs[0][0].float(), runs[1][0].float()
    assert (a - b).abs().max() <= 8 * ulp * a.abs().max()
    for x, y in zip(runs[0][1] + runs[0][2], runs[1][1] + runs[1][2]):
        assert (x.float() - y.float()).abs().max() <= 8 * ulp * x.float().abs().max()
