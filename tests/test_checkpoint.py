"""Host-side tests of the checkpoint container, the int8 on-disk layout and the quantizer command, with the
known-answer cases of the reference's own quantizer tests (crates/llm/tests/quantize.rs:101-290)."""
import json
import os

import numpy as np
import torch

from my_nn_engine_b200 import checkpoint as C
from my_nn_engine_b200.quantize import quantize_state_dict

Q = "model.layers.0.self_attn.q_proj.weight"
NORM = "model.layers.0.input_layernorm.weight"


def f32(shape, data):
    return torch.tensor(data, dtype=torch.float32).reshape(shape)


def test_container_round_trip_all_dtypes(tmp_path):
    rng = np.random.default_rng(0)
    tensors = {"a.f32": torch.from_numpy(rng.standard_normal((3, 5)).astype(np.float32)),
               "b.bf16": torch.from_numpy(rng.standard_normal((7,)).astype(np.float32)).bfloat16(),
               "c.f16": torch.from_numpy(rng.standard_normal((2, 2, 2)).astype(np.float16)),
               "d.i8": torch.from_numpy(rng.integers(-128, 128, (4, 9), dtype=np.int8)),
               "e.i64": torch.arange(5), "f.empty": torch.zeros(0, 3)}
    path = str(tmp_path / "x.safetensors")
    C.write_safetensors(path, tensors, {"format": "pt"})
    with open(path, "rb") as f:
        n = int.from_bytes(f.read(8), "little")
        header = json.loads(f.read(n))
    assert n % 8 == 0 and header["__metadata__"] == {"format": "pt"}
    assert header["b.bf16"] == {"dtype": "BF16", "shape": [7], "data_offsets": [60, 74]}
    back = C.read_safetensors(path)
    assert list(back) == list(tensors)
    for k, t in tensors.items():
        assert back[k].dtype == t.dtype and back[k].shape == t.shape and torch.equal(back[k], t)


def test_quantize_single_file_known_answers(tmp_path):
    src, dst = str(tmp_path / "in.safetensors"), str(tmp_path / "out.safetensors")
    q_data = [127.0, -127.0, 0.0, 64.0, 2.0, -1.0, 0.0, 0.5, 0.0, 0.0, 0.0, 0.0]
    norm_data = [1.0, 2.0, 3.0, 4.0]
    C.write_safetensors(src, {Q: f32((3, 4), q_data), NORM: f32((4,), norm_data)})
    assert C.quantize_int8(src, dst) == {"quantized": 1, "passthrough": 1}
    out = C.read_safetensors(dst)
    assert set(out) == {Q, Q + ".scale", NORM}
    assert out[Q].dtype == torch.int8 and out[Q].shape == (3, 4) and out[Q + ".scale"].dtype == torch.bfloat16
    scales = out[Q + ".scale"].float().numpy()
    assert np.abs(scales - np.array([1.0, 2.0 / 127.0, 1.0])).max() < 1e-3
    deq = out[Q].float().numpy() * scales[:, None]
    assert np.abs(deq - np.array(q_data).reshape(3, 4)).max() < 2e-2
    assert out[Q][0].tolist() == [127, -127, 0, 64] and out[Q][1].tolist() == [127, -64, 0, 32] and not out[Q][2].any()
    assert out[NORM].dtype == torch.float32 and out[NORM].tolist() == norm_data  # passthrough, byte for byte


def test_quantizer_rounds_half_away_without_a_biased_addition():
    """x / scale = 0.5 - 2^-25 must give 0 (f32::round), although f32(|r| + 0.5) == 1.0; exactly one half goes away from
    zero.  The row maximum 127 makes the scale exactly 1, so the ratios are the inputs themselves."""
    from my_nn_engine_b200.quantize import quantize_per_channel
    from oracle import ref_ops as R
    just_below = float(np.float32(0.49999997))
    row = [127.0, just_below, -just_below, 0.5, -0.5, 1.5, -2.5, 0.0]
    assert np.floor(np.float32(just_below) + np.float32(0.5)) == 1.0  # the trap the quantizer must not fall into
    q, s = quantize_per_channel(torch.tensor([row], dtype=torch.float32))
    assert q[0].tolist() == [127, 0, 0, 1, -1, 2, -3, 0] and float(s[0]) == 1.0
    q_ref, _ = R.quantize_per_channel(np.array([row], dtype=np.float32))
    assert q_ref[0].tolist() == q[0].tolist()
    y, _, _ = R.dynamic_quantize_linear(np.array([row], dtype=np.float32), symmetric=True, per_row=True, dtype="f32")
    assert y[0].tolist() == [127, 0, 0, 1, -1, 2, -3, 0]


def test_quantize_dir_keeps_shards_and_writes_index(tmp_path):
    src_dir, dst_dir = tmp_path / "src", tmp_path / "dst"
    src_dir.mkdir()
    C.write_safetensors(str(src_dir / "shard1.safetensors"),
                        {Q: f32((2, 4), [127.0, 0.0, -127.0, 64.0, 1.0, 2.0, -1.0, 0.5]), NORM: f32((4,), [1.0, 2.0, 3.0, 4.0])})
    C.write_safetensors(str(src_dir / "shard2.safetensors"),
                        {"lm_head.weight": f32((3, 2), [1.0, -0.5, 0.25, 0.125, -1.0, 0.5]),
                         "model.embed_tokens.weight": f32((5, 2), [1.0, -0.5, 0.25, 0.0, 2.0, -1.0, 0.0, 0.125, -2.0, 1.0])})
    index = {"metadata": {"total_size": 0}, "weight_map": {Q: "shard1.safetensors", NORM: "shard1.safetensors",
                                                            "lm_head.weight": "shard2.safetensors",
                                                            "model.embed_tokens.weight": "shard2.safetensors"}}
    (src_dir / C.SAFETENSORS_INDEX).write_text(json.dumps(index))
    assert C.quantize_int8(str(src_dir), str(dst_dir)) == {"quantized": 3, "passthrough": 1}
    assert (dst_dir / "shard1.safetensors").exists() and (dst_dir / "shard2.safetensors").exists()
    out_index = json.loads((dst_dir / C.SAFETENSORS_INDEX).read_text())
    assert out_index["weight_map"] == {Q: "shard1.safetensors", Q + ".scale": "shard1.safetensors", NORM: "shard1.safetensors",
                                       "lm_head.weight": "shard2.safetensors", "lm_head.weight.scale": "shard2.safetensors",
                                       "model.embed_tokens.weight": "shard2.safetensors",
                                       "model.embed_tokens.weight.scale": "shard2.safetensors"}
    assert out_index["metadata"]["total_size"] == (8 + 4) + 16 + (6 + 6) + (10 + 10)
    # the sharded int8 directory loads through the index; a single-file output of the same input holds the same tensors
    loaded = C.load_weights_dir(str(dst_dir))
    one = str(tmp_path / "one.safetensors")
    assert C.quantize_int8(str(src_dir), one) == {"quantized": 3, "passthrough": 1}
    single = C.read_safetensors(one)
    assert set(single) == set(loaded) and all(torch.equal(single[k], loaded[k]) for k in single)


def test_f16_passthrough_becomes_bf16(tmp_path):
    src, dst = str(tmp_path / "in.safetensors"), str(tmp_path / "out.safetensors")
    x = torch.tensor([1.0, 1.00390625, -3.14159, 65504.0], dtype=torch.float16)
    C.write_safetensors(src, {NORM: x})
    C.quantize_int8(src, dst)
    out = C.read_safetensors(dst)[NORM]
    assert out.dtype == torch.bfloat16 and torch.equal(out, x.float().to(torch.bfloat16))


def test_model_dir_lookup_order_and_in_memory_quantization(tmp_path, tiny_llama):
    cfg, weights, _, _, _ = tiny_llama
    state = {k: torch.from_numpy(v) for k, v in weights.items()}
    d = tmp_path / "model"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    C.write_safetensors(str(d / C.SINGLE_SAFETENSORS), state)
    want = quantize_state_dict(state)
    _, got = C.load_model_dir(str(d))  # float checkpoint: quantized while loading
    assert set(got) == set(want) and all(torch.equal(got[k], want[k]) for k in want)
    # once model.int8.safetensors exists it wins over the float file
    assert C.main([str(d / C.SINGLE_SAFETENSORS), str(d / C.QUANTIZED_SAFETENSORS)]) == 0
    os.remove(d / C.SINGLE_SAFETENSORS)
    _, got2 = C.load_model_dir(str(d))
    assert all(torch.equal(got2[k], want[k]) for k in want)
    assert C.main([]) == 1
