"""Convert the reference's own golden vectors for the decode path into small .npz fixtures.

Run once in the build container (the reference checkout is not available where the GPU tests
run):  ``python tests/golden/make_golden.py /path/to/reference``

Outputs, all under tests/golden/:
  single_op.npz          every hot-path directory of <ref>/models/test/single_op (inputs, outputs,
                         node attributes) except the 21 MB attention_causal_large case, which is
                         reduced to its first (batch, head) pair: causal attention is independent
                         per (batch, head), so the slice is itself a valid golden vector.
  tiny_llama_random.npz  the f32 weights of <ref>/models/hf/tiny-llama-random, its config, the
                         token ids of the prompt "Hello" (encoded without special tokens, as
                         crates/llm/src/session.rs:339-343 does) and the 8 expected greedy ids
                         from crates/llm/tests/tinyllama_random.rs:23-24.
bf16 tensors are kept as uint16 bit patterns.
"""
import json
import os
import struct
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import pbwire  # noqa: E402

HOT_PATH_DIRS = [
    "dequant_matmul", "dequant_matmul_16x16x16", "dequant_matmul_16x32x32", "dequant_matmul_32x32x64",
    "dequant_matmul_64x64x128", "dequant_matmul_128x128x64", "dequant_matmul_24x48x40",
    "dequant_matmul_17x17x17", "dequant_matmul_50x50x50", "dequant_matmul_80x96x96",
    "attention_decode", "attention_decode_gqa", "attention_decode_runtime_kv", "attention_causal",
    "attention_no_causal", "attention_causal_large", "kv_cache_update", "quantizing_kvcache_update",
    "dequantize_linear", "swish", "gather_default_axis",
    "dyn_quantize_linear_sym_per_row", "dyn_quantize_linear_sym_per_tensor", "dyn_quantize_linear_asym_per_row",
    "dyn_quantize_linear_asym_per_tensor", "quantized_matmul_64x64x64", "quantized_matmul_128x128x128",
    "quantized_matmul_256x128x128", "quantized_matmul_128x256x64", "quantized_matmul_1x128x128",
]


def read_safetensors(path):
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        blob = f.read()
    out = {}
    dts = {"F32": np.float32, "BF16": np.uint16, "F16": np.float16, "I8": np.int8}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        out[name] = np.frombuffer(blob[lo:hi], dtype=dts[meta["dtype"]]).reshape(meta["shape"]).copy()
    return out


def main(ref_root):
    so = os.path.join(ref_root, "models/test/single_op")
    pack = {}
    for d in HOT_PATH_DIRS:
        nodes, _ = pbwire.model_nodes(os.path.join(so, d, "model.onnx"))
        pack[f"{d}/nodes"] = np.frombuffer(json.dumps(nodes).encode(), dtype=np.uint8)
        files = sorted(f for f in os.listdir(os.path.join(so, d)) if f.endswith(".pb"))
        for f in files:
            _, dt, arr = pbwire.load_tensor(os.path.join(so, d, f))
            if d == "attention_causal_large":
                arr = arr[:1, :1].copy()
            pack[f"{d}/{f[:-3]}"] = arr
            pack[f"{d}/{f[:-3]}/dtype"] = np.int64(dt)
    here = os.path.dirname(os.path.abspath(__file__))
    np.savez_compressed(os.path.join(here, "single_op.npz"), **pack)

    from tokenizers import Tokenizer

    mdir = os.path.join(ref_root, "models/hf/tiny-llama-random")
    tok = Tokenizer.from_file(os.path.join(mdir, "tokenizer.json"))
    ids = tok.encode("Hello", add_special_tokens=False).ids
    ids_world = tok.encode(" world", add_special_tokens=False).ids
    weights = read_safetensors(os.path.join(mdir, "model.safetensors"))
    cfg = json.load(open(os.path.join(mdir, "config.json")))
    np.savez_compressed(
        os.path.join(here, "tiny_llama_random.npz"),
        config=np.frombuffer(json.dumps(cfg).encode(), dtype=np.uint8),
        prompt_ids=np.asarray(ids, dtype=np.int64),
        prompt_ids_world=np.asarray(ids_world, dtype=np.int64),
        expected_new_ids=np.asarray([3038, 25190, 6074, 6566, 21376, 8002, 12090, 28535], dtype=np.int64),
        **weights,
    )
    print("prompt ids", ids, ids_world, {k: v.shape for k, v in list(weights.items())[:12]})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
