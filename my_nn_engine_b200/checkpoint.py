"""Checkpoint I/O: the safetensors container, the engine's int8 on-disk layout and its quantizer command.

What the engine does (crates/llm/src/hf_weights.rs:65-112, crates/llm/src/quantize.rs:170-400,
crates/llm/src/bin/quantize_int8.rs) and what this module mirrors:

* a model directory is read from ``model.int8.safetensors`` if present, else from the shards named by
  ``model.safetensors.index.json``, else from ``model.safetensors``;
* a quantized tensor ``<name>`` (I8, [out, in]) travels with ``<name>.scale`` (BF16, [out]);
* ``quantize_int8 <input.safetensors|model_dir> <output.safetensors|output_dir>``: an output ending in ``.safetensors``
  is one file; otherwise the shard layout of the input directory is kept and an index is written.  Tensors that are
  not quantized pass through byte for byte, except F16, which is rewritten as BF16 (round to nearest even).

The container itself (8-byte little-endian header length, JSON header, raw little-endian tensor data) is read and
written here with numpy only; tensors are returned as torch tensors (BF16 through a uint16 view).
"""
from __future__ import annotations

import json
import os
import struct
import sys
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from .quantize import quantize_per_channel, should_quantize

QUANTIZED_SAFETENSORS = "model.int8.safetensors"
SAFETENSORS_INDEX = "model.safetensors.index.json"
SINGLE_SAFETENSORS = "model.safetensors"

_NP = {"F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I8": np.int8, "U8": np.uint8, "I32": np.int32,
       "I64": np.int64, "F64": np.float64, "BOOL": np.bool_, "I16": np.int16}
_TORCH_NAME = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.int8: "I8", torch.uint8: "U8",
               torch.int32: "I32", torch.int64: "I64", torch.float64: "F64", torch.bool: "BOOL", torch.int16: "I16"}


class CheckpointError(RuntimeError):
    pass


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """All tensors of one safetensors file (copied out of the file)."""
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise CheckpointError(f"{path}: truncated header")
        n = struct.unpack("<Q", head)[0]
        header = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        dt = meta["dtype"]
        if dt not in _NP:
            raise CheckpointError(f"{path}: tensor {name} has unsupported dtype {dt}")
        lo, hi = meta["data_offsets"]
        arr = np.frombuffer(blob[lo:hi], dtype=_NP[dt]).reshape(meta["shape"]).copy()
        t = torch.from_numpy(arr.view(np.int16)).view(torch.bfloat16) if dt == "BF16" else torch.from_numpy(arr)
        out[name] = t
    return out


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> None:
    """Write ``tensors`` in the order given; the header is padded with spaces to a multiple of 8 bytes."""
    header, chunks, off = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _TORCH_NAME:
            raise CheckpointError(f"tensor {name}: dtype {t.dtype} cannot be stored")
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        header[name] = {"dtype": _TORCH_NAME[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        chunks.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for c in chunks:
            f.write(c)


def list_shards(model_dir: str):
    """Shard files of a model directory, sorted (the index's distinct values, or the single file)."""
    index = os.path.join(model_dir, SAFETENSORS_INDEX)
    if os.path.exists(index):
        wm = json.load(open(index)).get("weight_map")
        if not isinstance(wm, dict):
            raise CheckpointError(f"{index}: missing weight_map")
        return [os.path.join(model_dir, s) for s in sorted(set(wm.values()))]
    return [os.path.join(model_dir, SINGLE_SAFETENSORS)]


def load_weights_dir(model_dir: str) -> Dict[str, torch.Tensor]:
    """The engine's lookup order: the int8 file, then the sharded index, then the single file."""
    int8 = os.path.join(model_dir, QUANTIZED_SAFETENSORS)
    if os.path.exists(int8):
        return read_safetensors(int8)
    if os.path.exists(os.path.join(model_dir, SAFETENSORS_INDEX)):
        out = {}
        for shard in list_shards(model_dir):
            out.update(read_safetensors(shard))
        return out
    single = os.path.join(model_dir, SINGLE_SAFETENSORS)
    if os.path.exists(single):
        return read_safetensors(single)
    raise CheckpointError(f"{model_dir}: no safetensors weights found")


def load_model_dir(model_dir: str) -> Tuple[dict, Dict[str, torch.Tensor]]:
    """(config.json as a dict, int8 state dict).  Float checkpoints are quantized in memory with the engine's
    quantizer, so the result is what ``quantize_int8`` followed by a load would give."""
    cfg = json.load(open(os.path.join(model_dir, "config.json")))
    state = load_weights_dir(model_dir)
    out = {}
    for name, t in state.items():
        if should_quantize(name) and t.dtype != torch.int8:
            q, s = quantize_per_channel(t)
            out[name], out[name + ".scale"] = q, s
        else:
            out[name] = t
    if cfg.get("tie_word_embeddings") and "lm_head.weight" not in out:
        out["lm_head.weight"] = out["model.embed_tokens.weight"]
        out["lm_head.weight.scale"] = out["model.embed_tokens.weight.scale"]
    for name in list(out):
        if should_quantize(name) and name + ".scale" not in out:
            raise CheckpointError(f"{name} is int8 but {name}.scale is missing")
    return cfg, out


def _convert(name: str, t: torch.Tensor, out: Dict[str, torch.Tensor], stats: dict) -> int:
    if should_quantize(name):
        q, s = quantize_per_channel(t)
        out[name], out[name + ".scale"] = q, s
        stats["quantized"] += 1
        return q.numel() + s.numel() * 2
    if t.dtype == torch.float16:
        t = t.float().to(torch.bfloat16)
    out[name] = t
    stats["passthrough"] += 1
    return t.numel() * t.element_size()


def quantize_files(files, dst: str) -> dict:
    """Several input files -> ONE output file."""
    stats = {"quantized": 0, "passthrough": 0}
    out: Dict[str, torch.Tensor] = {}
    for src in files:
        for name, t in read_safetensors(src).items():
            _convert(name, t, out, stats)
    write_safetensors(dst, out)
    return stats


def quantize_dir_streaming(src_dir: str, dst_dir: str) -> dict:
    """Shard by shard into ``dst_dir`` under the same file names; writes the index when the input had one or more than
    one shard."""
    os.makedirs(dst_dir, exist_ok=True)
    stats = {"quantized": 0, "passthrough": 0}
    weight_map, total = {}, 0
    shards = list_shards(src_dir)
    for src in shards:
        shard_name = os.path.basename(src)
        out: Dict[str, torch.Tensor] = {}
        for name, t in read_safetensors(src).items():
            total += _convert(name, t, out, stats)
        for name in out:
            weight_map[name] = shard_name
        write_safetensors(os.path.join(dst_dir, shard_name), out)
    if len(shards) > 1 or os.path.exists(os.path.join(src_dir, SAFETENSORS_INDEX)):
        with open(os.path.join(dst_dir, SAFETENSORS_INDEX), "w") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)
    return stats


def quantize_int8(in_path: str, out_path: str) -> dict:
    """The dispatch of the engine's ``quantize_int8`` command."""
    single_file_out = out_path.endswith(".safetensors")
    if os.path.isdir(in_path) and not single_file_out:
        return quantize_dir_streaming(in_path, out_path)
    if os.path.isdir(in_path):
        return quantize_files(list_shards(in_path), out_path)
    return quantize_files([in_path], out_path)


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 2:
        sys.stderr.write("usage: python -m my_nn_engine_b200.checkpoint <input.safetensors|model_dir> <output.safetensors|output_dir>\n"
                         "- if output ends with .safetensors: single-file output (loads all tensors in RAM)\n"
                         "- otherwise: sharded output dir mirroring input layout (streaming, low RAM)\n")
        return 1
    stats = quantize_int8(argv[0], argv[1])
    print(f"quantized {stats['quantized']} tensors, passed through {stats['passthrough']}")
    print(f"wrote {argv[1]}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
