"""Offline int8 per-output-channel weight quantizer: the on-disk format contract of the engine.

Mirrors ``quantize_per_channel`` of the engine (crates/llm/src/quantize.rs:124-169) and its target list
(:28-38): every ``*_proj.weight``, ``lm_head.weight`` and ``embed_tokens.weight`` becomes ``<name>`` (I8, [out, in])
plus ``<name>.scale`` (BF16, [out]).  This is checkpoint preparation, done once on the host; nothing on the decode
path calls it.
"""
from __future__ import annotations

import numpy as np
import torch

QUANT_PATTERNS = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight", "gate_proj.weight",
                  "up_proj.weight", "down_proj.weight", "lm_head.weight", "embed_tokens.weight")


def should_quantize(name: str) -> bool:
    return name.endswith(QUANT_PATTERNS)


def quantize_per_channel(w: torch.Tensor):
    """w float [N, ...] -> (int8 same shape, bf16 scale [N]).

    scale = max|row| / 127 (a zero row gets 1.0); q = clamp(round_half_away(x / scale), -128, 127) computed with the
    f32 scale; only afterwards is the scale rounded to bf16 (round to nearest even)."""
    if w.dim() < 2:
        raise ValueError(f"expected >=2D weight, got shape {tuple(w.shape)}")
    w32 = w.detach().to(torch.float32)
    rows = w32.reshape(w32.shape[0], -1)
    max_abs = rows.abs().amax(dim=1)
    scale = torch.where(max_abs == 0, torch.ones_like(max_abs), max_abs / 127.0)
    ratio = rows / scale[:, None]
    # f32::round (half away from zero) without forming |r| + 0.5, which rounds up for r = 0.5 - 2^-25: the fractional part
    # r - trunc(r) is exact in floating point
    t = torch.trunc(ratio)
    rounded = t + torch.sign(ratio) * ((ratio - t).abs() >= 0.5).to(ratio.dtype)
    q = rounded.clamp_(-128, 127).to(torch.int8).reshape(w32.shape)
    return q, scale.to(torch.bfloat16)


def quantize_state_dict(state: dict) -> dict:
    """Apply the engine's quantize_int8 pass to a dict of HF-named float tensors."""
    out = {}
    for name, t in state.items():
        if should_quantize(name):
            q, s = quantize_per_channel(t)
            out[name] = q
            out[name + ".scale"] = s
        else:
            out[name] = t
    return out


def random_llama_state(cfg: dict, seed: int = 0, std: float = 0.02, quantized: bool = True, device: str = "cpu") -> dict:
    """Random-init Llama-architecture checkpoint with HF tensor names: weights ~ N(0, std) (HF initializer_range),
    norm weights = 1.  With ``quantized`` the int8 tensors are produced layer by layer so that an 8B-class model never
    exists in float."""
    g = torch.Generator(device=device).manual_seed(seed)
    h, f, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hd = cfg.get("head_dim") or h // cfg["num_attention_heads"]
    nq, nkv = cfg["num_attention_heads"] * hd, cfg["num_key_value_heads"] * hd
    out = {}

    def put(name, shape):
        w = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std
        if quantized:
            q, s = quantize_per_channel(w)
            out[name], out[name + ".scale"] = q, s
        else:
            out[name] = w

    put("model.embed_tokens.weight", (v, h))
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        out[p + "input_layernorm.weight"] = torch.ones(h, device=device)
        out[p + "post_attention_layernorm.weight"] = torch.ones(h, device=device)
        put(p + "self_attn.q_proj.weight", (nq, h))
        put(p + "self_attn.k_proj.weight", (nkv, h))
        put(p + "self_attn.v_proj.weight", (nkv, h))
        put(p + "self_attn.o_proj.weight", (h, nq))
        put(p + "mlp.gate_proj.weight", (f, h))
        put(p + "mlp.up_proj.weight", (f, h))
        put(p + "mlp.down_proj.weight", (h, f))
    out["model.norm.weight"] = torch.ones(h, device=device)
    put("lm_head.weight", (v, h))
    return out
