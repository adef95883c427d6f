"""CPU oracle for the whole Llama decoder step and the greedy loop (numpy).

TEST INFRASTRUCTURE ONLY (see oracle/ref_ops.py).  Follows the graph the reference builds in
``crates/llm/src/decoder.rs:203-537,731-865`` and the loop in
``crates/llm/src/session.rs:333-537``, with one output store (rounding to the storage dtype) per
kernel of the reference's schedule:

  embed   DequantizeLinear(int8 table, per-row scale) stored, then Gather      decoder.rs:828-835
  layer   RMSNorm | q,k,v DequantMatMul | RoPE(q), RoPE(k) | KV append | Attention | o DequantMatMul
          | residual add | RMSNorm | gate, up DequantMatMul | Swish(gate)*up | down DequantMatMul
          | residual add                                                        decoder.rs:203-537
  head    final RMSNorm | lm_head DequantMatMul | logits -> f64 -> last-max argmax
                                                                                session.rs:683-690

The reference wires batch to 1 (decoder.rs:253-260,404,780); a leading batch dimension B is an
extension that treats every sequence independently and shares ``past_len`` across the batch, as
the reference's Attention operator shares one ``active_seq_kv`` (src/graph/operator.rs:193-197).
Weights may be float (plain MatMul, the tiny-llama-random golden) or (int8, scale) pairs.
"""
from __future__ import annotations

import numpy as np

from . import ref_ops as R


class LlamaConfig:
    def __init__(self, hidden, n_layers, n_heads, n_kv_heads, head_dim, ffn, vocab, eps, rope_theta):
        self.hidden, self.n_layers, self.n_heads, self.n_kv_heads = hidden, n_layers, n_heads, n_kv_heads
        self.head_dim, self.ffn, self.vocab, self.eps, self.rope_theta = head_dim, ffn, vocab, eps, rope_theta

    @classmethod
    def from_hf(cls, c: dict):
        """Field names of an HF config.json (crates/llm/src/hf_config.rs:46)."""
        hd = c.get("head_dim") or c["hidden_size"] // c["num_attention_heads"]
        return cls(c["hidden_size"], c["num_hidden_layers"], c["num_attention_heads"],
                   c.get("num_key_value_heads", c["num_attention_heads"]), hd, c["intermediate_size"],
                   c["vocab_size"], c["rms_norm_eps"], c.get("rope_theta", 10000.0))


class OracleLlama:
    """weights: dict of HF tensor names -> float array, or name -> int8 with name+'.scale' -> f32 array
    whose values are already representable in the storage dtype."""

    def __init__(self, cfg: LlamaConfig, weights: dict, dtype: str, max_seq_len: int, batch: int = 1,
                 kv_int8: bool = False, streaming=None, c_attention: bool = False):
        """streaming = (sink, window): the engine's ``streaming_kv`` build option (crates/llm/src/decoder.rs:280-360): K is
        cached UNROTATED in a sink + ring layout, every step re-rotates the cached keys at their recency rank
        (``rope_fused`` with ``kv_position``) and attention walks the ring in age order.  Index math: ref_ops.streaming_state.
        kv_int8: the engine's ``quant_kv_cache`` build option (crates/llm/src/decoder.rs:405-470): int8 caches with
        one scale per cached token, written by QuantizingKVCacheUpdate and read by the attention's scale operands."""
        self.cfg, self.dtype, self.max_seq, self.batch = cfg, dtype, max_seq_len, batch
        self.kv_int8 = kv_int8
        self.streaming = streaming
        # c_attention: run the attention recurrence in the C restatement (oracle.c, the same scalar loop as ref_ops.attention,
        # row-parallel) instead of numpy; for long contexts, where the numpy form takes seconds per call
        self.c_attention = c_attention and not streaming
        # streaming + kv_int8: the (streaming, quant_kv_cache) branch of the engine's graph (crates/llm/src/decoder.rs:314-326):
        # K is quantized UNROTATED into the int8 ring and rotated inside the attention kernel, in f32, at its recency rank
        self.w = {}
        for name, arr in weights.items():
            if name.endswith(".scale"):
                continue
            if arr.dtype == np.int8:
                self.w[name] = ("q", arr.astype(np.float32), np.asarray(weights[name + ".scale"], dtype=np.float32))
            else:
                self.w[name] = ("f", R.store_round(np.asarray(arr, dtype=np.float32), dtype), None)
        self.cos, self.sin = R.rope_table(max_seq_len, cfg.head_dim, cfg.rope_theta, dtype)
        shape = (batch, cfg.n_kv_heads, max_seq_len, cfg.head_dim)
        cdt = np.int8 if kv_int8 else np.float32
        self.k_cache = [np.zeros(shape, dtype=cdt) for _ in range(cfg.n_layers)]
        self.v_cache = [np.zeros(shape, dtype=cdt) for _ in range(cfg.n_layers)]
        self.k_scale = [np.zeros(shape[:3], dtype=np.float32) for _ in range(cfg.n_layers)]
        self.v_scale = [np.zeros(shape[:3], dtype=np.float32) for _ in range(cfg.n_layers)]
        self.past_len = 0

    def _st(self, x):
        return R.store_round(x, self.dtype)

    def _linear(self, x, name):
        kind, w, scale = self.w[name]
        m = int(np.prod(x.shape[:-1]))
        x2 = x.reshape(m, x.shape[-1])
        if kind == "f":
            out = x2 @ w.T
        elif m == 1:
            out = (x2 @ w.T) * scale[None, :]          # variant A (decode)
        else:
            out = x2 @ (w * scale[:, None]).T          # variant C (dequant workspace + sgemm)
        return self._st(out.reshape(x.shape[:-1] + (w.shape[0],)))

    def _embed(self, ids):
        kind, w, scale = self.w["model.embed_tokens.weight"]
        rows = w[ids]
        if kind == "q":
            rows = self._st(rows * scale[ids][..., None])
        return rows

    def forward(self, ids: np.ndarray, positions: np.ndarray, past_len: int, active: int, is_prefill: bool, stream=None):
        """ids [B,S] -> logits [B,S,V] (f32 values representable in the storage dtype).  ``stream``: the dict of
        ref_ops.streaming_state for a streaming step (positions are then the query positions)."""
        c = self.cfg
        b, s = ids.shape
        x = self._embed(ids)
        cos_r, sin_r = self.cos[positions], self.sin[positions]
        scale = np.float32(1.0) / np.sqrt(np.float32(c.head_dim))
        for l in range(c.n_layers):
            p = f"model.layers.{l}."
            n1 = self._st(R.rms_norm(x, self.w[p + "input_layernorm.weight"][1], c.eps))
            q = self._linear(n1, p + "self_attn.q_proj.weight").reshape(b, s, c.n_heads, c.head_dim).transpose(0, 2, 1, 3)
            k = self._linear(n1, p + "self_attn.k_proj.weight").reshape(b, s, c.n_kv_heads, c.head_dim).transpose(0, 2, 1, 3)
            v = self._linear(n1, p + "self_attn.v_proj.weight").reshape(b, s, c.n_kv_heads, c.head_dim).transpose(0, 2, 1, 3)
            q = self._st(R.rope(q, cos_r, sin_r))
            if stream is not None:
                if not self.kv_int8:
                    for t, slot in enumerate(stream["slots"]):  # keys are cached as the projection left them
                        self.k_cache[l][:, :, slot, :] = k[:, :, t, :]
                        self.v_cache[l][:, :, slot, :] = v[:, :, t, :]
                kp = stream["kv_position"]
                sink, window = self.streaming
                if self.kv_int8:
                    # slots are written like any quantized append; the attention then walks the live slots [0, active) with
                    # the per-slot position table and no ring remapping (the softmax does not depend on the row order, and
                    # chunks never evict, so a causal bound by slot equals the bound by rank)
                    for t, slot in enumerate(stream["slots"]):
                        R.quantizing_kv_cache_update(self.k_cache[l], self.k_scale[l], k[:, :, t:t + 1, :], slot, self.dtype)
                        R.quantizing_kv_cache_update(self.v_cache[l], self.v_scale[l], v[:, :, t:t + 1, :], slot, self.dtype)
                    a = self._st(R.attention_streaming(q, self.k_cache[l], self.v_cache[l], scale, stream["active"], 0, 0, 0,
                                                       is_causal=is_prefill, k_scale=self.k_scale[l], v_scale=self.v_scale[l],
                                                       cos_table=self.cos, sin_table=self.sin, kv_position=kp))
                else:
                    k_rot = self._st(R.rope(self.k_cache[l], self.cos[kp], self.sin[kp]))
                    a = self._st(R.attention_ring(q, k_rot, self.v_cache[l], scale, stream["active"], sink, window,
                                                  stream["ring_start"], is_causal=is_prefill))
                a = a.transpose(0, 2, 1, 3).reshape(b, s, c.n_heads * c.head_dim)
                o = self._linear(a, p + "self_attn.o_proj.weight")
                x = self._st(x + o)
                n2 = self._st(R.rms_norm(x, self.w[p + "post_attention_layernorm.weight"][1], c.eps))
                g = self._linear(n2, p + "mlp.gate_proj.weight")
                u = self._linear(n2, p + "mlp.up_proj.weight")
                h = self._st(R.swish_mul(g, u))
                d = self._linear(h, p + "mlp.down_proj.weight")
                x = self._st(x + d)
                continue
            k = self._st(R.rope(k, cos_r, sin_r))
            if self.kv_int8:
                R.quantizing_kv_cache_update(self.k_cache[l], self.k_scale[l], k, past_len, self.dtype)
                R.quantizing_kv_cache_update(self.v_cache[l], self.v_scale[l], v, past_len, self.dtype)
                if self.c_attention:
                    from . import c_oracle
                    a = self._st(c_oracle.attention_q8(q, self.k_cache[l], self.v_cache[l], self.k_scale[l], self.v_scale[l],
                                                       float(scale), active, is_prefill, parallel=True))
                else:
                    a = self._st(R.attention(q, self.k_cache[l], self.v_cache[l], scale, active, is_causal=is_prefill,
                                             k_scale=self.k_scale[l], v_scale=self.v_scale[l]))
            else:
                R.kv_cache_update(self.k_cache[l], k, past_len)
                R.kv_cache_update(self.v_cache[l], v, past_len)
                if self.c_attention:
                    from . import c_oracle
                    a = self._st(c_oracle.attention(np.ascontiguousarray(q, dtype=np.float32), self.k_cache[l], self.v_cache[l],
                                                    float(scale), active, is_prefill, parallel=True))
                else:
                    a = self._st(R.attention(q, self.k_cache[l], self.v_cache[l], scale, active, is_causal=is_prefill))
            a = a.transpose(0, 2, 1, 3).reshape(b, s, c.n_heads * c.head_dim)
            o = self._linear(a, p + "self_attn.o_proj.weight")
            x = self._st(x + o)
            n2 = self._st(R.rms_norm(x, self.w[p + "post_attention_layernorm.weight"][1], c.eps))
            g = self._linear(n2, p + "mlp.gate_proj.weight")
            u = self._linear(n2, p + "mlp.up_proj.weight")
            h = self._st(R.swish_mul(g, u))
            d = self._linear(h, p + "mlp.down_proj.weight")
            x = self._st(x + d)
        xn = self._st(R.rms_norm(x, self.w["model.norm.weight"][1], c.eps))
        return self._linear(xn, "lm_head.weight")

    # ---- decode loop (crates/llm/src/session.rs:333-537) ----
    def decode_step(self, tokens: np.ndarray) -> np.ndarray:
        """tokens [B] -> next tokens [B]; inputs are [token], [past_len], past_len, past_len+1."""
        ids = np.asarray(tokens, dtype=np.int64).reshape(self.batch, 1)
        if self.streaming:
            st = R.streaming_state(self.past_len, 1, self.streaming[0], self.streaming[1], self.max_seq)
            logits = self.forward(ids, st["q_positions"], self.past_len, st["active"], False, stream=st)
        else:
            logits = self.forward(ids, np.array([self.past_len]), self.past_len, self.past_len + 1, False)
        self.last_logits = logits[:, 0, :]
        self.past_len += 1
        return np.array([R.argmax_last(row.astype(np.float64)) for row in logits[:, 0, :]], dtype=np.int64)

    def prefill(self, prompt: np.ndarray, prefill_len: int) -> np.ndarray:
        """Chunked prefill: pad each chunk to prefill_len with token 0, is_causal, active = past+prefill_len,
        past_len advances by the real chunk size; the last chunk's row chunk_size-1 gives the token
        (crates/llm/src/session.rs:426-480).  prompt [B, T]."""
        prompt = np.asarray(prompt, dtype=np.int64).reshape(self.batch, -1)
        t = prompt.shape[1]
        pos0 = 0
        while True:
            chunk = min(t - pos0, prefill_len)
            padded = np.zeros((self.batch, prefill_len), dtype=np.int64)
            padded[:, :chunk] = prompt[:, pos0:pos0 + chunk]
            if self.streaming:
                # the engine pads streaming chunks too; padding rows would occupy ring slots, so the chunk is run at
                # its real length here (rows past it influence nothing that is kept)
                st = R.streaming_state(self.past_len, chunk, self.streaming[0], self.streaming[1], self.max_seq)
                logits = self.forward(padded[:, :chunk], st["q_positions"], self.past_len, st["active"], True, stream=st)
            else:
                positions = self.past_len + np.arange(prefill_len)
                logits = self.forward(padded, positions, self.past_len, self.past_len + prefill_len, True)
            self.past_len += chunk
            pos0 += chunk
            if pos0 == t:
                self.last_logits = logits[:, chunk - 1, :]
                return np.array([R.argmax_last(r.astype(np.float64)) for r in logits[:, chunk - 1, :]], dtype=np.int64)

    def generate(self, prompt: np.ndarray, max_new_tokens: int, prefill_len: int | None = None) -> np.ndarray:
        """Greedy ids [B, max_new_tokens].  Without prefill the prompt is fed token by token and only the
        last step's pick is kept (crates/llm/src/session.rs:371-383).  EOS / stop strings are host-loop
        features tested separately."""
        prompt = np.asarray(prompt, dtype=np.int64).reshape(self.batch, -1)
        out = []
        for i in range(max_new_tokens):
            if not self.streaming and self.max_seq < self.past_len + 1:
                break
            if i == 0:
                if prefill_len:
                    tok = self.prefill(prompt, prefill_len)
                else:
                    for j in range(prompt.shape[1]):
                        tok = self.decode_step(prompt[:, j])
            else:
                tok = self.decode_step(out[-1])
            out.append(tok)
        return np.stack(out, axis=1) if out else np.zeros((self.batch, 0), dtype=np.int64)
