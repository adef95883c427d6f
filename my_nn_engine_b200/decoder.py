"""Host side of the decoder: lays a Llama-family int8 checkpoint out in HBM for the sm_100a kernels and drives
the library's ``model_init`` / ``model`` / ``model_destroy`` entry points.

It stands where the engine has ``ModelSpec::from_hf`` + ``build_decoder`` + ``Session::from_graph``
(crates/llm/src/decoder.rs:541-865, src/session.rs:449-624): the host owns the weights and the KV
``SessionState`` buffers (zero-initialised, one K and one V buffer ``[batch, kv_heads, max_seq, head_dim]`` per
layer, src/session.rs:337-394) and hands device pointers to the library in a fixed order.

HBM layout chosen for the kernels
  * q/k/v weights of a layer are one contiguous int8 block ``[(Hq+2Hkv)*D, hidden]`` (and their scales one block), so
    the three projections stream as a single DequantMatMul; gate/up likewise.  Bytes and scale indexing of each
    tensor are unchanged slices of the checkpoint.
  * Tensor parallel rank r of G keeps rows ``[r*N/G, (r+1)*N/G)`` of q/k/v/gate/up/lm_head (whole heads) and columns
    ``[r*K/G, (r+1)*K/G)`` of o/down with the full scale vector (f32, applied to the partial sums); embedding, norms
    and RoPE tables are replicated; each rank holds only its own KV heads.
"""
from __future__ import annotations

import ctypes
import math

import numpy as np
import torch

from . import ffi

_TORCH_DT = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}
_FFI_DT = {"bf16": ffi.BF16, "f16": ffi.F16, "f32": ffi.F32}


def rope_table(max_seq: int, head_dim: int, base: float, dtype: str):
    """cos/sin tables [max_seq, head_dim] exactly as the engine builds its initializers: angles in f64 with
    inv_freq[i] = 1 / base^(2i/D) and dim j sharing the frequency of j % (D/2) (crates/llm/src/builder.rs:359-393),
    then f64 -> f32 -> bf16 by TRUNCATION, the conversion applied to every initializer tensor
    (src/session.rs:171-175).  f16 (an extension) rounds to nearest."""
    half = head_dim // 2
    base64 = float(np.float32(base))
    inv_freq = np.array([1.0 / math.pow(base64, 2.0 * i / head_dim) for i in range(half)], dtype=np.float64)
    ang = np.arange(max_seq, dtype=np.float64)[:, None] * inv_freq[np.arange(head_dim) % half][None, :]
    out = []
    for t in (np.cos(ang), np.sin(ang)):
        f32 = t.astype(np.float32)
        if dtype == "bf16":
            bits = (f32.view(np.uint32) >> 16).astype(np.uint16)
            out.append(torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16))
        else:
            out.append(torch.from_numpy(f32).to(_TORCH_DT[dtype]))
    return out[0], out[1]


def _shard_rows(t, rank, world):
    n = t.shape[0] // world
    return t[rank * n:(rank + 1) * n]


def _shard_cols(t, rank, world):
    k = t.shape[1] // world
    return t[:, rank * k:(rank + 1) * k]


def _shard_heads(t, n_heads, rank, world):
    """Rows of a projection grouped by head: keep heads [rank*n/G, (rank+1)*n/G)."""
    per = t.shape[0] // n_heads
    h0, h1 = rank * (n_heads // world), (rank + 1) * (n_heads // world)
    return t[h0 * per:h1 * per]


class DecoderModel:
    """One tensor-parallel rank of a Llama-family decoder resident on the current CUDA device.

    cfg: HF config dict.  state: HF-named tensors with int8 weights and ``<name>.scale`` vectors (the engine's
    ``model.int8.safetensors`` contents).  output: 'logits' (the engine's graph output) or 'ids' (greedy argmax on
    the device with the engine's last-maximum tie rule).
    """

    def __init__(self, cfg: dict, state: dict, dtype: str = "bf16", max_seq_len: int = 256, batch: int = 1,
                 tp_rank: int = 0, tp_world: int = 1, output: str = "logits", use_graph: bool = True,
                 max_prefill: int = 0, device=None, tensor_gemm: bool = True, tp_fused: bool = True,
                 kv_int8: bool = False, streaming=None):
        if not torch.cuda.is_available():
            raise RuntimeError("DecoderModel needs a CUDA device: the decode path has no CPU implementation")
        self.lib = ffi.lib()
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.cfg, self.dtype, self.max_seq_len, self.batch = cfg, dtype, max_seq_len, batch
        self.tp_rank, self.tp_world, self.output = tp_rank, tp_world, output
        td = _TORCH_DT[dtype]
        h = cfg["hidden_size"]
        self.n_heads, self.n_kv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
        self.head_dim = cfg.get("head_dim") or h // self.n_heads
        self.vocab, self.ffn, self.n_layers = cfg["vocab_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
        G, r = tp_world, tp_rank
        dev = self.device

        def w8(name):
            t = state[name]
            if t.dtype != torch.int8:
                raise TypeError(f"{name}: the decode path takes int8 weights (got {t.dtype}); quantize the checkpoint first")
            return t

        def sc(name):
            return state[name + ".scale"]

        self._keep = []  # owns every device buffer handed to the library
        init = []

        def put(t, dt=None):
            t = t.to(device=dev, dtype=dt if dt is not None else t.dtype).contiguous()
            self._keep.append(t)
            init.append(t.data_ptr())
            return t

        put(w8("model.embed_tokens.weight"))
        put(sc("model.embed_tokens.weight"), td)
        for l in range(self.n_layers):
            p = f"model.layers.{l}."
            put(state[p + "input_layernorm.weight"], td)
            # q, k, v: one contiguous block, whole heads per rank
            qw = _shard_heads(w8(p + "self_attn.q_proj.weight"), self.n_heads, r, G)
            kw = _shard_heads(w8(p + "self_attn.k_proj.weight"), self.n_kv, r, G)
            vw = _shard_heads(w8(p + "self_attn.v_proj.weight"), self.n_kv, r, G)
            qs = _shard_heads(sc(p + "self_attn.q_proj.weight"), self.n_heads, r, G)
            ks = _shard_heads(sc(p + "self_attn.k_proj.weight"), self.n_kv, r, G)
            vs = _shard_heads(sc(p + "self_attn.v_proj.weight"), self.n_kv, r, G)
            wblk = torch.cat([qw, kw, vw], 0).to(dev).contiguous()
            sblk = torch.cat([qs, ks, vs], 0).to(device=dev, dtype=td).contiguous()
            self._keep += [wblk, sblk]
            nq, nkv = qw.shape[0], kw.shape[0]
            esz = sblk.element_size()
            init += [wblk.data_ptr(), sblk.data_ptr(), wblk.data_ptr() + nq * h, sblk.data_ptr() + nq * esz,
                     wblk.data_ptr() + (nq + nkv) * h, sblk.data_ptr() + (nq + nkv) * esz]
            # o: row-parallel (columns of wq), full scale; f32 scale when partial sums are all-reduced
            put(_shard_cols(w8(p + "self_attn.o_proj.weight"), r, G))
            put(sc(p + "self_attn.o_proj.weight"), torch.float32 if G > 1 else td)
            put(state[p + "post_attention_layernorm.weight"], td)
            gw = _shard_rows(w8(p + "mlp.gate_proj.weight"), r, G)
            uw = _shard_rows(w8(p + "mlp.up_proj.weight"), r, G)
            gs = _shard_rows(sc(p + "mlp.gate_proj.weight"), r, G)
            us = _shard_rows(sc(p + "mlp.up_proj.weight"), r, G)
            wblk = torch.cat([gw, uw], 0).to(dev).contiguous()
            sblk = torch.cat([gs, us], 0).to(device=dev, dtype=td).contiguous()
            self._keep += [wblk, sblk]
            f = gw.shape[0]
            init += [wblk.data_ptr(), sblk.data_ptr(), wblk.data_ptr() + f * h, sblk.data_ptr() + f * esz]
            put(_shard_cols(w8(p + "mlp.down_proj.weight"), r, G))
            put(sc(p + "mlp.down_proj.weight"), torch.float32 if G > 1 else td)
        put(state["model.norm.weight"], td)
        put(_shard_rows(w8("lm_head.weight"), r, G))
        put(_shard_rows(sc("lm_head.weight"), r, G), td)
        cos, sin = rope_table(max_seq_len, self.head_dim, cfg.get("rope_theta", 10000.0), dtype)
        put(cos)
        put(sin)

        # KV SessionState buffers: zero-initialised, owned here, persistent across steps
        kv_shape = (batch, self.n_kv // G, max_seq_len, self.head_dim)
        # kv_int8 (the engine's quant_kv_cache build option): int8 caches plus one scale per cached token
        self.kv_int8 = bool(kv_int8)
        # streaming = (sink, window): the engine's streaming_kv option; steps then go through stream()
        self.streaming = tuple(streaming) if streaming else None
        cache_dt = torch.int8 if kv_int8 else td
        self.k_cache = [torch.zeros(kv_shape, dtype=cache_dt, device=dev) for _ in range(self.n_layers)]
        self.v_cache = [torch.zeros(kv_shape, dtype=cache_dt, device=dev) for _ in range(self.n_layers)]
        self.k_scale = [torch.zeros(kv_shape[:3], dtype=td, device=dev) for _ in range(self.n_layers if kv_int8 else 0)]
        self.v_scale = [torch.zeros(kv_shape[:3], dtype=td, device=dev) for _ in range(self.n_layers if kv_int8 else 0)]
        states = []
        for l, (kc, vc) in enumerate(zip(self.k_cache, self.v_cache)):
            states += [kc.data_ptr(), vc.data_ptr()]
            if kv_int8:
                states += [self.k_scale[l].data_ptr(), self.v_scale[l].data_ptr()]

        c = ffi.ModelConfig(n_layers=self.n_layers, hidden=h, n_heads=self.n_heads, n_kv_heads=self.n_kv,
                            head_dim=self.head_dim, ffn=self.ffn, vocab=self.vocab, max_seq_len=max_seq_len, batch=batch,
                            dtype=_FFI_DT[dtype], output_mode=1 if output == "ids" else 0, tp_rank=r, tp_world=G,
                            use_graph=int(use_graph), max_prefill=max_prefill, use_tensor_gemm=int(tensor_gemm),
                            kv_int8=int(kv_int8), stream_sink=streaming[0] if streaming else 0,
                            stream_window=streaming[1] if streaming else 0,
                            rms_eps=cfg["rms_norm_eps"])
        ffi.check(self.lib.mynn_b200_model_configure(ctypes.byref(c)))
        self._init_arr = (ctypes.c_void_p * len(init))(*init)
        self._state_arr = (ctypes.c_void_p * len(states))(*states)
        with torch.cuda.device(dev):
            self.state = self.lib.model_init(self._init_arr, self._state_arr)
        ffi.check(self.lib.mynn_b200_model_status())
        if not self.state:
            raise RuntimeError("model_init returned no state")
        self.tp_fused = False
        if G > 1 and tp_fused and tensor_gemm and batch <= 32 and h % 16 == 0:
            # hand every rank's partial-sum block to every other rank (64-byte IPC handles over torch.distributed)
            import torch.distributed as dist
            buf = ctypes.create_string_buffer(64)
            ffi.check(self.lib.mynn_b200_model_tp_export(self.state, buf))
            handles = [None] * G
            dist.all_gather_object(handles, buf.raw)
            blob = ctypes.create_string_buffer(b"".join(handles), 64 * G)
            ffi.check(self.lib.mynn_b200_model_tp_attach(self.state, blob))
            self.tp_fused = True

        # host staging in pinned memory, as the engine's alloc_pinned buffers
        self._ids = torch.zeros(batch, dtype=torch.int64).pin_memory()
        self._scalars = torch.zeros(3, dtype=torch.int64).pin_memory()  # position_id, past_len, active_seq_kv
        n_out = batch if output == "ids" else batch * self.vocab
        self._out = torch.zeros(n_out, dtype=torch.int32 if output == "ids" else td).pin_memory()
        sp = self._scalars.data_ptr()
        self._in_arr = (ctypes.c_void_p * 4)(self._ids.data_ptr(), sp, sp + 8, sp + 16)
        self._out_arr = (ctypes.c_void_p * 1)(self._out.data_ptr())
        self.h2d_bytes_per_step = 16 + 8 * batch
        self.d2h_bytes_per_step = self._out.numel() * self._out.element_size()

    # ---- the engine's Session::run for the decode graph ----
    @classmethod
    def from_pretrained(cls, model_dir: str, **kwargs):
        """Build the model from a Hugging Face style directory: ``config.json`` plus ``model.int8.safetensors`` (the
        engine's quantized layout), or float safetensors that are quantized while loading."""
        from .checkpoint import load_model_dir
        cfg, state = load_model_dir(model_dir)
        return cls(cfg, state, **kwargs)

    def step(self, tokens, past_len: int, active_seq_kv: int | None = None):
        """One decode step through ``model(state, outputs, inputs)`` with HOST buffers: inputs are
        input_ids [batch,1], position_id [1] = past_len, past_len, active_seq_kv = past_len + 1
        (crates/llm/src/session.rs:508-537).  Returns a pinned host tensor: logits [batch, vocab] or ids [batch]."""
        self._ids.copy_(torch.as_tensor(tokens, dtype=torch.int64).reshape(self.batch))
        self._scalars[0] = past_len
        self._scalars[1] = past_len
        self._scalars[2] = past_len + 1 if active_seq_kv is None else active_seq_kv
        self.lib.model(self.state, self._out_arr, self._in_arr)
        ffi.check(self.lib.mynn_b200_model_status())
        return self._out if self.output == "ids" else self._out.view(self.batch, self.vocab)

    def prefill(self, tokens, past_len: int):
        """Prefill T tokens per sequence at cache rows [past_len, past_len+T); returns what step() returns for the
        last position."""
        ids = torch.as_tensor(tokens, dtype=torch.int64).reshape(self.batch, -1).contiguous()
        ffi.check(self.lib.mynn_b200_model_prefill(self.state, ids.data_ptr(), ids.shape[1], past_len, self._out.data_ptr()))
        return self._out if self.output == "ids" else self._out.view(self.batch, self.vocab)

    def stream(self, tokens, stream_pos: int):
        """Streaming-cache step: tokens [batch] (a decode step) or [batch, T] (a prefill chunk that must not evict) at
        absolute stream positions stream_pos..; returns what step() returns for the last position."""
        ids = torch.as_tensor(tokens, dtype=torch.int64).reshape(self.batch, -1).contiguous()
        ffi.check(self.lib.mynn_b200_model_stream(self.state, ids.data_ptr(), ids.shape[1], int(stream_pos), self._out.data_ptr()))
        return self._out if self.output == "ids" else self._out.view(self.batch, self.vocab)

    def step_device(self, ids_dev, past_len: int, out_dev=None, stream=None):
        """Device-resident step: ids int64 CUDA tensor [batch] (or None to reuse the resident ids); no host sync."""
        st = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        ffi.check(self.lib.mynn_b200_model_step_device(self.state, st, None if ids_dev is None else ids_dev.data_ptr(),
                                                       past_len, None if out_dev is None else out_dev.data_ptr()))

    def reset_cache(self):
        for t in self.k_cache + self.v_cache + self.k_scale + self.v_scale:
            t.zero_()

    def weight_bytes(self) -> int:
        return sum(t.numel() for t in self._keep if t.dtype == torch.int8)

    def close(self):
        if getattr(self, "state", None):
            self.lib.model_destroy(self.state)
            self.state = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
