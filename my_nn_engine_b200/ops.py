"""Operator-level host API: the engine's decode-path operators over torch CUDA tensors.

Each function mirrors one operator of the engine's graph (same operand order and meaning as the ``Operator``
variants and ``args::*`` slots in src/graph/operator.rs of the engine) and forwards raw device pointers to the
C ABI.  torch is used only for device memory and streams.  Nothing here computes on the CPU: inputs must be CUDA
tensors and the call raises otherwise.
"""
from __future__ import annotations

import ctypes

import torch

from . import ffi

_DT = {torch.float32: ffi.F32, torch.bfloat16: ffi.BF16, torch.float16: ffi.F16}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}") from None


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("mynn_b200 operators need CUDA tensors (there is no CPU path)")
    if not t.is_contiguous():
        raise ValueError("mynn_b200 operators need contiguous tensors")
    return t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


_gemm_ws: dict = {}


def dequant_matmul_workspace(m, n, k, device):
    """Zero-initialised scratch for DequantMatMul (the operator's WORKSPACE slot), cached per device and stream."""
    need = ffi.lib().mynn_b200_dequant_matmul_workspace_bytes(m, n, k)
    key = (str(device), torch.cuda.current_stream().cuda_stream)
    ws = _gemm_ws.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 512), dtype=torch.uint8, device=device)
        _gemm_ws[key] = ws
    return ws


def check_workspace(ws):
    """Raise if a bounded wait inside the tcgen05 kernel expired during an earlier call that used ``ws``."""
    ffi.check(ffi.lib().mynn_b200_dequant_matmul_check(_stream(), _ptr(ws)))


def attention_check():
    """Raise if a bounded wait inside the tcgen05 prefill-attention kernel expired during an earlier call."""
    ffi.check(ffi.lib().mynn_b200_attention_check(_stream()))


def dequant_matmul(act, wq, scale, axis: int = 0, out=None, workspace="auto"):
    """``DequantMatMul{axis}(act, wq, scale[, workspace])``: act [..., K]; wq int8 [N, K] (axis 0) or [K, N] (axis 1);
    scale [N].  Output dtype = scale dtype (src/transform/shape.rs:326-345).  workspace: 'auto' (a cached scratch
    buffer), None (use only the kernels that need no scratch) or a zeroed uint8 CUDA tensor."""
    if wq.dtype != torch.int8:
        raise TypeError("wq must be int8")
    if axis not in (0, 1):
        raise ValueError("axis must be 0 or 1")
    n, k = (wq.shape[0], wq.shape[1]) if axis == 0 else (wq.shape[1], wq.shape[0])
    if act.shape[-1] != k or scale.numel() != n:
        raise ValueError(f"shape mismatch: act {tuple(act.shape)}, wq {tuple(wq.shape)}, scale {tuple(scale.shape)}")
    m = act.numel() // k if k else 0
    if out is None:
        out = torch.empty(act.shape[:-1] + (n,), dtype=scale.dtype, device=act.device)
    if isinstance(workspace, str):
        workspace = dequant_matmul_workspace(m, n, k, act.device) if axis == 0 and m > 0 else None
    ffi.check(ffi.lib().mynn_b200_dequant_matmul(_stream(), _ptr(out), _ptr(act), _ptr(wq), _ptr(scale), m, n, k,
                                                 _dt(act), _dt(scale), ffi.W_NK if axis == 0 else ffi.W_KN,
                                                 _ptr(workspace), 0 if workspace is None else workspace.numel()))
    return out


def dequant_matmul_same_act(act_like, wq, scale, out=None, workspace="auto"):
    """DequantMatMul of another weight matrix with the activations of the previous ``dequant_matmul`` call on the same
    workspace; ``act_like`` only supplies shape and dtype (its data is not read)."""
    k = wq.shape[1]
    m = act_like.numel() // k
    n = wq.shape[0]
    if out is None:
        out = torch.empty(act_like.shape[:-1] + (n,), dtype=scale.dtype, device=wq.device)
    if isinstance(workspace, str):
        workspace = dequant_matmul_workspace(m, n, k, wq.device)
    ffi.check(ffi.lib().mynn_b200_dequant_matmul_same_act(_stream(), _ptr(out), _ptr(wq), _ptr(scale), m, n, k, _dt(act_like),
                                                          _dt(scale), None if workspace is None else _ptr(workspace),
                                                          0 if workspace is None else workspace.numel()))
    return out


def dequant_matmul_residual(act, wq, scale, residual, out=None, workspace="auto"):
    """round(residual + round(DequantMatMul(act, wq, scale))); ``out`` may alias ``residual``."""
    n, k = wq.shape
    m = act.numel() // k
    if out is None:
        out = torch.empty_like(residual)
    if isinstance(workspace, str):
        workspace = dequant_matmul_workspace(m, n, k, act.device)
    ffi.check(ffi.lib().mynn_b200_dequant_matmul_residual(_stream(), _ptr(out), _ptr(act), _ptr(wq), _ptr(scale),
                                                          _ptr(residual), m, n, k, _dt(act), _ptr(workspace),
                                                          0 if workspace is None else workspace.numel()))
    return out


_workspaces: dict = {}


def attention_workspace(b, hq, hkv, d, cache_seq_len, device):
    """Zero-initialised scratch for the split-KV decode kernel, cached per shape and device."""
    need = ffi.lib().mynn_b200_attention_workspace_bytes(b, hq, hkv, d, cache_seq_len)
    key = (b, hkv, d, str(device))
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 256), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def attention(q, k, v, scale: float, active_seq_kv=None, is_causal: bool = False, out=None, workspace=None, mask=None):
    """``Attention{is_causal, scale}``: q [B,Hq,Sq,D]; k, v [B,Hkv,cache_seq_len,D]; ``active_seq_kv`` is an int
    (host scalar, as the engine passes it) or an int32 CUDA tensor (read on the device); None = all rows.
    ``mask``: the operator's optional additive mask, a tensor of q's dtype whose shape broadcasts against
    [B, Hq, Sq, cache_seq_len] the way the engine's launch allows: last dim cache_seq_len, second-to-last Sq or 1, leading
    dims either all 1 or [B, Hq]."""
    b, hq, sq, d = q.shape
    hkv, sk = k.shape[1], k.shape[2]
    if out is None:
        out = torch.empty_like(q)
    dev_ptr, host_val = None, sk
    if isinstance(active_seq_kv, torch.Tensor):
        if active_seq_kv.dtype != torch.int32:
            raise TypeError("device active_seq_kv must be int32")
        dev_ptr = _ptr(active_seq_kv)
    elif active_seq_kv is not None:
        host_val = int(active_seq_kv)
    if mask is not None:
        if mask.dtype != q.dtype or mask.shape[-1] != sk:
            raise ValueError("mask must have q's dtype and cache_seq_len as its last dim")
        rows = mask.shape[-2] if mask.dim() >= 2 else 1
        outer = 1
        for n in mask.shape[:-2]:
            outer *= n
        if rows not in (1, sq) or outer not in (1, b * hq):
            raise ValueError(f"mask shape {tuple(mask.shape)} does not broadcast against [{b}, {hq}, {sq}, {sk}]")
        ffi.check(ffi.lib().mynn_b200_attention_masked(_stream(), _ptr(out), _ptr(q), _ptr(k), _ptr(v), _ptr(mask),
                                                       rows * sk if outer > 1 else 0, sk if rows > 1 else 0, float(scale), b,
                                                       hq, hkv, sq, d, sk, host_val, dev_ptr, int(is_causal), _dt(q)))
        return out
    if workspace is None:
        workspace = attention_workspace(b, hq, hkv, d, sk, q.device)
    ffi.check(ffi.lib().mynn_b200_attention(_stream(), _ptr(out), _ptr(q), _ptr(k), _ptr(v), float(scale), b, hq, hkv,
                                            sq, d, sk, host_val, dev_ptr, int(is_causal), _dt(q), _ptr(workspace),
                                            workspace.numel()))
    return out


def kv_cache_update(cache, new, offset):
    """``KVCacheUpdate``: cache[b,h,offset+t,:] = new[b,h,t,:] in place; offset int or int32 CUDA tensor."""
    bh = cache.shape[0] * cache.shape[1]
    dev_ptr, host_val = None, 0
    if isinstance(offset, torch.Tensor):
        dev_ptr = _ptr(offset)
    else:
        host_val = int(offset)
    ffi.check(ffi.lib().mynn_b200_kv_cache_update(_stream(), _ptr(cache), _ptr(new), bh, cache.shape[2], new.shape[2],
                                                  cache.shape[3], host_val, dev_ptr, _dt(cache)))
    return cache


def quantizing_kv_cache_update(cache, scale, new, offset):
    """``QuantizingKVCacheUpdate``: quantize new[b,h,t,:] to int8 with one scale per token and write both into the
    int8 cache [B,H,S,D] / scale [B,H,S] (dtype of ``new``) in place; offset int or int32 CUDA tensor."""
    if cache.dtype != torch.int8:
        raise TypeError("cache must be int8")
    if scale.dtype != new.dtype:
        raise TypeError("scale and new rows must share a dtype")
    bh = cache.shape[0] * cache.shape[1]
    dev_ptr, host_val = None, 0
    if isinstance(offset, torch.Tensor):
        dev_ptr = _ptr(offset)
    else:
        host_val = int(offset)
    ffi.check(ffi.lib().mynn_b200_quantizing_kv_cache_update(_stream(), _ptr(cache), _ptr(scale), _ptr(new), bh,
                                                             cache.shape[2], new.shape[2], cache.shape[3], host_val,
                                                             dev_ptr, _dt(new)))
    return cache, scale


def attention_q8(q, k, v, k_scale, v_scale, scale: float, active_seq_kv=None, is_causal: bool = False, out=None,
                 workspace=None):
    """``Attention`` over an int8 KV cache: k, v int8 [B,Hkv,S,D], k_scale/v_scale [B,Hkv,S] in q's dtype."""
    b, hq, sq, d = q.shape
    hkv, sk = k.shape[1], k.shape[2]
    if k.dtype != torch.int8 or v.dtype != torch.int8:
        raise TypeError("k and v must be int8")
    if k_scale.dtype != q.dtype or v_scale.dtype != q.dtype:
        raise TypeError("scales must have the dtype of q")
    if out is None:
        out = torch.empty_like(q)
    dev_ptr, host_val = None, sk
    if isinstance(active_seq_kv, torch.Tensor):
        if active_seq_kv.dtype != torch.int32:
            raise TypeError("device active_seq_kv must be int32")
        dev_ptr = _ptr(active_seq_kv)
    elif active_seq_kv is not None:
        host_val = int(active_seq_kv)
    if workspace is None:
        workspace = attention_workspace(b, hq, hkv, d, sk, q.device)
    ffi.check(ffi.lib().mynn_b200_attention_q8(_stream(), _ptr(out), _ptr(q), _ptr(k), _ptr(v), _ptr(k_scale),
                                               _ptr(v_scale), float(scale), b, hq, hkv, sq, d, sk, host_val, dev_ptr,
                                               int(is_causal), _dt(q), _ptr(workspace), workspace.numel()))
    return out


def dynamic_quantize_linear(x, symmetric: bool = True, per_row: bool = True):
    """``DynamicQuantizeLinear{axis, symmetric}`` on a 2-D tensor: returns (y, scale, zero_point); y is int8 when
    symmetric, uint8 otherwise; per_row=True gives one scale per row, False one for the whole tensor."""
    rows, inner = x.shape
    qdt = torch.int8 if symmetric else torch.uint8
    y = torch.empty(x.shape, dtype=qdt, device=x.device)
    n = rows if per_row else 1
    scale = torch.empty(n, dtype=x.dtype, device=x.device)
    zp = torch.empty(n, dtype=qdt, device=x.device)
    ffi.check(ffi.lib().mynn_b200_dynamic_quantize_linear(_stream(), _ptr(y), _ptr(scale), _ptr(zp), _ptr(x), rows, inner,
                                                          int(symmetric), int(per_row), _dt(x)))
    if not per_row:
        return y, scale.reshape(()), zp.reshape(())
    return y, scale, zp


def quantized_matmul(lhs, lhs_scale, rhs, rhs_scale, out=None, workspace="auto"):
    """``QuantizedMatMul``: lhs int8 [M,K] with scale [M] (or a scalar), rhs int8 [N,K] with per-channel scale [N];
    the output has the dtype of the scales.  workspace None selects the plain kernel."""
    m, k = lhs.shape
    n = rhs.shape[0]
    if lhs.dtype != torch.int8 or rhs.dtype != torch.int8:
        raise TypeError("lhs and rhs must be int8")
    if out is None:
        out = torch.empty(m, n, dtype=rhs_scale.dtype, device=lhs.device)
    if isinstance(workspace, str):
        workspace = dequant_matmul_workspace(1, n, k, lhs.device)
    per_row = lhs_scale.dim() > 0 and lhs_scale.numel() == m and not (m == 1 and lhs_scale.dim() == 0)
    ffi.check(ffi.lib().mynn_b200_quantized_matmul(_stream(), _ptr(out), _ptr(lhs), _ptr(lhs_scale), int(per_row), _ptr(rhs),
                                                   _ptr(rhs_scale), m, n, k, _dt(rhs_scale),
                                                   None if workspace is None else _ptr(workspace),
                                                   0 if workspace is None else workspace.numel()))
    return out


def kv_cache_update_ring(cache, new, offset: int, ring_sink: int, ring_window: int, ring_start: int):
    """``KVCacheUpdate`` with ring operands: row offset+t goes to slot ring_phys_index(offset+t)."""
    bh = cache.shape[0] * cache.shape[1]
    ffi.check(ffi.lib().mynn_b200_kv_cache_update_ring(_stream(), _ptr(cache), _ptr(new), bh, cache.shape[2], new.shape[2],
                                                       cache.shape[3], int(offset), ring_sink, ring_window, ring_start, _dt(cache)))
    return cache


def rope_cache_rows(cache, cos_table, sin_table, kv_position, active_seq_kv: int, out=None):
    """``rope_fused`` over a cache [B,H,S,D]: slot s < active rotates at table row kv_position[s] (int64 CUDA [S])."""
    b, h, s, d = cache.shape
    if out is None:
        out = torch.zeros_like(cache)
    ffi.check(ffi.lib().mynn_b200_rope_cache_rows(_stream(), _ptr(out), _ptr(cache), _ptr(cos_table), _ptr(sin_table),
                                                  _ptr(kv_position), b * h, s, d, int(active_seq_kv), _dt(cache)))
    return out


def attention_ring(q, k, v, scale: float, active_seq_kv: int, ring_sink: int, ring_window: int, ring_start: int,
                   is_causal: bool = False, out=None, workspace=None):
    """``Attention`` with the ring operands of the streaming cache."""
    b, hq, sq, d = q.shape
    hkv, sk = k.shape[1], k.shape[2]
    if out is None:
        out = torch.empty_like(q)
    if workspace is None:
        workspace = attention_workspace(b, hq, hkv, d, sk, q.device)
    ffi.check(ffi.lib().mynn_b200_attention_ring(_stream(), _ptr(out), _ptr(q), _ptr(k), _ptr(v), float(scale), b, hq, hkv, sq,
                                                 d, sk, int(active_seq_kv), int(is_causal), ring_sink, ring_window, ring_start,
                                                 _dt(q), _ptr(workspace), workspace.numel()))
    return out


def rms_norm(x, weight, eps: float, out=None):
    d = x.shape[-1]
    if out is None:
        out = torch.empty_like(x)
    ffi.check(ffi.lib().mynn_b200_rms_norm(_stream(), _ptr(out), _ptr(x), _ptr(weight), float(eps), x.numel() // d, d, _dt(x)))
    return out


def add_rms_norm(a, b, weight, eps: float):
    """Returns (round(a + b), RMSNorm of it)."""
    d = a.shape[-1]
    s, n = torch.empty_like(a), torch.empty_like(a)
    ffi.check(ffi.lib().mynn_b200_add_rms_norm(_stream(), _ptr(s), _ptr(n), _ptr(a), _ptr(b), _ptr(weight), float(eps),
                                               a.numel() // d, d, _dt(a)))
    return s, n


def rope(x, cos_table, sin_table, position, out=None):
    """Fused RoPE: x [..., S, D]; tables [max_pos, D]; position int64 CUDA tensor [S]."""
    s, d = x.shape[-2], x.shape[-1]
    if out is None:
        out = torch.empty_like(x)
    ffi.check(ffi.lib().mynn_b200_rope(_stream(), _ptr(out), _ptr(x), _ptr(cos_table), _ptr(sin_table), _ptr(position),
                                       x.numel() // (s * d) if s * d else 0, s, d, _dt(x)))
    return out


def swish_mul(gate, up, out=None):
    if out is None:
        out = torch.empty_like(gate)
    ffi.check(ffi.lib().mynn_b200_swish_mul(_stream(), _ptr(out), _ptr(gate), _ptr(up), gate.numel(), _dt(gate)))
    return out


def add(a, b, out=None):
    if out is None:
        out = torch.empty_like(a)
    ffi.check(ffi.lib().mynn_b200_add(_stream(), _ptr(out), _ptr(a), _ptr(b), a.numel(), _dt(a)))
    return out


def embed_gather_dequant(table, scale, ids):
    """Gather(DequantizeLinear(table, scale, axis=0), ids): table int8 [V,H]; scale [V]; ids int64 CUDA tensor."""
    v, h = table.shape
    out = torch.empty(tuple(ids.shape) + (h,), dtype=scale.dtype, device=table.device)
    ffi.check(ffi.lib().mynn_b200_embed_gather_dequant(_stream(), _ptr(out), _ptr(table), _ptr(scale), _ptr(ids),
                                                       ids.numel(), h, v, _dt(scale)))
    return out


def argmax_last(logits):
    """Per-row greedy pick, last index among equal maxima; returns int32 CUDA tensor [rows]."""
    v = logits.shape[-1]
    rows = logits.numel() // v
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    ffi.check(ffi.lib().mynn_b200_argmax_last(_stream(), _ptr(out), _ptr(logits), rows, v, _dt(logits)))
    return out


def attention_streaming(q, k, v, scale: float, active_seq_kv: int, is_causal: bool = False, ring=(0, 0, 0), k_scale=None, v_scale=None,
                        cos_table=None, sin_table=None, kv_position=None, out=None):
    """``Attention`` with its streaming operands: ring = (sink, window, start); k/v int8 with k_scale/v_scale, or of q's dtype;
    kv_position (int64 CUDA tensor, indexed by logical row) switches the in-kernel key rotation on."""
    b, hq, sq, d = q.shape
    hkv, sk = k.shape[1], k.shape[2]
    if out is None:
        out = torch.empty_like(q)
    q8 = k.dtype == torch.int8
    ffi.check(ffi.lib().mynn_b200_attention_streaming(_stream(), _ptr(out), _ptr(q), _ptr(k), _ptr(v), _ptr(k_scale), _ptr(v_scale),
                                                      float(scale), b, hq, hkv, sq, d, sk, int(active_seq_kv), None, int(is_causal),
                                                      ring[0], ring[1], ring[2], _ptr(cos_table), _ptr(sin_table), _ptr(kv_position),
                                                      _dt(q), int(q8)))
    return out


# ---- fused tensor-parallel operators (one TpGroup per rank; see include/mynn_b200.h) ----------------------------------
class TpGroup:
    """One rank's view of a tensor-parallel group: ``blocks`` are the uint8 CUDA tensors of every rank's shared block as this
    process sees them (``tp_block_bytes`` each, initialised by their owner with ``tp_block_init``; blocks[rank] is the rank's own)."""

    def __init__(self, blocks, rank: int, max_rows: int, hidden: int):
        self.blocks, self.rank, self.world, self.max_rows, self.hidden = list(blocks), rank, len(blocks), max_rows, hidden
        self.c = ffi.TpGroup()
        for i, b in enumerate(self.blocks):
            self.c.blocks[i] = _ptr(b)
        self.c.rank, self.c.world, self.c.max_rows, self.c.hidden = rank, self.world, max_rows, hidden


def tp_block_bytes(max_rows: int, hidden: int, world: int) -> int:
    return ffi.lib().mynn_b200_tp_block_bytes(max_rows, hidden, world)


def tp_block_init(block, max_rows: int, hidden: int, world: int) -> None:
    """Header zero, every partial-sum slot empty; once per block, before any rank's first push (and again, with all ranks
    idle, after a reduction that timed out on a late peer)."""
    ffi.check(ffi.lib().mynn_b200_tp_block_init(_stream(), _ptr(block), max_rows, hidden, world))


def tp_dequant_matmul_push(group: TpGroup, buffer: int, act, wq, scale, workspace="auto"):
    """Row-parallel DequantMatMul of this rank's K shard; the f32 partial sums go into every rank's block."""
    n, k = wq.shape
    m = act.numel() // k
    if n != group.hidden or scale.dtype != torch.float32:
        raise ValueError("push: wq must have `hidden` rows and an f32 scale")
    if isinstance(workspace, str):
        workspace = dequant_matmul_workspace(m, n, k, act.device)
    ffi.check(ffi.lib().mynn_b200_tp_dequant_matmul_push(_stream(), ctypes.byref(group.c), buffer, _ptr(act), _ptr(wq), _ptr(scale), m, k,
                                                         _dt(act), _ptr(workspace), workspace.numel()))


def tp_reduce_norm(group: TpGroup, buffer: int, x, weight, eps: float, workspace):
    """Sum the partial rows of all ranks, add them to ``x``, RMSNorm; the result is left in ``workspace`` as the activation of
    the DequantMatMul that follows (``dequant_matmul_same_act`` with the same workspace)."""
    m = x.numel() // group.hidden
    ffi.check(ffi.lib().mynn_b200_tp_reduce_norm(_stream(), ctypes.byref(group.c), buffer, _ptr(x), None if weight is None else _ptr(weight),
                                                 float(eps), m, _dt(x), _ptr(workspace), workspace.numel()))


def tp_check(group: TpGroup):
    ffi.check(ffi.lib().mynn_b200_tp_check(_stream(), ctypes.byref(group.c)))
