"""ctypes loader for the C oracle (oracle/oracle.c).  TEST INFRASTRUCTURE ONLY."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle.so")
F32, BF16 = 0, 1


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def _p(a):
    return ctypes.c_void_p(a.ctypes.data)


def _dt(a):
    return BF16 if a.dtype == np.uint16 else F32


def dequant_matmul_fused(act, wq, scale, use_omp=True):
    """act [M,K] f32 or bf16 bits; wq [N,K] int8; scale [N] f32 or bf16 bits -> out [M,N] in scale's dtype."""
    act = np.ascontiguousarray(act)
    wq = np.ascontiguousarray(wq)
    scale = np.ascontiguousarray(scale)
    m, k = act.shape
    n = wq.shape[0]
    out = np.empty((m, n), dtype=scale.dtype)
    lib().orc_dequant_matmul_fused(_p(out), _p(act), _p(wq), _p(scale), ctypes.c_int64(m), ctypes.c_int64(n),
                                   ctypes.c_int64(k), _dt(act), _dt(scale), int(use_omp))
    return out


def dequant_matmul_workspace(act, wq, scale):
    act = np.ascontiguousarray(act)
    wq = np.ascontiguousarray(wq)
    scale = np.ascontiguousarray(scale)
    m, k = act.shape
    n = wq.shape[0]
    out = np.empty((m, n), dtype=scale.dtype)
    lib().orc_dequant_matmul_workspace(_p(out), _p(act), _p(wq), _p(scale), ctypes.c_int64(m), ctypes.c_int64(n),
                                       ctypes.c_int64(k), _dt(act), _dt(scale))
    return out


def attention(q, k, v, scale, active=None, is_causal=False, parallel=False):
    q = np.ascontiguousarray(q)
    k = np.ascontiguousarray(k)
    v = np.ascontiguousarray(v)
    b, hq, sq, d = q.shape
    hkv, sk = k.shape[1], k.shape[2]
    out = np.empty_like(q)
    lib().orc_attention(_p(out), _p(q), _p(k), _p(v), ctypes.c_float(scale), *(ctypes.c_int64(x) for x in
                        (b, hq, hkv, sq, sk, d, sk if active is None else int(active))), int(is_causal), _dt(q),
                        int(parallel))
    return out


def attention_q8(q, k, v, k_scale, v_scale, scale, active=None, is_causal=False, parallel=False):
    """q f32 [B,Hq,Sq,D]; k, v int8 [B,Hkv,Sk,D]; k_scale, v_scale f32 [B,Hkv,Sk] -> f32 [B,Hq,Sq,D]."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.int8)
    v = np.ascontiguousarray(v, dtype=np.int8)
    ks = np.ascontiguousarray(k_scale, dtype=np.float32)
    vs = np.ascontiguousarray(v_scale, dtype=np.float32)
    b, hq, sq, d = q.shape
    hkv, sk = k.shape[1], k.shape[2]
    out = np.empty_like(q)
    lib().orc_attention_q8(_p(out), _p(q), _p(k), _p(v), _p(ks), _p(vs), ctypes.c_float(scale), *(ctypes.c_int64(x) for x in
                           (b, hq, hkv, sq, sk, d, sk if active is None else int(active))), int(is_causal), int(parallel))
    return out


def rms_norm(x, w, eps):
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    d = x.shape[-1]
    lib().orc_rms_norm(_p(out), _p(x), _p(np.ascontiguousarray(w)), ctypes.c_float(eps), ctypes.c_int64(x.size // d),
                       ctypes.c_int64(d), _dt(x))
    return out


def swish_mul(g, u):
    g = np.ascontiguousarray(g)
    u = np.ascontiguousarray(u)
    out = np.empty_like(g)
    lib().orc_swish_mul(_p(out), _p(g), _p(u), ctypes.c_int64(g.size), _dt(g))
    return out


def rope(x, cos_rows, sin_rows):
    x = np.ascontiguousarray(x)
    s, d = x.shape[-2], x.shape[-1]
    out = np.empty_like(x)
    lib().orc_rope(_p(out), _p(x), _p(np.ascontiguousarray(cos_rows)), _p(np.ascontiguousarray(sin_rows)),
                   ctypes.c_int64(x.size // (s * d)), ctypes.c_int64(s), ctypes.c_int64(d), _dt(x))
    return out


def kv_cache_update(cache, new, offset):
    bh = cache.shape[0] * cache.shape[1]
    lib().orc_kv_cache_update(_p(cache), _p(np.ascontiguousarray(new)), ctypes.c_int64(bh), ctypes.c_int64(cache.shape[2]),
                              ctypes.c_int64(new.shape[2]), ctypes.c_int64(cache.shape[3]), ctypes.c_int64(int(offset)),
                              ctypes.c_int64(cache.itemsize))
    return cache
