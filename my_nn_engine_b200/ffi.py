"""ctypes binding of ``libmynn_b200.so`` — the same C ABI a Rust ``extern "C"`` block would bind.

The library is loaded lazily from the package directory (it is built in-tree by ``my_nn_engine_b200.build``).
Loading never falls back to anything else: a missing library raises ``RuntimeError``.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmynn_b200.so")

F32, BF16, F16 = 0, 1, 2
W_NK, W_KN = 0, 1
OK, E_ARG, E_CUDA, E_UNSUPPORTED, E_COMM, E_STATE = 0, -1, -2, -3, -4, -5
OPT_WAIT_BUDGET_US, OPT_KSPLIT, OPT_PREFILL_ATTENTION, OPT_INJECT_STALL, OPT_FUSE_ROPE, OPT_DECODE_RING = 1, 2, 3, 4, 5, 6


class MynnError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"mynn_b200 error {code}: {message}")
        self.code = code


class ModelConfig(ctypes.Structure):
    """Mirror of ``mynn_b200_model_config`` (include/mynn_b200.h)."""

    _fields_ = [(n, c_int32) for n in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "ffn", "vocab",
                                       "max_seq_len", "batch", "dtype", "output_mode", "tp_rank", "tp_world",
                                       "use_graph", "max_prefill", "use_tensor_gemm", "stream_sink", "stream_window", "kv_int8")] + [("rms_eps", c_float)]


class TpGroup(ctypes.Structure):
    """Mirror of ``mynn_b200_tp_group`` (include/mynn_b200.h)."""

    _fields_ = [("blocks", c_void_p * 8), ("rank", c_int32), ("world", c_int32), ("max_rows", c_int32), ("hidden", c_int32)]


# name -> (restype, argtypes); every symbol declared in include/mynn_b200.h
SIGNATURES = {
    "mynn_b200_last_error": (c_char_p, []),
    "mynn_b200_set_option": (c_int, [c_int, ctypes.c_longlong]),
    "mynn_b200_abi_version": (c_int, []),
    "mynn_b200_compiled_arch": (c_int, []),
    "mynn_b200_dequant_matmul_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "mynn_b200_dequant_matmul": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_size_t]),
    "mynn_b200_dequant_matmul_residual": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_size_t]),
    "mynn_b200_dequant_matmul_same_act": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_size_t]),
    "mynn_b200_dequant_matmul_check": (c_int, [c_void_p, c_void_p]),
    "mynn_b200_attention_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "mynn_b200_attention_check": (c_int, [c_void_p]),
    "mynn_b200_attention": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_size_t]),
    "mynn_b200_attention_masked": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_longlong, ctypes.c_longlong, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int]),
    "mynn_b200_attention_decode_noalloc_max_bytes": (c_size_t, []),
    "mynn_b200_attention_decode_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int]),
    "mynn_b200_kv_cache_update": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int]),
    "mynn_b200_quantizing_kv_cache_update": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int]),
    "mynn_b200_attention_q8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_size_t]),
    "mynn_b200_dynamic_quantize_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int]),
    "mynn_b200_quantized_matmul_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "mynn_b200_quantized_matmul": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_size_t]),
    "mynn_b200_kv_cache_update_ring": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    "mynn_b200_rope_cache_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int]),
    "mynn_b200_attention_ring": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_size_t]),
    "mynn_b200_attention_streaming": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int]),
    "mynn_b200_rms_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int]),
    "mynn_b200_add_rms_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int]),
    "mynn_b200_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int]),
    "mynn_b200_swish_mul": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int]),
    "mynn_b200_add": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int]),
    "mynn_b200_embed_gather_dequant": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int]),
    "mynn_b200_argmax_last": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int]),
    "mynn_b200_comm_unique_id": (c_int, [c_void_p]),
    "mynn_b200_comm_init": (c_int, [c_void_p, c_int, c_int]),
    "mynn_b200_comm_rank": (c_int, []),
    "mynn_b200_comm_world_size": (c_int, []),
    "mynn_b200_all_reduce": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int]),
    "mynn_b200_comm_barrier": (c_int, [c_void_p]),
    "mynn_b200_comm_destroy": (c_int, []),
    "mynn_b200_model_configure": (c_int, [POINTER(ModelConfig)]),
    "model_init": (c_void_p, [POINTER(c_void_p), POINTER(c_void_p)]),
    "model": (None, [c_void_p, POINTER(c_void_p), POINTER(c_void_p)]),
    "model_destroy": (None, [c_void_p]),
    "mynn_b200_model_status": (c_int, []),
    "mynn_b200_model_step_device": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "mynn_b200_model_prefill": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "mynn_b200_model_stream": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_void_p]),
    "mynn_b200_model_tp_export": (c_int, [c_void_p, c_void_p]),
    "mynn_b200_model_tp_attach": (c_int, [c_void_p, c_void_p]),
    "mynn_b200_attention_decode_splits": (c_int, [c_int, c_int, c_int, c_int]),
    "mynn_b200_tp_block_bytes": (c_size_t, [c_int, c_int, c_int]),
    "mynn_b200_tp_block_init": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int]),
    "mynn_b200_tp_dequant_matmul_push": (c_int, [c_void_p, POINTER(TpGroup), c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_size_t]),
    "mynn_b200_tp_reduce_norm": (c_int, [c_void_p, POINTER(TpGroup), c_int, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p, c_size_t]),
    "mynn_b200_tp_check": (c_int, [c_void_p, POINTER(TpGroup)]),
    "mynn_b200_launch_count": (c_int64, []),
    "alloc_pinned": (c_void_p, [c_size_t]),
    "free_pinned": (None, [c_void_p]),
}
_lib = None


def lib() -> ctypes.CDLL:
    """Load the library (once) and type every entry point."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m my_nn_engine_b200.build` "
                               "(there is no fallback implementation)")
        handle = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def set_option(option: int, value: int) -> None:
    check(lib().mynn_b200_set_option(option, value))


def check(code: int) -> None:
    if code != OK:
        raise MynnError(code, lib().mynn_b200_last_error().decode(errors="replace"))


def last_error() -> str:
    return lib().mynn_b200_last_error().decode(errors="replace")
