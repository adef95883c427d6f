"""CPU-only checks of the C-ABI boundary: the library loads, exports every symbol the header declares, and
rejects bad arguments with a status code and message (no compute calls are made without a GPU)."""
import os
import re

import pytest

from my_nn_engine_b200 import ffi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "mynn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\(", text)
    return sorted({n for n in names if n.startswith("mynn_b200_") or n in ("model_init", "model", "model_destroy", "alloc_pinned", "free_pinned")})


def test_header_symbols_are_exported_and_bound():
    lib = ffi.lib()
    syms = declared_symbols()
    assert len(syms) >= 30
    for name in syms:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
        assert name in ffi.SIGNATURES, f"{name} has no ctypes signature"
    assert set(ffi.SIGNATURES) == set(syms)


def test_version_and_arch():
    assert ffi.lib().mynn_b200_abi_version() == 1
    assert ffi.lib().mynn_b200_compiled_arch() == 100


def test_argument_errors_return_status_not_exit():
    lib = ffi.lib()
    assert lib.mynn_b200_rms_norm(None, None, None, None, 1e-5, -1, 4, ffi.BF16) == ffi.E_ARG
    assert "rms_norm" in ffi.last_error()
    assert lib.mynn_b200_dequant_matmul(None, None, None, None, None, 1, 16, 64, 7, ffi.BF16, ffi.W_NK, None, 0) == ffi.E_ARG
    assert lib.mynn_b200_dequant_matmul(None, None, None, None, None, 1, 16, 64, ffi.BF16, ffi.BF16, 5, None, 0) == ffi.E_ARG
    assert lib.mynn_b200_attention(None, None, None, None, None, 1.0, 1, 3, 2, 1, 64, 8, 8, None, 0, ffi.BF16, None, 0) == ffi.E_ARG
    assert "multiple" in ffi.last_error()
    assert lib.mynn_b200_kv_cache_update(None, None, None, 1, -1, 1, 4, 0, None, ffi.BF16) == ffi.E_ARG
    # empty problems are accepted without touching a device
    assert lib.mynn_b200_dequant_matmul(None, None, None, None, None, 0, 16, 64, ffi.BF16, ffi.BF16, ffi.W_NK, None, 0) == ffi.OK
    assert lib.mynn_b200_swish_mul(None, None, None, None, 0, ffi.BF16) == ffi.OK


def test_model_configure_validation():
    lib = ffi.lib()
    cfg = ffi.ModelConfig(n_layers=2, hidden=64, n_heads=4, n_kv_heads=3, head_dim=16, ffn=128, vocab=100,
                          max_seq_len=32, batch=1, dtype=ffi.BF16, output_mode=0, tp_rank=0, tp_world=1, use_graph=0,
                          max_prefill=0, use_tensor_gemm=1, stream_sink=0, stream_window=0, kv_int8=0, rms_eps=1e-5)
    assert lib.mynn_b200_model_configure(cfg) == ffi.E_ARG  # 4 heads not a multiple of 3 kv heads
    cfg.n_kv_heads = 2
    assert lib.mynn_b200_model_configure(cfg) == ffi.OK
    cfg.tp_world = 2  # no communicator of that size
    assert lib.mynn_b200_model_configure(cfg) == ffi.E_STATE
    cfg.n_heads, cfg.n_kv_heads, cfg.ffn, cfg.vocab, cfg.tp_world, cfg.tp_rank = 32, 16, 1024, 1600, 16, 3
    assert lib.mynn_b200_model_configure(cfg) == ffi.E_UNSUPPORTED  # the peer tables of the fused reduction hold 8 ranks
    assert "tp_world" in ffi.last_error()
    with pytest.raises(ffi.MynnError):
        ffi.check(lib.mynn_b200_model_configure(None))


def test_communicator_identity_world():
    """world_size 1 needs no NCCL and behaves as the identity (mirrors crates/comm/src/uds.rs:258-316 of the
    reference: world_size=1 identity); bad ranks are rejected."""
    lib = ffi.lib()
    assert lib.mynn_b200_comm_init(None, 0, 0) == ffi.E_ARG
    assert lib.mynn_b200_comm_init(None, 2, 2) == ffi.E_ARG
    assert lib.mynn_b200_comm_init(None, 0, 1) == ffi.OK
    assert lib.mynn_b200_comm_rank() == 0 and lib.mynn_b200_comm_world_size() == 1
    assert lib.mynn_b200_all_reduce(None, None, None, -1, ffi.F32) == ffi.E_ARG
    assert lib.mynn_b200_comm_destroy() == ffi.OK


def test_set_option_validates_without_a_device():
    lib = ffi.lib()
    assert lib.mynn_b200_set_option(99, 0) == ffi.E_ARG
    assert lib.mynn_b200_set_option(ffi.OPT_KSPLIT, 3) == ffi.E_ARG
    assert lib.mynn_b200_set_option(ffi.OPT_KSPLIT, 4) == ffi.OK and lib.mynn_b200_set_option(ffi.OPT_KSPLIT, 0) == ffi.OK
    assert lib.mynn_b200_set_option(ffi.OPT_PREFILL_ATTENTION, 7) == ffi.E_ARG
    assert lib.mynn_b200_set_option(ffi.OPT_WAIT_BUDGET_US, 0) == ffi.E_ARG
    assert lib.mynn_b200_set_option(ffi.OPT_INJECT_STALL, 5) == ffi.E_ARG
    assert lib.mynn_b200_set_option(ffi.OPT_FUSE_ROPE, 2) == ffi.E_ARG and lib.mynn_b200_set_option(ffi.OPT_FUSE_ROPE, 1) == ffi.OK
    assert lib.mynn_b200_set_option(ffi.OPT_DECODE_RING, -1) == ffi.E_ARG and lib.mynn_b200_set_option(ffi.OPT_DECODE_RING, 1) == ffi.OK


def test_decode_attention_split_rule():
    """Host arithmetic of the kv-row split: one wave of CTAs, at least four tiles per warp and split, at most eight splits
    unless a split would exceed 2048 rows, and then full chunks of eight."""
    lib = ffi.lib()
    f = lib.mynn_b200_attention_decode_splits
    assert f(32, 8, 2112, 2) == 1          # the benchmark step: 256 pairs fill the wave
    assert f(16, 8, 4096, 2) == 2          # config 3
    assert f(32, 2, 2112, 2) == 4 and f(32, 1, 2112, 2) == 8   # tensor-parallel shards
    assert f(1, 4, 264, 4) == 1            # a short context is not split
    assert f(1, 4, 1024, 4) == 4
    assert f(1, 8, 8192, 2) == 8 and f(1, 8, 32768, 2) == 16 and f(1, 8, 1 << 20, 2) == 32
    assert f(0, 8, 100, 2) == 0
    for pairs in (1, 3, 8, 40, 300):
        last = 1
        for rows in (16, 255, 256, 1000, 5000, 70000):
            s = f(pairs, 1, rows, 2)
            assert 1 <= s <= 64 and s * pairs <= max(296, pairs) and (s <= 8 or s % 8 == 0)
            assert s >= last  # more rows never mean fewer splits
            last = s


def test_tensor_parallel_block_geometry_and_argument_checks():
    """Host-side checks of the fused tensor-parallel operators: block size = 256-byte header + two buffers of
    world x max_rows x hidden f32 words (each rounded up to 256 bytes); bad geometry, null or misaligned blocks and bad ranks
    are refused before anything touches a device."""
    import ctypes
    lib = ffi.lib()
    assert lib.mynn_b200_tp_block_bytes(32, 4096, 8) == 256 + 2 * 8 * 32 * 4096 * 4
    assert lib.mynn_b200_tp_block_bytes(5, 48, 3) == 256 + 2 * ((3 * 5 * 48 * 4 + 255) // 256 * 256)
    for bad in ((0, 4096, 2), (33, 4096, 2), (32, 4100, 2), (32, 8, 2), (32, 4096, 0), (32, 4096, 9)):
        assert lib.mynn_b200_tp_block_bytes(*bad) == 0
        assert lib.mynn_b200_tp_block_init(None, ctypes.c_void_p(4096), *bad) == ffi.E_ARG
    assert lib.mynn_b200_tp_block_init(None, None, 32, 4096, 2) == ffi.E_ARG
    assert lib.mynn_b200_tp_block_init(None, ctypes.c_void_p(4096 + 16), 32, 4096, 2) == ffi.E_ARG  # not 256-byte aligned
    g = ffi.TpGroup()
    g.rank, g.world, g.max_rows, g.hidden = 2, 2, 32, 4096  # rank outside the group
    assert lib.mynn_b200_tp_check(None, ctypes.byref(g)) == ffi.E_ARG
    g.rank, g.world = 0, 9
    assert lib.mynn_b200_tp_reduce_norm(None, ctypes.byref(g), 0, ctypes.c_void_p(256), None, 1e-5, 1, ffi.BF16, None, 0) == ffi.E_ARG
    g.world = 2  # blocks are null
    assert lib.mynn_b200_tp_dequant_matmul_push(None, ctypes.byref(g), 0, ctypes.c_void_p(256), ctypes.c_void_p(256), ctypes.c_void_p(256),
                                                1, 64, ffi.BF16, None, 0) == ffi.E_ARG
