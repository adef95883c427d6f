"""Decode attention through the entry point that needs no workspace and allocates nothing (collected last on purpose).

Some hosts of this library cannot give an operator scratch memory: the engine's Attention operator has no workspace
operand and its planner has already spent the device-memory budget when a step runs.  For them the library keeps the
split-KV partial results in a 4 MiB array of its own.  The test drives that entry point through the C ABI twice in a
row (the array is shared and keeps the last call's contents, so the second call proves it is reusable) and compares
with the CPU oracle (two-pass softmax attention in float64) and with the regular entry point, which gets a caller-owned
workspace, to the tolerance of the other attention tests."""
import numpy as np
import pytest
import torch

from oracle import ref_ops as R

pytestmark = pytest.mark.gpu


def _call_noalloc(ffi, q, k, v, scale, active, out, active_dev=None):
    b, hq, _, d = q.shape
    hkv, sk = k.shape[1], k.shape[2]
    dt = {torch.bfloat16: ffi.BF16, torch.float16: ffi.F16}[q.dtype]
    return ffi.lib().mynn_b200_attention_decode_noalloc(
        torch.cuda.current_stream().cuda_stream, out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), float(scale),
        b, hq, hkv, d, sk, int(active), None if active_dev is None else active_dev.data_ptr(), dt)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_noalloc_decode_attention_matches_workspace_entry_point_twice(dtype):
    from my_nn_engine_b200 import ffi, ops
    assert torch.cuda.is_available()
    assert ffi.lib().mynn_b200_attention_decode_noalloc_max_bytes() == 4 << 20
    g = torch.Generator(device="cuda").manual_seed(5)
    for (b, hq, hkv, d, sk, active) in [(4, 32, 8, 128, 1024, 1000), (2, 8, 2, 64, 512, 300)]:
        q = torch.randn(b, hq, 1, d, device="cuda", generator=g).to(dtype)
        k = torch.randn(b, hkv, sk, d, device="cuda", generator=g).to(dtype)
        v = torch.randn(b, hkv, sk, d, device="cuda", generator=g).to(dtype)
        scale = 1.0 / np.sqrt(d)
        want = ops.attention(q, k, v, scale, active).float()
        oracle = R.attention_softmax_f64(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(), scale, active)
        for call in range(2):  # second call reuses the array as the first left it
            out = torch.full_like(q, float("nan"))
            ffi.check(_call_noalloc(ffi, q, k, v, scale, active, out))
            torch.cuda.synchronize()
            err = (out.float() - want).abs().max().item() / want.abs().max().item()
            assert err <= 1e-2, (call, err)
            got = out.float().cpu().numpy()
            assert np.abs(got - oracle).max() / np.abs(oracle).max() <= 1e-2, call
        # device-side active length, as a replayed step would pass it
        act_dev = torch.tensor([active], dtype=torch.int32, device="cuda")
        out = torch.full_like(q, float("nan"))
        ffi.check(_call_noalloc(ffi, q, k, v, scale, sk, out, act_dev))
        torch.cuda.synchronize()
        assert (out.float() - want).abs().max().item() / want.abs().max().item() <= 1e-2


def test_noalloc_rejects_what_it_cannot_hold():
    from my_nn_engine_b200 import ffi
    q = torch.zeros(1, 4, 1, 32, device="cuda", dtype=torch.bfloat16)
    k = torch.zeros(1, 2, 64, 32, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros_like(q)
    assert _call_noalloc(ffi, q, k, k, 1.0, 64, out) == ffi.E_UNSUPPORTED  # head_dim 32 is not a fast-path shape
    assert "head_dim" in ffi.last_error()
    rc = ffi.lib().mynn_b200_attention_decode_noalloc(None, out.data_ptr(), q.data_ptr(), k.data_ptr(), k.data_ptr(), 1.0,
                                                      1, 4, 2, 64, 32, 32, None, ffi.F32)
    assert rc == ffi.E_UNSUPPORTED  # f32 tensors take the generic kernel of the regular entry point instead
    rc = ffi.lib().mynn_b200_attention_decode_noalloc(None, out.data_ptr(), q.data_ptr(), k.data_ptr(), k.data_ptr(), 1.0,
                                                      1, 3, 2, 64, 32, 32, None, ffi.BF16)
    assert rc == ffi.E_ARG
