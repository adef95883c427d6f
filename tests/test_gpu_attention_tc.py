"""Prefill attention on the tcgen05 / tensor-memory kernel against the CPU oracle (engine semantics:
src/codegen/cpu/kernels/attention.rs; causal bound min(active, active - Sq + row + 1))."""
import numpy as np
import pytest
import torch

from oracle import ref_ops as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from my_nn_engine_b200 import ops as o
    return o


@pytest.fixture(scope="module")
def ffi():
    from my_nn_engine_b200 import ffi as f
    return f


def rel_err(got, want):
    return float(np.abs(got.astype(np.float64) - want).max() / max(np.abs(want).max(), 1e-30))


def make(rng, b, hq, hkv, sq, d, cache, dtype, qmul=1.0):
    q = torch.from_numpy(rng.standard_normal((b, hq, sq, d)).astype(np.float32) * qmul).to(dtype)
    k = torch.from_numpy(rng.standard_normal((b, hkv, cache, d)).astype(np.float32)).to(dtype)
    v = torch.from_numpy(rng.standard_normal((b, hkv, cache, d)).astype(np.float32)).to(dtype)
    return q, k, v


CASES = [
    # b, hq, hkv, sq, d, cache, active, causal
    (1, 4, 2, 128, 128, 128, 128, True),      # exactly one tile in both directions
    (2, 8, 2, 100, 128, 300, 250, True),      # ragged query tile, past of 150 rows, partial last kv tile
    (1, 2, 1, 130, 128, 512, 130, True),      # two query tiles, the second with two rows
    (1, 4, 4, 64, 64, 64, 64, True),          # smallest accepted chunk, head dim 64
    (3, 6, 3, 65, 64, 129, 129, True),
    (1, 8, 8, 257, 128, 257, 257, False),     # full (non-causal) attention, three kv tiles
    (1, 8, 2, 512, 128, 1024, 700, True),     # past 188: the diagonal crosses tile borders
    (2, 4, 1, 384, 64, 640, 640, True),       # GQA group of 4, past 256
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b,hq,hkv,sq,d,cache,active,causal", CASES)
def test_tc_prefill_attention_vs_oracle(ops, dtype, b, hq, hkv, sq, d, cache, active, causal):
    """Rows past active_seq_kv are NaN in both K and V: they must not matter.  Also the device-scalar active length."""
    rng = np.random.default_rng(sq * 11 + active + d)
    q, k, v = make(rng, b, hq, hkv, sq, d, cache, dtype)
    scale = 1.0 / np.sqrt(d)
    want = R.attention(q.float().numpy(), k.float().numpy(), v.float().numpy(), scale, active, is_causal=causal)
    k[:, :, active:] = float("nan")
    v[:, :, active:] = float("nan")
    out = ops.attention(q.cuda(), k.cuda(), v.cuda(), scale, active, causal)
    ops.attention_check()
    assert rel_err(out.float().cpu().numpy(), want) <= 1e-2
    out2 = ops.attention(q.cuda(), k.cuda(), v.cuda(), scale, torch.tensor([active], dtype=torch.int32, device="cuda"), causal)
    ops.attention_check()
    assert torch.equal(out, out2)


@pytest.mark.parametrize("d", [64, 128])
def test_tc_prefill_attention_running_maximum_moves(ops, d):
    """Scores that keep growing along the kv axis: the maximum in use has to advance (and the output accumulator be
    rescaled in tensor memory) several times in every row."""
    rng = np.random.default_rng(3)
    b, hq, hkv, sq = 1, 2, 1, 640
    q, k, v = make(rng, b, hq, hkv, sq, d, sq, torch.bfloat16)
    q = q.abs()
    ramp = torch.linspace(0.0, 6.0, sq).view(1, 1, sq, 1)
    k = (k.float().abs() * ramp).bfloat16()  # q . k grows roughly linearly with the kv index
    scale = 1.0 / np.sqrt(d)
    want = R.attention(q.float().numpy(), k.float().numpy(), v.float().numpy(), scale, sq, is_causal=True)
    out = ops.attention(q.cuda(), k.cuda(), v.cuda(), scale, sq, True)
    ops.attention_check()
    assert rel_err(out.float().cpu().numpy(), want) <= 1e-2


def test_tc_and_mma_sync_prefill_kernels_agree(ops, ffi):
    rng = np.random.default_rng(9)
    q, k, v = make(rng, 1, 8, 2, 300, 128, 400, torch.bfloat16)
    scale = 1.0 / np.sqrt(128)
    a = ops.attention(q.cuda(), k.cuda(), v.cuda(), scale, 400, True)
    ops.attention_check()
    ffi.set_option(ffi.OPT_PREFILL_ATTENTION, 0)
    try:
        b_ = ops.attention(q.cuda(), k.cuda(), v.cuda(), scale, 400, True)
    finally:
        ffi.set_option(ffi.OPT_PREFILL_ATTENTION, 1)
    assert rel_err(a.float().cpu().numpy(), b_.float().cpu().numpy().astype(np.float64)) <= 1e-2
