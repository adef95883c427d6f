"""GPU parity tests for the int8 KV cache: the quantizing append must reproduce the oracle's bytes exactly (the
reference compares its int8 cache output exactly, tests/single_op.rs:1233-1244) and attention over the quantized cache
must agree with the oracle within 1e-2 of the output scale for bf16/fp16."""
import numpy as np
import pytest
import torch

from oracle import ref_ops as R

pytestmark = pytest.mark.gpu

ops = None
NAME = {torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32"}


@pytest.fixture(scope="module", autouse=True)
def _load():
    global ops
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from my_nn_engine_b200 import ops as _ops
    ops = _ops


def rel_err(got, want):
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def test_quantizing_kv_cache_update_golden(single_op):
    fx = single_op("quantizing_kvcache_update")
    cache, scale, new, offset = fx.inputs
    c = torch.from_numpy(cache.copy()).cuda()
    s = torch.from_numpy(scale.view(np.int16).copy()).cuda().view(torch.bfloat16)
    n = torch.from_numpy(new.view(np.int16).copy()).cuda().view(torch.bfloat16)
    ops.quantizing_kv_cache_update(c, s, n, int(offset))
    assert np.array_equal(c.cpu().numpy(), fx.outputs[0])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("b,h,s,d,t,offset", [(1, 2, 8, 4, 2, 3), (2, 8, 64, 128, 1, 63), (3, 4, 40, 64, 7, 11),
                                              (1, 1, 16, 96, 16, 0), (32, 8, 33, 128, 1, 5)])
def test_quantizing_kv_cache_update_bytes_equal_oracle(dtype, b, h, s, d, t, offset):
    rng = np.random.default_rng(b * 131 + s + d + t)
    new = torch.from_numpy((rng.standard_normal((b, h, t, d)) * rng.uniform(0.01, 30, (b, h, t, 1))).astype(np.float32)).to(dtype)
    new[0, 0, 0] = 0  # an all-zero row: scale 0, bytes 0
    if t > 1:
        new[0, 0, 1, 1:] = 0  # a single non-zero value maps to +-127
    cache = torch.from_numpy(rng.integers(-128, 128, (b, h, s, d), dtype=np.int8))
    scale = torch.from_numpy(rng.standard_normal((b, h, s)).astype(np.float32)).to(dtype)
    want_c, want_s = R.quantizing_kv_cache_update(cache.numpy().copy(), scale.float().numpy().copy(), new.float().numpy(),
                                                  offset, NAME[dtype])
    c, sc = cache.cuda(), scale.cuda()
    # the offset once as a host scalar, once as a device scalar
    ops.quantizing_kv_cache_update(c, sc, new.cuda(), offset)
    assert np.array_equal(c.cpu().numpy(), want_c)
    assert np.array_equal(sc.float().cpu().numpy(), want_s)
    c2, sc2 = cache.cuda(), scale.cuda()
    ops.quantizing_kv_cache_update(c2, sc2, new.cuda(), torch.tensor([offset], dtype=torch.int32, device="cuda"))
    assert torch.equal(c2, c) and torch.equal(sc2, sc)


def test_quantizing_kv_cache_update_rejects_rows_past_the_cache():
    from my_nn_engine_b200 import ffi
    c = torch.zeros(1, 2, 8, 4, dtype=torch.int8, device="cuda")
    s = torch.zeros(1, 2, 8, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ffi.MynnError):
        ops.quantizing_kv_cache_update(c, s, torch.ones(1, 2, 2, 4, dtype=torch.bfloat16, device="cuda"), 7)
    # device-side offset: out-of-range rows are skipped, nothing is written
    ops.quantizing_kv_cache_update(c, s, torch.ones(1, 2, 2, 4, dtype=torch.bfloat16, device="cuda"),
                                   torch.tensor([8], dtype=torch.int32, device="cuda"))
    assert not c.any() and not s.any()


def _quantized_cache(rng, b, hkv, sk, d, dtype):
    k = rng.standard_normal((b, hkv, sk, d)).astype(np.float32) * rng.uniform(0.2, 3, (b, hkv, sk, 1)).astype(np.float32)
    v = rng.standard_normal((b, hkv, sk, d)).astype(np.float32) * rng.uniform(0.2, 3, (b, hkv, sk, 1)).astype(np.float32)
    kc, ks = np.zeros((b, hkv, sk, d), np.int8), np.zeros((b, hkv, sk), np.float32)
    vc, vs = np.zeros((b, hkv, sk, d), np.int8), np.zeros((b, hkv, sk), np.float32)
    R.quantizing_kv_cache_update(kc, ks, k, 0, NAME[dtype])
    R.quantizing_kv_cache_update(vc, vs, v, 0, NAME[dtype])
    return kc, ks, vc, vs


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b,hq,hkv,d,sk,active", [(1, 32, 4, 64, 256, 256), (1, 32, 4, 64, 256, 1), (2, 8, 8, 128, 96, 17),
                                                  (3, 32, 8, 128, 512, 333), (16, 32, 8, 128, 1024, 1000),
                                                  (2, 4, 1, 128, 4096, 4096), (1, 16, 2, 64, 160, 64), (2, 6, 2, 64, 81, 81),
                                                  (1, 8, 2, 128, 7, 7)])
def test_attention_q8_decode_vs_oracle(dtype, b, hq, hkv, d, sk, active):
    rng = np.random.default_rng(b * 7919 + hq * 31 + sk + active)
    q = torch.from_numpy(rng.standard_normal((b, hq, 1, d)).astype(np.float32)).to(dtype)
    kc, ks, vc, vs = _quantized_cache(rng, b, hkv, sk, d, dtype)
    scale = 1.0 / np.sqrt(d)
    want = R.attention(q.float().numpy(), kc, vc, scale, active, k_scale=ks, v_scale=vs)
    args = (q.cuda(), torch.from_numpy(kc).cuda(), torch.from_numpy(vc).cuda(), torch.from_numpy(ks).to(dtype).cuda(),
            torch.from_numpy(vs).to(dtype).cuda(), scale)
    out = ops.attention_q8(*args, active)
    assert rel_err(out.float().cpu().numpy(), want) <= 1e-2
    out2 = ops.attention_q8(*args, torch.tensor([active], dtype=torch.int32, device="cuda"))
    assert rel_err(out2.float().cpu().numpy(), want) <= 1e-2


def test_attention_q8_one_hot_rows_select_exact_values():
    """With one overwhelmingly likely row per head the output must be that row's dequantised V (checks the permuted
    head-dim and kv-row index maps of the fragment layout element by element)."""
    b, hq, hkv, d, sk = 2, 16, 2, 128, 192
    rng = np.random.default_rng(9)
    kc = np.zeros((b, hkv, sk, d), np.int8)
    vc = rng.integers(-127, 128, (b, hkv, sk, d), dtype=np.int8)
    ks = np.ones((b, hkv, sk), np.float32)
    vs = (2.0 ** rng.integers(-3, 3, (b, hkv, sk))).astype(np.float32)
    q = np.zeros((b, hq, 1, d), np.float32)
    pick = rng.integers(0, sk, (b, hq))
    col = rng.integers(0, d, (b, hq))
    for bi in range(b):
        for h in range(hq):
            q[bi, h, 0, col[bi, h]] = 1.0
    # row r of kv head g has 100 in the column of every query head that picks it
    for bi in range(b):
        for h in range(hq):
            kc[bi, h // (hq // hkv), pick[bi, h], col[bi, h]] = 100
    out = ops.attention_q8(torch.from_numpy(q).bfloat16().cuda(), torch.from_numpy(kc).cuda(), torch.from_numpy(vc).cuda(),
                           torch.from_numpy(ks).bfloat16().cuda(), torch.from_numpy(vs).bfloat16().cuda(), 1.0, sk)
    want = R.attention(q, kc, vc, 1.0, sk, k_scale=ks, v_scale=vs)
    assert rel_err(out.float().cpu().numpy(), want) <= 1e-2
    got = out.float().cpu().numpy()
    for bi in range(b):
        for h in range(hq):
            g = h // (hq // hkv)
            others = [(pick[bi, hh], col[bi, hh]) for hh in range(hq) if hh // (hq // hkv) == g]
            if sum(1 for (r, c) in others if c == col[bi, h]) > 1:
                continue  # two heads of the group share a column: not one-hot
            expect = vc[bi, g, pick[bi, h]].astype(np.float32) * vs[bi, g, pick[bi, h]]
            assert np.abs(got[bi, h, 0] - expect).max() <= 0.51  # bf16 rounding of values up to 127 * 4


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("b,hq,hkv,sq,d,sk,active,causal", [(1, 4, 2, 5, 32, 16, 9, True), (2, 8, 8, 3, 128, 24, 24, True),
                                                            (1, 12, 4, 1, 96, 40, 33, False), (1, 18, 2, 1, 128, 64, 64, False)])
def test_attention_q8_generic_path_vs_oracle(dtype, b, hq, hkv, sq, d, sk, active, causal):
    rng = np.random.default_rng(sq * 100 + d)
    q = torch.from_numpy(rng.standard_normal((b, hq, sq, d)).astype(np.float32)).to(dtype)
    kc, ks, vc, vs = _quantized_cache(rng, b, hkv, sk, d, dtype)
    want = R.attention(q.float().numpy(), kc, vc, 0.2, active, is_causal=causal, k_scale=ks, v_scale=vs)
    out = ops.attention_q8(q.cuda(), torch.from_numpy(kc).cuda(), torch.from_numpy(vc).cuda(),
                           torch.from_numpy(ks).to(dtype).cuda(), torch.from_numpy(vs).to(dtype).cuda(), 0.2, active, causal)
    assert rel_err(out.float().cpu().numpy(), want) <= (1e-2 if dtype != torch.float32 else 1e-5)


def test_attention_q8_ignores_rows_past_active():
    b, hq, hkv, d, sk, active = 1, 8, 2, 128, 128, 70
    rng = np.random.default_rng(5)
    q = torch.from_numpy(rng.standard_normal((b, hq, 1, d)).astype(np.float32)).bfloat16()
    kc, ks, vc, vs = _quantized_cache(rng, b, hkv, sk, d, torch.bfloat16)
    want = R.attention(q.float().numpy(), kc, vc, 0.1, active, k_scale=ks, v_scale=vs)
    ks[:, :, active:] = np.nan
    vs[:, :, active:] = np.inf
    out = ops.attention_q8(q.cuda(), torch.from_numpy(kc).cuda(), torch.from_numpy(vc).cuda(),
                           torch.from_numpy(ks).bfloat16().cuda(), torch.from_numpy(vs).bfloat16().cuda(), 0.1, active)
    assert rel_err(out.float().cpu().numpy(), want) <= 1e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b,hq,hkv,sk,active", [(2, 8, 2, 704, 613), (3, 32, 8, 136, 97), (4, 32, 8, 4096, 4096), (1, 8, 8, 64, 1),
                                                (2, 16, 2, 200, 200), (2, 8, 2, 129, 129)])
def test_attention_q8_ring_and_direct_loads_agree(dtype, b, hq, hkv, sk, active):
    """MYNN_OPT_DECODE_RING on the int8-cache decode kernel (head_dim 128): K / V boxes and the row scales through the TMA-fed
    rings against loads issued by the threads.  Rows past active_seq_kv hold the extreme byte and NaN scales (whole boxes are
    copied: they must not leak); a cache length that is not a multiple of 8 keeps the direct form (scale rows could not be
    addressed by a 16-byte bulk copy); the last tile of the last head runs into the end of the tensor."""
    from my_nn_engine_b200 import ffi
    d = 128
    rng = np.random.default_rng(b + hq + sk + active)
    q = torch.from_numpy(rng.standard_normal((b, hq, 1, d)).astype(np.float32)).to(dtype)
    kc, ks, vc, vs = _quantized_cache(rng, b, hkv, sk, d, dtype)
    scale = 1.0 / np.sqrt(d)
    want = R.attention(q.float().numpy(), kc, vc, scale, active, k_scale=ks, v_scale=vs)
    kc, vc, ks, vs = kc.copy(), vc.copy(), ks.copy(), vs.copy()
    kc[:, :, active:] = -128
    vc[:, :, active:] = -128
    ks[:, :, active:] = np.nan
    vs[:, :, active:] = np.nan
    args = (q.cuda(), torch.from_numpy(kc).cuda(), torch.from_numpy(vc).cuda(), torch.from_numpy(ks).to(dtype).cuda(),
            torch.from_numpy(vs).to(dtype).cuda(), scale)
    outs = []
    try:
        for ring in (0, 1):
            ffi.set_option(ffi.OPT_DECODE_RING, ring)
            outs.append(ops.attention_q8(*args, active).clone())
            outs.append(ops.attention_q8(*args, torch.tensor([active], dtype=torch.int32, device="cuda")).clone())
    finally:
        ffi.set_option(ffi.OPT_DECODE_RING, 1)
    ops.attention_check()
    for o in outs:
        assert torch.isfinite(o.float()).all()
        assert rel_err(o.float().cpu().numpy(), want) <= 1e-2
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    assert (outs[0].float() - outs[2].float()).abs().max() <= 2 * ulp * outs[0].float().abs().max()
    if sk <= 200:  # same number of splits in both forms: same sums in the same order
        assert torch.equal(outs[0], outs[2]) and torch.equal(outs[1], outs[3])
