"""GPU parity tests, operator level: the CUDA kernels (called through the C ABI) against the CPU oracle and the
reference's golden vectors.  Tolerances: the reference's own rule per fixture (|a-e| < eps or |a-e|/|e| < eps), and
for seeded bf16/fp16 cases max relative error <= 1e-2 measured against the output scale."""
import numpy as np
import pytest
import torch

from conftest import eq_with_epsilon
from oracle import ref_ops as R

pytestmark = pytest.mark.gpu

ops = None


@pytest.fixture(scope="module", autouse=True)
def _load():
    global ops
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from my_nn_engine_b200 import ops as _ops
    ops = _ops


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def bf16_dev(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().view(torch.bfloat16)


def to_np(t):
    return t.float().cpu().numpy()


def rel_err(got, want):
    """max |got - want| / max |want|: error relative to the output scale (robust near zero crossings)."""
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


DQMM = ["dequant_matmul", "dequant_matmul_16x16x16", "dequant_matmul_16x32x32", "dequant_matmul_32x32x64",
        "dequant_matmul_64x64x128", "dequant_matmul_128x128x64", "dequant_matmul_24x48x40",
        "dequant_matmul_17x17x17", "dequant_matmul_50x50x50", "dequant_matmul_80x96x96"]


@pytest.mark.parametrize("name", DQMM)
def test_dequant_matmul_goldens(single_op, name):
    fx = single_op(name)
    act, wq, scale = fx.inputs
    out = ops.dequant_matmul(bf16_dev(act), dev(wq), bf16_dev(scale))
    want = R.bf16_bits_to_f32(fx.outputs[0])
    ok, md = eq_with_epsilon(to_np(out).reshape(want.shape), want, 1e-1)
    assert ok, md


@pytest.mark.parametrize("path", ["tcgen05_i8", "mma_sync"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("m,n,k", [(1, 5632, 2048), (1, 2048, 5632), (2, 256, 2048), (3, 1024, 4096), (8, 512, 1024),
                                   (9, 512, 1024), (16, 4096, 4096), (17, 2048, 512), (32, 6144, 4096), (32, 4096, 14336),
                                   (32, 1008, 448), (1, 16, 64), (5, 144, 192), (40, 256, 512)])
def test_dequant_matmul_vs_oracle(path, dtype, m, n, k):
    """Both DequantMatMul kernels against the oracle: the tcgen05 int8 kernel (workspace given) and the mma.sync
    streaming kernel (no workspace).  Shapes outside a kernel's fast path exercise the generic kernel."""
    if path == "mma_sync" and dtype == torch.float32 and m * 3 > 32:
        pytest.skip("f32 activations use the mma.sync streaming kernel up to 10 rows")
    rng = np.random.default_rng(m * 1000003 + n * 101 + k)
    wq = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    scale = torch.from_numpy(rng.uniform(0.002, 0.02, size=n).astype(np.float32)).to(dtype)
    act = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(dtype)
    out = ops.dequant_matmul(act.cuda(), dev(wq), scale.cuda(), workspace="auto" if path == "tcgen05_i8" else None)
    if path == "tcgen05_i8":
        ops.check_workspace(ops.dequant_matmul_workspace(m, n, k, "cuda"))
    want = R.dequant_matmul(act.float().numpy(), wq, scale.float().numpy())
    tol = 1e-2 if dtype != torch.float32 else 1e-5
    assert rel_err(to_np(out), want) <= tol
    if dtype == torch.bfloat16:  # per-element check against the rounded oracle: at most one bf16 ulp apart
        w = R.round_bf16(want)
        assert np.abs(to_np(out) - w).max() <= np.abs(w).max() * 2.0 ** -7


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k", [(33, 128, 128), (128, 512, 1024), (200, 384, 512), (256, 1024, 4096), (300, 1008, 448),
                                   (1024, 256, 2048)])
def test_dequant_matmul_prefill_kernel_vs_oracle(dtype, m, n, k):
    """More than 32 activation rows with a workspace: the large-tile tcgen05 int8 kernel (two activation limbs).
    Tile edges in every dimension: rows 33/200/300 (128-token tiles), n 1008 (128-row tiles), k 448 (128-wide blocks)."""
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    wq = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    scale = torch.from_numpy(rng.uniform(0.002, 0.02, size=n).astype(np.float32)).to(dtype)
    act = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(dtype)
    res = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).to(dtype)
    out = ops.dequant_matmul(act.cuda(), dev(wq), scale.cuda())
    ops.check_workspace(ops.dequant_matmul_workspace(m, n, k, "cuda"))
    want = R.dequant_matmul(act.float().numpy(), wq, scale.float().numpy())
    assert rel_err(to_np(out), want) <= 1e-2
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    assert np.abs(to_np(out) - want).max() <= np.abs(want).max() * ulp
    out2 = ops.dequant_matmul_residual(act.cuda(), dev(wq), scale.cuda(), res.cuda())
    name = "bf16" if dtype == torch.bfloat16 else "f16"
    want2 = R.store_round(R.store_round(want, name) + res.float().numpy(), name)
    assert np.abs(to_np(out2) - want2).max() <= np.abs(want2).max() * 2 * ulp


@pytest.mark.parametrize("path", ["tcgen05_i8", "mma_sync"])
@pytest.mark.parametrize("ksplit", [1, 2, 4, 8])
def test_dequant_matmul_cluster_splits_agree(ksplit, path):
    """Every cluster K-split gives the oracle's result; the reduction order is fixed, so repeated calls are bit-equal.
    The int8 kernel accumulates exact integers, so its result is also identical across splits."""
    from my_nn_engine_b200 import ffi
    rng = np.random.default_rng(7)
    wq = rng.integers(-127, 128, size=(400, 2048), dtype=np.int8)
    scale = torch.from_numpy(rng.uniform(0.002, 0.02, size=400).astype(np.float32)).bfloat16()
    act = torch.from_numpy(rng.standard_normal((32, 2048)).astype(np.float32)).bfloat16()
    ws = "auto" if path == "tcgen05_i8" else None
    ref1 = ops.dequant_matmul(act.cuda(), dev(wq), scale.cuda(), workspace=ws) if ksplit > 1 else None
    ffi.set_option(ffi.OPT_KSPLIT, ksplit)
    try:
        a = ops.dequant_matmul(act.cuda(), dev(wq), scale.cuda(), workspace=ws)
        b = ops.dequant_matmul(act.cuda(), dev(wq), scale.cuda(), workspace=ws)
    finally:
        ffi.set_option(ffi.OPT_KSPLIT, 0)
    if path == "tcgen05_i8" and ref1 is not None:
        assert torch.equal(a, ref1)
    want = R.dequant_matmul(act.float().numpy(), wq, scale.float().numpy())
    assert rel_err(to_np(a), want) <= 1e-2
    assert torch.equal(a, b)


def test_dequant_matmul_same_activations_skip_the_conversion():
    """Two weight matrices on one activation tensor: the second call reuses the limbs left in the workspace and gives
    exactly what a full call gives."""
    rng = np.random.default_rng(17)
    act = torch.from_numpy(rng.standard_normal((32, 4096)).astype(np.float32)).bfloat16().cuda()
    w1, w2 = (dev(rng.integers(-127, 128, size=(n, 4096), dtype=np.int8)) for n in (1024, 6144))
    s1, s2 = (torch.from_numpy(rng.uniform(0.002, 0.02, n).astype(np.float32)).bfloat16().cuda() for n in (1024, 6144))
    full2 = ops.dequant_matmul(act, w2, s2)
    ops.dequant_matmul(act, w1, s1)
    again2 = ops.dequant_matmul_same_act(act, w2, s2)
    assert torch.equal(again2, full2)
    from my_nn_engine_b200 import ffi
    with pytest.raises(ffi.MynnError):
        ops.dequant_matmul_same_act(act, w2, s2, workspace=None)


def test_dequant_matmul_config1_both_layouts():
    """The single-op GEMV benchmark graph: int8 W [2048,5632] uniform in [-127,127], f32 per-output-channel scale U(0.002,0.02),
    f32 activation [1,2048] ~ N(0,1), seed 0 — as the literal [K,N]/axis-1 graph and as the fused [N,K]/axis-0 op."""
    rng = np.random.default_rng(0)
    w_kn = rng.integers(-127, 128, size=(2048, 5632), dtype=np.int8)
    scale = rng.uniform(0.002, 0.02, size=5632).astype(np.float32)
    act = rng.standard_normal((1, 2048)).astype(np.float32)
    want = R.dequant_matmul_variant_a(act, np.ascontiguousarray(w_kn.T), scale)
    out_kn = ops.dequant_matmul(dev(act), dev(w_kn), dev(scale), axis=1)
    w_nk = dev(np.ascontiguousarray(w_kn.T))
    assert rel_err(to_np(out_kn), want) <= 1e-5
    assert rel_err(to_np(ops.dequant_matmul(dev(act), w_nk, dev(scale), axis=0)), want) <= 1e-5
    assert rel_err(to_np(ops.dequant_matmul(dev(act), w_nk, dev(scale), axis=0, workspace=None)), want) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k", [(1, 5632, 2048), (2, 1040, 512), (1, 16, 64), (4, 528, 4112), (1, 2048, 72), (3, 100, 50)])
def test_dequant_matmul_kn_layout_vs_oracle(dtype, m, n, k):
    """The [K,N] / axis-1 form (per-column scale): the cluster-split kernel for N % 16 == 0 (column groups that are partly
    empty, k ranges that do not divide by the 8-way split, more than one pass per CTA) and the plain kernels otherwise."""
    rng = np.random.default_rng(m + n + k)
    w_kn = rng.integers(-127, 128, size=(k, n), dtype=np.int8)
    scale = torch.from_numpy(rng.uniform(0.002, 0.02, size=n).astype(np.float32)).to(dtype)
    act = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(dtype)
    want = R.dequant_matmul_variant_a(act.float().numpy(), np.ascontiguousarray(w_kn.T), scale.float().numpy())
    out = ops.dequant_matmul(act.cuda(), dev(w_kn), scale.cuda(), axis=1)
    assert rel_err(to_np(out), want) <= (1e-5 if dtype == torch.float32 else 1e-2)
    # one-hot rows read single weights back exactly: column indexing of weights and scales
    hot = torch.zeros((1, k), dtype=dtype)
    hot[0, k // 3] = 1.0
    got = to_np(ops.dequant_matmul(hot.cuda(), dev(w_kn), scale.cuda(), axis=1))[0]
    exact = R.store_round(scale.float().numpy() * w_kn[k // 3].astype(np.float32), {torch.float32: "f32", torch.bfloat16: "bf16", torch.float16: "f16"}[dtype])
    assert np.array_equal(got, exact)


def test_weight_bytes_and_scale_indexing_bit_exact():
    """One-hot activations read single weights back: out[n] = scale[n] * wq[n,k0] must be exact in f32, for every
    row n (scale indexing) and several k0 (byte position inside the 16-byte lane loads)."""
    rng = np.random.default_rng(3)
    n, k = 272, 512
    wq = rng.integers(-128, 128, size=(n, k), dtype=np.int8)
    scale = rng.uniform(0.002, 0.02, size=n).astype(np.float32)
    for k0 in [0, 1, 15, 16, 63, 64, 255, 256, 300, 511]:
        act = np.zeros((1, k), np.float32)
        act[0, k0] = 1.0
        for ws in ("auto", None):
            out = to_np(ops.dequant_matmul(dev(act), dev(wq), dev(scale), workspace=ws))
            assert np.array_equal(out[0], scale * wq[:, k0].astype(np.float32)), (k0, ws)


def test_dequant_matmul_residual_epilogue():
    rng = np.random.default_rng(11)
    wq = rng.integers(-127, 128, size=(512, 1024), dtype=np.int8)
    scale = torch.from_numpy(rng.uniform(0.002, 0.02, size=512).astype(np.float32)).bfloat16()
    act = torch.from_numpy(rng.standard_normal((4, 1024)).astype(np.float32)).bfloat16()
    res = torch.from_numpy(rng.standard_normal((4, 512)).astype(np.float32)).bfloat16()
    prod = R.round_bf16(R.dequant_matmul(act.float().numpy(), wq, scale.float().numpy()))
    want = R.round_bf16(prod + res.float().numpy())
    for ws in ("auto", None):
        out = ops.dequant_matmul_residual(act.cuda(), dev(wq), scale.cuda(), res.cuda(), workspace=ws)
        assert np.abs(to_np(out) - want).max() <= np.abs(want).max() * 2.0 ** -6


def test_int8_kernel_handles_outliers_zero_rows_and_non_finite_inputs():
    """The fixed-point activation split keeps its accuracy with a 1e4x outlier in a row, passes all-zero rows
    through, and turns a row holding Inf/NaN into NaN outputs (what f32 arithmetic would give) without touching the
    other rows."""
    rng = np.random.default_rng(13)
    wq = rng.integers(-127, 128, size=(256, 1024), dtype=np.int8)
    scale = rng.uniform(0.002, 0.02, 256).astype(np.float32)
    act = rng.standard_normal((4, 1024)).astype(np.float32)
    act[0, 7] = 1.0e4
    act[1] = 0.0
    act[2, 100] = np.inf
    out = to_np(ops.dequant_matmul(dev(act), dev(wq), dev(scale)))
    want = R.dequant_matmul_variant_a(act[[0, 1, 3]], wq, scale)
    assert rel_err(out[0], want[0]) <= 1e-5
    assert not out[1].any()
    assert np.isnan(out[2]).all()
    assert rel_err(out[3], want[2]) <= 1e-5


@pytest.mark.parametrize("name,n_in", [("attention_decode", 3), ("attention_decode_gqa", 3),
                                       ("attention_decode_runtime_kv", 4), ("attention_causal", 3),
                                       ("attention_no_causal", 3), ("attention_causal_large", 3)])
def test_attention_goldens(single_op, name, n_in):
    fx = single_op(name)
    q, k, v = (dev(x) for x in fx.inputs[:3])
    active = int(fx.inputs[3]) if n_in == 4 else None
    out = ops.attention(q, k, v, fx.attr("scale"), active, bool(fx.attr("is_causal", 0)))
    ok, md = eq_with_epsilon(to_np(out), fx.outputs[0], 1e-4)
    assert ok, md


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b,hq,hkv,d,sk,active", [(1, 32, 4, 64, 256, 256), (1, 32, 4, 64, 256, 1), (2, 8, 8, 128, 96, 17),
                                                  (3, 32, 8, 128, 512, 333), (16, 32, 8, 128, 1024, 1000),
                                                  (2, 4, 1, 128, 4096, 4096), (1, 16, 2, 64, 160, 64), (2, 6, 2, 64, 80, 80)])
def test_attention_decode_vs_oracle(dtype, b, hq, hkv, d, sk, active):
    rng = np.random.default_rng(b * 7919 + hq * 31 + sk + active)
    q = torch.from_numpy(rng.standard_normal((b, hq, 1, d)).astype(np.float32)).to(dtype)
    k = torch.from_numpy(rng.standard_normal((b, hkv, sk, d)).astype(np.float32)).to(dtype)
    v = torch.from_numpy(rng.standard_normal((b, hkv, sk, d)).astype(np.float32)).to(dtype)
    scale = 1.0 / np.sqrt(d)
    want = R.attention_softmax_f64(q.float().numpy(), k.float().numpy(), v.float().numpy(), scale, active)
    out = ops.attention(q.cuda(), k.cuda(), v.cuda(), scale, active)
    assert rel_err(to_np(out), want) <= 1e-2
    # the device-scalar form of active_seq_kv gives the same answer (it changes how rows are split)
    act_dev = torch.tensor([active], dtype=torch.int32, device="cuda")
    out2 = ops.attention(q.cuda(), k.cuda(), v.cuda(), scale, act_dev)
    assert rel_err(to_np(out2), want) <= 1e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b,hq,hkv,sq,d,cache,active,causal", [(2, 8, 2, 100, 128, 300, 250, True), (1, 4, 4, 64, 64, 64, 64, True),
                                                               (1, 2, 1, 130, 128, 512, 130, True), (2, 4, 2, 33, 64, 200, 77, False),
                                                               (1, 32, 8, 2, 128, 40, 9, True), (3, 6, 3, 65, 64, 129, 129, True),
                                                               (1, 8, 8, 257, 128, 257, 257, False)])
def test_attention_prefill_tiled_kernel_vs_oracle(dtype, b, hq, hkv, sq, d, cache, active, causal):
    """Several query rows on the tiled tensor-core kernel: tile edges in the query rows (100, 130, 33, 2, 65, 257 over
    64-row tiles) and in the kv rows, a past longer than the chunk, GQA groups 1..4, causal and full attention, and rows
    past active_seq_kv filled with NaN (they must not matter).  Also the device-scalar form of active_seq_kv."""
    rng = np.random.default_rng(sq * 7 + active + d)
    q = torch.from_numpy(rng.standard_normal((b, hq, sq, d)).astype(np.float32)).to(dtype)
    k = torch.from_numpy(rng.standard_normal((b, hkv, cache, d)).astype(np.float32)).to(dtype)
    v = torch.from_numpy(rng.standard_normal((b, hkv, cache, d)).astype(np.float32)).to(dtype)
    scale = 1.0 / np.sqrt(d)
    want = R.attention(q.float().numpy(), k.float().numpy(), v.float().numpy(), scale, active, is_causal=causal)
    k[:, :, active:] = float("nan")
    v[:, :, active:] = float("nan")
    out = ops.attention(q.cuda(), k.cuda(), v.cuda(), scale, active, causal)
    assert rel_err(to_np(out), want) <= 1e-2
    out2 = ops.attention(q.cuda(), k.cuda(), v.cuda(), scale, torch.tensor([active], dtype=torch.int32, device="cuda"), causal)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mask_shape,sq,causal", [((2, 4, 5, 24), 5, False), ((1, 1, 5, 24), 5, True), ((2, 4, 1, 24), 1, False),
                                                  ((1, 24), 3, False), ((24,), 1, False)])
def test_attention_mask_operand_vs_oracle(dtype, mask_shape, sq, causal):
    """The operator's additive mask (slot 3): full [B,Hq,Sq,Sk], broadcast over batch and heads, broadcast over query rows,
    and rank-2 / rank-1 forms, with -inf entries that remove kv rows, against the oracle's CPU recurrence."""
    rng = np.random.default_rng(sq * 31 + len(mask_shape))
    b, hq, hkv, d, sk, active = 2, 4, 2, 16, 24, 20
    q = torch.from_numpy(rng.standard_normal((b, hq, sq, d)).astype(np.float32)).to(dtype)
    k = torch.from_numpy(rng.standard_normal((b, hkv, sk, d)).astype(np.float32)).to(dtype)
    v = torch.from_numpy(rng.standard_normal((b, hkv, sk, d)).astype(np.float32)).to(dtype)
    m = rng.standard_normal(mask_shape).astype(np.float32)
    m[..., 3] = -np.inf  # kv row 3 is masked out everywhere
    mask = torch.from_numpy(m).to(dtype)
    want = R.attention(q.float().numpy(), k.float().numpy(), v.float().numpy(), 0.25, active, is_causal=causal,
                       mask=np.broadcast_to(mask.float().numpy(), (b, hq, sq, sk)) if len(mask_shape) > 2 else mask.float().numpy())
    out = ops.attention(q.cuda(), k.cuda(), v.cuda(), 0.25, active, causal, mask=mask.cuda())
    ok, md = eq_with_epsilon(to_np(out), want, 1e-4 if dtype == torch.float32 else 1e-2)
    assert ok, md


def test_attention_ignores_rows_past_active_even_if_nan():
    b, hq, hkv, d, sk, active = 1, 8, 2, 128, 128, 70
    rng = np.random.default_rng(5)
    q = torch.from_numpy(rng.standard_normal((b, hq, 1, d)).astype(np.float32)).bfloat16()
    k = torch.from_numpy(rng.standard_normal((b, hkv, sk, d)).astype(np.float32)).bfloat16()
    v = torch.from_numpy(rng.standard_normal((b, hkv, sk, d)).astype(np.float32)).bfloat16()
    want = R.attention_softmax_f64(q.float().numpy(), k.float().numpy(), v.float().numpy(), 0.1, active)
    k[:, :, active:] = float("nan")
    v[:, :, active:] = float("inf")
    out = ops.attention(q.cuda(), k.cuda(), v.cuda(), 0.1, active)
    assert rel_err(to_np(out), want) <= 1e-2


def test_kv_cache_update_golden_and_persistence(single_op):
    fx = single_op("kv_cache_update")
    cache, new, offset = fx.inputs
    c = dev(cache)
    ops.kv_cache_update(c, dev(new), int(offset))
    ok, md = eq_with_epsilon(1.0 / (1.0 + np.exp(-to_np(c).astype(np.float64))), fx.outputs[0], 1e-5)
    assert ok, md
    # zero-initialised cache, three appends, device-side offset: rows persist across calls, later rows stay zero
    kc = torch.zeros(1, 2, 8, 4, dtype=torch.bfloat16, device="cuda")
    ref = np.zeros((1, 2, 8, 4), np.float32)
    off = torch.zeros(1, dtype=torch.int32, device="cuda")
    for step in range(3):
        new = torch.full((1, 2, 1, 4), float(step + 1), dtype=torch.bfloat16, device="cuda")
        off.fill_(step)
        ops.kv_cache_update(kc, new, off)
        R.kv_cache_update(ref, to_np(new), step)
    assert np.array_equal(to_np(kc), ref) and not to_np(kc)[:, :, 3:].any()
    from my_nn_engine_b200 import ffi
    with pytest.raises(ffi.MynnError):
        ops.kv_cache_update(kc, torch.zeros(1, 2, 2, 4, dtype=torch.bfloat16, device="cuda"), 7)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_glue_ops_vs_oracle(dtype):
    rng = np.random.default_rng(21)
    name = {torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32"}[dtype]
    tol = 0 if dtype == torch.float32 else 1
    ulp = {"bf16": 2.0 ** -7, "f16": 2.0 ** -10, "f32": 2.0 ** -22}[name]

    def close(got, want):
        assert np.abs(to_np(got) - want).max() <= np.abs(want).max() * ulp, np.abs(to_np(got) - want).max()

    x = torch.from_numpy(rng.standard_normal((5, 4096)).astype(np.float32)).to(dtype)
    w = torch.from_numpy(rng.uniform(0.5, 1.5, 4096).astype(np.float32)).to(dtype)
    close(ops.rms_norm(x.cuda(), w.cuda(), 1e-5), R.store_round(R.rms_norm(x.float().numpy(), w.float().numpy(), 1e-5), name))
    y = torch.from_numpy(rng.standard_normal((5, 4096)).astype(np.float32)).to(dtype)
    s, n = ops.add_rms_norm(x.cuda(), y.cuda(), w.cuda(), 1e-5)
    s_ref = R.store_round(x.float().numpy() + y.float().numpy(), name)
    close(s, s_ref)
    close(n, R.store_round(R.rms_norm(s_ref, w.float().numpy(), 1e-5), name))
    close(ops.swish_mul(x.cuda(), y.cuda()), R.store_round(R.swish_mul(x.float().numpy(), y.float().numpy()), name))
    close(ops.add(x.cuda(), y.cuda()), s_ref)
    # RoPE with a position gather
    cos, sin = R.rope_table(64, 128, 500000.0, name)
    pos = np.array([5, 0, 63], dtype=np.int64)
    xr = torch.from_numpy(rng.standard_normal((2, 4, 3, 128)).astype(np.float32)).to(dtype)
    got = ops.rope(xr.cuda(), dev(cos, dtype), dev(sin, dtype), dev(pos))
    close(got, R.store_round(R.rope(xr.float().numpy(), cos[pos], sin[pos]), name))
    # embedding gather + dequant, argmax with ties
    table = rng.integers(-127, 128, size=(1000, 256), dtype=np.int8)
    sc = torch.from_numpy(rng.uniform(0.002, 0.02, 1000).astype(np.float32)).to(dtype)
    ids = np.array([[0, 999], [17, 17]], dtype=np.int64)
    got = ops.embed_gather_dequant(dev(table), sc.cuda(), dev(ids))
    close(got, R.store_round(table[ids].astype(np.float32) * sc.float().numpy()[ids][..., None], name))
    logits = torch.from_numpy(rng.standard_normal((3, 128256)).astype(np.float32)).to(dtype)
    logits[0, 100] = logits[0, 90000] = 50.0
    logits[1, 128255] = 60.0
    logits[2, 0] = 70.0
    got = ops.argmax_last(logits.cuda()).cpu().numpy().tolist()
    assert got == [R.argmax_last(r) for r in logits.float().numpy()] == [90000, 128255, 0]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b,hq,hkv,d,sk,active", [(2, 8, 2, 64, 700, 613), (1, 32, 8, 64, 2048, 2048), (3, 4, 4, 128, 130, 97),
                                                  (8, 32, 8, 128, 4096, 4096), (2, 16, 2, 128, 96, 17), (1, 8, 8, 128, 64, 1)])
def test_attention_decode_ring_and_direct_loads_agree(dtype, b, hq, hkv, d, sk, active):
    """MYNN_OPT_DECODE_RING: K / V tiles through the TMA-fed shared-memory rings against fragments loaded from global memory by
    the threads themselves.  Same fragments, same arithmetic: bit-identical outputs when the split count is the same (head_dim
    64, and short contexts at head_dim 128); otherwise only the order of the final merge differs.  Rows past active_seq_kv
    hold NaN (the ring copies whole 16-row boxes: they must not leak into the result), and the last row of the tensor is the
    last row of a tile (zero fill past the end)."""
    from my_nn_engine_b200 import ffi
    rng = np.random.default_rng(b + hq + sk + active)
    q = torch.from_numpy(rng.standard_normal((b, hq, 1, d)).astype(np.float32)).to(dtype).cuda()
    k = torch.from_numpy(rng.standard_normal((b, hkv, sk, d)).astype(np.float32)).to(dtype).cuda()
    v = torch.from_numpy(rng.standard_normal((b, hkv, sk, d)).astype(np.float32)).to(dtype).cuda()
    k[:, :, active:] = float("nan")
    v[:, :, active:] = float("nan")
    scale = 1.0 / np.sqrt(d)
    outs = []
    try:
        for ring in (0, 1):
            ffi.set_option(ffi.OPT_DECODE_RING, ring)
            outs.append(ops.attention(q, k, v, scale, active).clone())
            act_dev = torch.tensor([active], dtype=torch.int32, device="cuda")
            outs.append(ops.attention(q, k, v, scale, act_dev).clone())
    finally:
        ffi.set_option(ffi.OPT_DECODE_RING, 1)
    ops.attention_check()
    want = R.attention_softmax_f64(q.float().cpu().numpy(), k.float().cpu().numpy()[:, :, :active], v.float().cpu().numpy()[:, :, :active], scale, active)
    for o in outs:
        assert torch.isfinite(o.float()).all()
        assert rel_err(to_np(o), want) <= 1e-2
    same_splits = d == 64 or sk <= 130
    if same_splits:
        assert torch.equal(outs[0], outs[2]) and torch.equal(outs[1], outs[3])
    else:
        ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
        assert (outs[0].float() - outs[2].float()).abs().max() <= 2 * ulp * outs[0].float().abs().max()
