"""GPU parity tests for the W8A8 operators: DynamicQuantizeLinear must reproduce the reference's golden bytes and the
oracle's bytes on seeded inputs; QuantizedMatMul accumulates exact integers, so it must agree with the oracle to the
last bit of the storage dtype (both round the same f32 value)."""
import numpy as np
import pytest
import torch

from conftest import eq_with_epsilon
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


def bf16_dev(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().view(torch.bfloat16)


@pytest.mark.parametrize("name,symmetric,per_row", [("dyn_quantize_linear_sym_per_row", True, True),
                                                    ("dyn_quantize_linear_sym_per_tensor", True, False),
                                                    ("dyn_quantize_linear_asym_per_row", False, True),
                                                    ("dyn_quantize_linear_asym_per_tensor", False, False)])
def test_dynamic_quantize_linear_goldens(single_op, name, symmetric, per_row):
    fx = single_op(name)
    y, scale, zp = ops.dynamic_quantize_linear(bf16_dev(fx.inputs[0]), symmetric, per_row)
    assert np.array_equal(y.cpu().numpy(), fx.outputs[0])
    ok, md = eq_with_epsilon(scale.float().cpu().numpy(), R.bf16_bits_to_f32(fx.outputs[1]), 1e-3)
    assert ok, md
    assert np.array_equal(zp.cpu().numpy(), fx.outputs[2])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("symmetric,per_row", [(True, True), (True, False), (False, True), (False, False)])
@pytest.mark.parametrize("rows,inner", [(1, 8), (4, 4096), (33, 1000), (2, 14336)])
def test_dynamic_quantize_linear_bytes_equal_oracle(dtype, symmetric, per_row, rows, inner):
    rng = np.random.default_rng(rows * 31 + inner)
    x = torch.from_numpy((rng.standard_normal((rows, inner)) * rng.uniform(0.1, 8, (rows, 1))).astype(np.float32)).to(dtype)
    if rows > 1:
        x[1] = 0  # an all-zero row
    want_y, want_s, want_zp = R.dynamic_quantize_linear(x.float().numpy(), symmetric, per_row, NAME[dtype])
    y, s, zp = ops.dynamic_quantize_linear(x.cuda(), symmetric, per_row)
    assert np.array_equal(y.cpu().numpy(), want_y)
    assert np.array_equal(s.float().cpu().numpy(), want_s)
    assert np.array_equal(zp.cpu().numpy(), want_zp)


@pytest.mark.parametrize("name", ["quantized_matmul_64x64x64", "quantized_matmul_128x128x128", "quantized_matmul_256x128x128",
                                  "quantized_matmul_128x256x64", "quantized_matmul_1x128x128"])
@pytest.mark.parametrize("workspace", ["auto", None])
def test_quantized_matmul_goldens(single_op, name, workspace):
    fx = single_op(name)
    lhs, ls, rhs, rs = fx.inputs
    out = ops.quantized_matmul(torch.from_numpy(lhs).cuda(), bf16_dev(ls), torch.from_numpy(rhs).cuda(), bf16_dev(rs),
                               workspace=workspace)
    want = R.bf16_bits_to_f32(fx.outputs[0])
    ok, md = eq_with_epsilon(out.float().cpu().numpy(), want, 1e-1)
    assert ok, md


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("m,n,k,per_row", [(1, 5632, 2048, True), (1, 2048, 5632, False), (7, 1008, 448, True), (32, 4096, 4096, True),
                                           (33, 384, 512, True), (256, 1024, 1024, True), (257, 640, 1040, False), (700, 256, 2048, True),
                                           (5, 100, 24, True), (3, 64, 72, True)])
def test_quantized_matmul_is_bit_equal_to_the_oracle(dtype, m, n, k, per_row):
    """Tile edges in every dimension (rows 257/700 over 256-row tiles, n 1008/640 over 128-row tiles, k 448/1040 over
    128-byte blocks) on the tensor-core kernel; k = 24 and 72 (not multiples of 16) take the plain kernel."""
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    lhs = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
    rhs = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    ls = torch.from_numpy(rng.uniform(0.005, 0.05, size=m if per_row else 1).astype(np.float32)).to(dtype)
    rs = torch.from_numpy(rng.uniform(0.002, 0.02, size=n).astype(np.float32)).to(dtype)
    ls_arg = ls if per_row else ls.reshape(())
    out = ops.quantized_matmul(torch.from_numpy(lhs).cuda(), ls_arg.cuda(), torch.from_numpy(rhs).cuda(), rs.cuda())
    ops.check_workspace(ops.dequant_matmul_workspace(1, n, k, "cuda"))
    want = R.store_round(R.quantized_matmul(lhs, ls.float().numpy() if per_row else float(ls.float()[0]), rhs, rs.float().numpy()),
                         NAME[dtype])
    assert np.array_equal(out.float().cpu().numpy(), want)
    plain = ops.quantized_matmul(torch.from_numpy(lhs).cuda(), ls_arg.cuda(), torch.from_numpy(rhs).cuda(), rs.cuda(), workspace=None)
    assert torch.equal(plain, out)


def test_w8a8_linear_close_to_the_float_product():
    """Quantize activations per row, multiply by int8 weights: the result tracks the float product within the int8
    quantisation error (a sanity check of the two operators used together, as quantize_activations wires them)."""
    rng = np.random.default_rng(3)
    x = torch.from_numpy(rng.standard_normal((64, 2048)).astype(np.float32)).bfloat16().cuda()
    wq = torch.from_numpy(rng.integers(-127, 128, size=(512, 2048), dtype=np.int8)).cuda()
    ws = torch.from_numpy(rng.uniform(0.002, 0.02, 512).astype(np.float32)).bfloat16().cuda()
    y, s, _ = ops.dynamic_quantize_linear(x, True, True)
    out = ops.quantized_matmul(y, s, wq, ws).float()
    ref = x.float() @ (wq.float() * ws.float()[:, None]).T
    assert float((out - ref).abs().max() / ref.abs().max()) < 3e-2
