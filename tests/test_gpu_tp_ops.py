"""The fused tensor-parallel operators (row-parallel DequantMatMul that pushes its partial sums -> reduce + add + RMSNorm ->
the next DequantMatMul) on ONE GPU: all ranks of a group live in this process and their calls are issued in lock step (every
push before any reduce), so every cross-rank wait is already satisfied when its kernel starts and no kernel ever waits for
one that has not run.  The results are compared with the CPU oracle of the unsharded operators.  The bounded wait is also
made to run out, by leaving a rank's product out, with a 20 ms budget."""
import numpy as np
import pytest
import torch

from oracle import ref_ops as R

pytestmark = pytest.mark.gpu


def make_groups(world, max_rows, hidden):
    from my_nn_engine_b200 import ops
    nbytes = ops.tp_block_bytes(max_rows, hidden, world)
    assert nbytes > 0
    blocks = [torch.empty(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    for b in blocks:
        ops.tp_block_init(b, max_rows, hidden, world)
    return [ops.TpGroup(blocks, r, max_rows, hidden) for r in range(world)]


def oracle_reduction(act, w_row, s_row, x, w_norm, world, eps):
    """Partial products of the K shards summed in rank order (f32), rounded, added to x, normed: the engine's tensor-parallel
    sequence DequantMatMul -> AllReduce -> Add -> RMSNorm with one bf16 store per operator."""
    k = act.shape[1] // world
    total = np.zeros((act.shape[0], w_row.shape[0]), np.float32)
    for r in range(world):
        total = total + R.dequant_matmul(act[:, r * k:(r + 1) * k], w_row[:, r * k:(r + 1) * k], s_row).astype(np.float32)
    x_new = R.round_bf16(x + R.round_bf16(total))
    return x_new, R.round_bf16(R.rms_norm(x_new, w_norm, eps))


@pytest.mark.parametrize("world,m,hidden,k_total,n_out", [(2, 32, 512, 1024, 384), (4, 32, 512, 2048, 256), (8, 32, 4096, 4096, 256),
                                                          (8, 5, 512, 1024, 128), (4, 1, 256, 512, 128), (2, 7, 4096, 14336, 512)])
def test_lock_step_ranks_match_the_unsharded_oracle(world, m, hidden, k_total, n_out):
    from my_nn_engine_b200 import ops
    rng = np.random.default_rng(world * 1000 + m + hidden)
    groups = make_groups(world, 32, hidden)
    eps = 1e-5
    x0 = R.round_bf16(rng.standard_normal((m, hidden)).astype(np.float32))
    xs = [torch.from_numpy(x0).bfloat16().cuda() for _ in range(world)]  # every rank's copy of the residual stream
    x_ref = x0
    ksh = k_total // world
    for it in range(3):  # three reductions on alternating buffers: every slot is emptied by the reduction that read it
        buf = it & 1
        w_row = rng.integers(-127, 128, size=(hidden, k_total), dtype=np.int8)
        s_row = rng.uniform(0.0002, 0.002, hidden).astype(np.float32)
        act = R.round_bf16(rng.standard_normal((m, k_total)).astype(np.float32))
        w_norm = R.round_bf16(rng.uniform(0.5, 1.5, hidden).astype(np.float32))
        w_col = rng.integers(-127, 128, size=(n_out, hidden), dtype=np.int8)
        s_col = R.round_bf16(rng.uniform(0.002, 0.02, n_out).astype(np.float32))
        wr_dev = [torch.from_numpy(np.ascontiguousarray(w_row[:, r * ksh:(r + 1) * ksh])).cuda() for r in range(world)]
        act_dev = [torch.from_numpy(np.ascontiguousarray(act[:, r * ksh:(r + 1) * ksh])).bfloat16().cuda() for r in range(world)]
        s_dev = torch.from_numpy(s_row).cuda()
        wn_dev = torch.from_numpy(w_norm).bfloat16().cuda()
        wc_dev, sc_dev = torch.from_numpy(w_col).cuda(), torch.from_numpy(s_col).bfloat16().cuda()
        wss = [torch.zeros(1 << 20, dtype=torch.uint8, device="cuda") for _ in range(world)]  # each rank's GEMM workspace
        for r in range(world):
            ops.tp_dequant_matmul_push(groups[r], buf, act_dev[r], wr_dev[r], s_dev, workspace=wss[r])
        outs = []
        for r in range(world):
            ops.tp_reduce_norm(groups[r], buf, xs[r], wn_dev, eps, wss[r])
            outs.append(ops.dequant_matmul_same_act(xs[r], wc_dev, sc_dev, workspace=wss[r]))
        for r in range(world):
            ops.tp_check(groups[r])
        x_ref, y_ref = oracle_reduction(act, w_row, s_row, x_ref, w_norm, world, eps)
        want = R.dequant_matmul(y_ref, w_col, s_col)
        ulp = 2.0 ** -7
        for r in range(world):
            got_x = xs[r].float().cpu().numpy()
            assert np.abs(got_x - x_ref).max() <= 2 * ulp * np.abs(x_ref).max(), (it, r)
            got = outs[r].float().cpu().numpy()
            assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max(), (it, r)
            assert torch.equal(outs[r], outs[0]) and torch.equal(xs[r], xs[0])  # every rank computes identical rows
        x_ref = xs[0].float().cpu().numpy()  # carry the device's own residual rows forward, as the oracle carries x_ref


def _small_problem(rng, hidden=256, k_total=512, m=8):
    w_row = torch.from_numpy(rng.integers(-127, 128, size=(hidden, k_total // 2), dtype=np.int8)).cuda()
    s_row = torch.from_numpy(rng.uniform(0.0002, 0.002, hidden).astype(np.float32)).cuda()
    act = torch.from_numpy(rng.standard_normal((m, k_total // 2)).astype(np.float32)).bfloat16().cuda()
    x = torch.from_numpy(rng.standard_normal((m, hidden)).astype(np.float32)).bfloat16().cuda()
    w_norm = torch.ones(hidden, dtype=torch.bfloat16, device="cuda")
    w_col = torch.from_numpy(rng.integers(-127, 128, size=(128, hidden), dtype=np.int8)).cuda()
    s_col = torch.full((128,), 0.01, dtype=torch.bfloat16, device="cuda")
    return w_row, s_row, act, x, w_norm, w_col, s_col


def test_wait_for_partial_sums_runs_out_when_a_rank_never_delivers():
    """Two ranks; only rank 0 runs its product.  Rank 0's reduction waits 20 ms for rank 1's partial sums, records status 21,
    finishes and returns; tp_check reports MYNN_E_COMM once.  The reduction leaves every slot it read empty again, so after a
    rank that delivered NOTHING the same group works again at the next reduction, and so does a product whose deliveries were
    switched off by MYNN_OPT_INJECT_STALL = 2."""
    from my_nn_engine_b200 import ffi, ops
    rng = np.random.default_rng(1)
    w_row, s_row, act, x, w_norm, w_col, s_col = _small_problem(rng)
    groups = make_groups(2, 32, 256)
    wss = [torch.zeros(1 << 18, dtype=torch.uint8, device="cuda") for _ in range(2)]
    ffi.set_option(ffi.OPT_WAIT_BUDGET_US, 20000)
    try:
        ops.tp_dequant_matmul_push(groups[0], 0, act, w_row, s_row, workspace=wss[0])
        ops.tp_reduce_norm(groups[0], 0, x.clone(), w_norm, 1e-5, wss[0])
        with pytest.raises(ffi.MynnError) as err:
            ops.tp_check(groups[0])
        assert err.value.code == ffi.E_COMM and "21" in str(err.value)
        ops.tp_check(groups[0])  # reported once
        # rank 1 catches up with the reduction it missed (nobody delivers to it: it times out as well)
        ops.tp_reduce_norm(groups[1], 0, x.clone(), w_norm, 1e-5, wss[1])
        with pytest.raises(ffi.MynnError):
            ops.tp_check(groups[1])
        # next reduction, on the other buffer, with rank 1's deliveries switched off: both time out
        ops.tp_dequant_matmul_push(groups[0], 1, act, w_row, s_row, workspace=wss[0])
        ffi.set_option(ffi.OPT_INJECT_STALL, 2)
        ops.tp_dequant_matmul_push(groups[1], 1, act, w_row, s_row, workspace=wss[1])
        for r in range(2):
            ops.tp_reduce_norm(groups[r], 1, x.clone(), w_norm, 1e-5, wss[r])
            with pytest.raises(ffi.MynnError):
                ops.tp_check(groups[r])
    finally:
        ffi.set_option(ffi.OPT_INJECT_STALL, 0)
        ffi.set_option(ffi.OPT_WAIT_BUDGET_US, 2000000)
    # the same group, in step again: a complete reduction on buffer 0
    for r in range(2):
        ops.tp_dequant_matmul_push(groups[r], 0, act, w_row, s_row, workspace=wss[r])
    xs, outs = [x.clone(), x.clone()], []
    for r in range(2):
        ops.tp_reduce_norm(groups[r], 0, xs[r], w_norm, 1e-5, wss[r])
        outs.append(ops.dequant_matmul_same_act(xs[r], w_col, s_col, workspace=wss[r]))
        ops.tp_check(groups[r])
    assert torch.equal(outs[0], outs[1]) and torch.isfinite(outs[0].float()).all()
    part = R.dequant_matmul(act.float().cpu().numpy(), w_row.cpu().numpy(), s_row.cpu().numpy())
    want_x = R.round_bf16(x.float().cpu().numpy() + R.round_bf16(part + part))
    assert np.abs(xs[0].float().cpu().numpy() - want_x).max() <= 2.0 ** -6 * np.abs(want_x).max()
