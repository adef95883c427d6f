"""The bounded device-side waits, made to run out in the allowed way: a wait for something that never arrives, with a short
time limit, after which the kernel records a status code and returns.  Nothing faults, traps or hangs, the CUDA context stays
usable and the next normal call succeeds."""
import numpy as np
import pytest
import torch

from oracle import ref_ops as R

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,k", [(256, 1024), (4096, 4096)])
def test_dequant_matmul_wait_runs_out_and_the_next_call_is_clean(n, k):
    """MYNN_OPT_INJECT_STALL = 1 makes the TMA producer of ONE tcgen05 DequantMatMul launch leave out its last stage: the MMA
    thread's wait for that stage expires after the (shortened) budget, status 2 lands in the workspace,
    mynn_b200_dequant_matmul_check reports MYNN_E_CUDA once, and the following call gives the oracle's result.  The second
    shape splits K over a cluster, so every CTA of a cluster also has to reach the cluster barriers after giving up."""
    from my_nn_engine_b200 import ffi, ops
    rng = np.random.default_rng(n + k)
    wq = torch.from_numpy(rng.integers(-127, 128, size=(n, k), dtype=np.int8)).cuda()
    scale = torch.from_numpy(rng.uniform(0.002, 0.02, n).astype(np.float32)).bfloat16().cuda()
    act = torch.from_numpy(rng.standard_normal((8, k)).astype(np.float32)).bfloat16().cuda()
    want = R.dequant_matmul(act.float().cpu().numpy(), wq.cpu().numpy(), scale.float().cpu().numpy())
    ws = ops.dequant_matmul_workspace(8, n, k, "cuda")
    ffi.set_option(ffi.OPT_WAIT_BUDGET_US, 20000)
    try:
        ffi.set_option(ffi.OPT_INJECT_STALL, 1)
        ops.dequant_matmul(act, wq, scale, workspace=ws)
        with pytest.raises(ffi.MynnError) as err:
            ops.check_workspace(ws)
        assert err.value.code == ffi.E_CUDA and "timed out" in str(err.value)
        ops.check_workspace(ws)  # reported once, then cleared
        out = ops.dequant_matmul(act, wq, scale, workspace=ws)
        ops.check_workspace(ws)
        assert np.abs(out.float().cpu().numpy() - want).max() <= 1e-2 * np.abs(want).max()
    finally:
        ffi.set_option(ffi.OPT_INJECT_STALL, 0)
        ffi.set_option(ffi.OPT_WAIT_BUDGET_US, 2000000)
