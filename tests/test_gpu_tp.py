"""Tensor-parallel decode on 2, 4 and 8 GPUs (each case is skipped when the box has fewer): every rank's logits / greedy ids
against the CPU ORACLE of the unsharded model, with the per-layer reduction done either by the fused peer-memory operators
(the row-parallel product stores its partial sums into every rank's memory, each rank reduces + adds + norms) or by
ncclAllReduce inside the captured step.  Ranks are child processes with NVLS off; failures are made on the host (a rank
that leaves a delivery out), no GPU fault is provoked, and every device-side wait is bounded."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from oracle import ref_ops as R
from oracle.ref_model import LlamaConfig, OracleLlama

pytestmark = pytest.mark.gpu

# 16 query / 8 kv heads: shards down to one kv head per rank at 8 ranks
MID8 = dict(hidden_size=512, num_hidden_layers=3, num_attention_heads=16, num_key_value_heads=8, head_dim=64,
            intermediate_size=1408, vocab_size=2048, rms_norm_eps=1e-5, rope_theta=10000.0)
LLAMA3_SLICE = dict(hidden_size=4096, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                    intermediate_size=14336, vocab_size=4096, rms_norm_eps=1e-5, rope_theta=500000.0)
CASES = {"mid": (MID8, 4, 8, 6, 3), "llama3_slice": (LLAMA3_SLICE, 32, 16, 3, 5)}  # cfg, batch, prompt, decode steps, seed


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(case):
    cfg, batch, prompt_len, steps, seed = CASES[case]
    rng = np.random.default_rng(seed)
    prompt = rng.integers(0, cfg["vocab_size"], size=(batch, prompt_len))
    toks = [rng.integers(0, cfg["vocab_size"], size=batch) for _ in range(steps)]
    return prompt, toks


def _rank_main(rank, world, port, q, case, modes):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from my_nn_engine_b200 import collective
    from my_nn_engine_b200.decoder import DecoderModel
    from my_nn_engine_b200.quantize import random_llama_state
    comm = collective.set_communicator(rank, world)
    # the communicator itself: f32 sum of unequal vectors, in place
    t = torch.full((1000,), float(rank + 1), device="cuda")
    comm.all_reduce(t)
    comm.barrier()
    assert t.cpu().tolist() == [world * (world + 1) / 2.0] * 1000
    cfg, batch, prompt_len, steps, seed = CASES[case]
    state = random_llama_state(cfg, seed=seed, device="cuda")
    prompt, toks = _inputs(case)
    outs = {}
    for mode in modes:
        output, fused = mode.split("_")[0], not mode.endswith("nccl")
        m = DecoderModel(cfg, state, batch=batch, max_seq_len=prompt_len + steps + 2, tp_rank=rank, tp_world=world, output=output,
                         max_prefill=prompt_len, tp_fused=fused)
        assert m.tp_fused == fused
        res = [m.prefill(prompt, 0).clone()]
        for step in range(steps):
            res.append(m.step(toks[step], prompt_len + step).clone())
        outs[mode] = torch.stack([r.float() for r in res]).numpy()
        m.close()
    q.put((rank, outs))
    collective.destroy_communicator()
    dist.destroy_process_group()


def _oracle_run(case):
    from my_nn_engine_b200.quantize import random_llama_state
    cfg, batch, prompt_len, steps, seed = CASES[case]
    state = random_llama_state(cfg, seed=seed, device="cuda")
    w = {}
    for k, v in state.items():
        if v.dtype == torch.int8:
            w[k] = v.cpu().numpy()
        elif k.endswith(".scale"):
            w[k] = R.round_bf16(v.float().cpu().numpy())
        else:
            w[k] = v.float().cpu().numpy()
    del state
    torch.cuda.empty_cache()
    oracle = OracleLlama(LlamaConfig.from_hf(cfg), w, "bf16", prompt_len + steps + 2, batch, c_attention=True)
    prompt, toks = _inputs(case)
    oracle.prefill(prompt, prompt_len)
    logits = [oracle.last_logits.copy()]
    for step in range(steps):
        oracle.decode_step(toks[step])
        logits.append(oracle.last_logits.copy())
    return np.stack(logits)


def _collect(q, procs, world, timeout=600.0):
    """One result per rank from the queue; gives up at once (instead of waiting out the timeout) when a rank has died."""
    import queue
    import time
    got, t0 = [], time.time()
    while len(got) < world:
        try:
            got.append(q.get(timeout=2.0))
            continue
        except queue.Empty:
            pass
        dead = [(i, p.exitcode) for i, p in enumerate(procs) if p.exitcode not in (None, 0)]
        assert not dead, f"rank processes died (rank, exit code): {dead}"
        assert time.time() - t0 < timeout, f"only {len(got)} of {world} ranks answered within {timeout:.0f} s"
    return got


def _spawn(world, target, args):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, q) + args, daemon=True) for r in range(world)]  # never outlive the test run
    for p in procs:
        p.start()
    return q, procs


@pytest.mark.parametrize("case", ["mid", "llama3_slice"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_matches_the_oracle(world, case):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    modes = ("logits", "ids", "logits_nccl") if case == "mid" else ("logits", "ids")
    q, procs = _spawn(world, _rank_main, (case, modes))
    want = _oracle_run(case)  # the unsharded model on the CPU, while the ranks run
    got = dict(_collect(q, procs, world))
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    scale = np.abs(want).max()
    for rank in range(world):
        for key in modes:
            if key == "ids":
                continue
            lg = got[rank][key]
            assert np.abs(lg - want).max() <= 3e-2 * scale, (rank, key, float(np.abs(lg - want).max() / scale))
        assert np.array_equal(got[rank]["logits"], got[0]["logits"])  # every rank holds the identical result
        assert np.array_equal(got[rank]["ids"], got[0]["ids"])
    ids_ref = np.array([[len(r) - 1 - np.argmax(r[::-1]) for r in step] for step in got[0]["logits"]])
    assert np.array_equal(got[0]["ids"].astype(np.int64), ids_ref)  # sharded argmax == argmax of the gathered logits
    # greedy picks against the oracle: equal unless the oracle's own top two are closer than 4 bf16 steps
    flips = 0
    for step in range(want.shape[0]):
        for b in range(want.shape[1]):
            w_, g_ = R.argmax_last(want[step, b]), int(ids_ref[step, b])
            if w_ != g_:
                assert want[step, b, w_] - want[step, b, g_] <= 4 * 2.0 ** -7 * abs(want[step, b, w_]), (step, b)
                flips += 1
    print(f"tp{world} {case}: {flips} near-tie flips in {want.shape[0] * want.shape[1]} greedy picks")


def _stall_rank_main(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from my_nn_engine_b200 import collective, ffi
    from my_nn_engine_b200.decoder import DecoderModel
    from my_nn_engine_b200.quantize import random_llama_state
    collective.set_communicator(rank, world)
    state = random_llama_state(MID8, seed=3, device="cuda")
    m = DecoderModel(MID8, state, batch=4, max_seq_len=16, tp_rank=rank, tp_world=world, output="ids", use_graph=False)
    tok = np.arange(4)
    m.step(tok, 0)  # a clean step first
    ffi.set_option(ffi.OPT_WAIT_BUDGET_US, 50000)
    if rank == 1:
        ffi.set_option(ffi.OPT_INJECT_STALL, 2)  # this rank's next row-parallel product delivers nothing
    code = 0
    try:
        m.step(tok, 1)
    except ffi.MynnError as e:
        code = e.code
    again = m.step(tok, 1).clone()  # the ranks are in step again: this one succeeds (and overwrites the broken row)
    q.put((rank, code, again.tolist()))
    dist.barrier()  # leave together, with nothing in flight
    m.close()
    collective.destroy_communicator()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_a_rank_that_delivers_nothing_is_reported_not_waited_for():
    """Rank 1 leaves the deliveries of one row-parallel product out (host-side switch).  Every rank's reduction waits 50 ms for
    the missing partial sums, records its status and carries on; the step returns MYNN_E_COMM on the host; the following step
    is clean again on both ranks (every reduction leaves the slots it read empty again); both ranks exit cleanly."""
    from my_nn_engine_b200 import ffi
    q, procs = _spawn(2, _stall_rank_main, ())
    got = {r: (c, ids) for r, c, ids in _collect(q, procs, 2, timeout=300.0)}
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert got[0][0] == ffi.E_COMM and got[1][0] == ffi.E_COMM
    assert got[0][1] == got[1][1]
