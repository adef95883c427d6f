"""Tensor-parallel decode on 2 GPUs (skipped with fewer): every rank's logits / greedy ids equal the single-GPU model's
to the end-to-end tolerance, with the per-layer reduction done either by reading the peers' partial sums over NVLink
inside the residual-add + RMSNorm kernel or by ncclAllReduce inside the captured step.  Ranks are child processes; failures
are host-side (a rank exits with a non-zero code), no GPU fault is provoked."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

MID = dict(hidden_size=512, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
           intermediate_size=1408, vocab_size=2048, rms_norm_eps=1e-5, rope_theta=10000.0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
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
    assert t.cpu().tolist() == [3.0] * 1000
    state = random_llama_state(MID, seed=3)
    outs = {}
    for output, fused in (("logits", True), ("ids", True), ("logits_nccl", False)):
        m = DecoderModel(MID, state, batch=4, max_seq_len=48, tp_rank=rank, tp_world=world, output=output.split("_")[0],
                         max_prefill=8, tp_fused=fused)
        assert m.tp_fused == fused
        rng = np.random.default_rng(0)
        prompt = rng.integers(0, 2048, size=(4, 8))
        res = [m.prefill(prompt, 0).clone()]
        tok = rng.integers(0, 2048, size=4)
        for step in range(6):
            res.append(m.step(tok, 8 + step).clone())
            tok = rng.integers(0, 2048, size=4)
        outs[output] = torch.stack([r.float() for r in res]).numpy()
        m.close()
    q.put((rank, outs))
    collective.destroy_communicator()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_matches_single_gpu():
    from my_nn_engine_b200.decoder import DecoderModel
    from my_nn_engine_b200.quantize import random_llama_state
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    # single-GPU reference run of the same steps
    state = random_llama_state(MID, seed=3)
    m = DecoderModel(MID, state, batch=4, max_seq_len=48, output="logits", max_prefill=8)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, 2048, size=(4, 8))
    ref = [m.prefill(prompt, 0).float().clone()]
    tok = rng.integers(0, 2048, size=4)
    for step in range(6):
        ref.append(m.step(tok, 8 + step).float().clone())
        tok = rng.integers(0, 2048, size=4)
    ref = torch.stack(ref).numpy()
    m.close()
    for rank in (0, 1):
        for key in ("logits", "logits_nccl"):  # peer-memory reduction fused into the norm kernel, and ncclAllReduce
            lg = got[rank][key]
            assert np.abs(lg - ref).max() <= 3e-2 * np.abs(ref).max(), key
        assert np.array_equal(got[rank]["logits"], got[0]["logits"])  # every rank computes the identical sum
        assert np.array_equal(got[rank]["ids"], got[0]["ids"])
    ids_ref = np.array([[len(r) - 1 - np.argmax(r[::-1]) for r in step] for step in got[0]["logits"]])
    assert np.array_equal(got[0]["ids"].astype(np.int64), ids_ref)  # sharded argmax == argmax of gathered logits
