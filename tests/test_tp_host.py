"""Tensor-parallel host logic on CPU: the sharding arithmetic (sharded == unsharded on the oracle) and the
unique-id exchange over a 2-rank gloo group."""
import os
import socket

import numpy as np
import torch
import torch.multiprocessing as mp

from my_nn_engine_b200.decoder import _shard_cols, _shard_heads, _shard_rows
from oracle import ref_ops as R


def test_column_parallel_shards_are_exact_slices():
    rng = np.random.default_rng(0)
    w = torch.from_numpy(rng.integers(-127, 128, size=(64, 32), dtype=np.int8))
    s = torch.from_numpy(rng.uniform(0.002, 0.02, 64).astype(np.float32))
    x = rng.standard_normal((3, 32)).astype(np.float32)
    full = R.dequant_matmul_variant_a(x, w.numpy(), s.numpy())
    for world in (2, 4, 8):
        parts = [R.dequant_matmul_variant_a(x, _shard_heads(w, 8, r, world).numpy(), _shard_heads(s, 8, r, world).numpy())
                 for r in range(world)]
        assert np.array_equal(np.concatenate(parts, axis=1), full)  # whole heads, bit-exact
        parts = [R.dequant_matmul_variant_a(x, _shard_rows(w, r, world).numpy(), _shard_rows(s, r, world).numpy())
                 for r in range(world)]
        assert np.array_equal(np.concatenate(parts, axis=1), full)


def test_row_parallel_partials_sum_to_the_full_product():
    rng = np.random.default_rng(1)
    w = torch.from_numpy(rng.integers(-127, 128, size=(48, 256), dtype=np.int8))
    s = rng.uniform(0.002, 0.02, 48).astype(np.float32)
    x = rng.standard_normal((2, 256)).astype(np.float32)
    full = R.dequant_matmul_variant_a(x, w.numpy(), s)
    for world in (2, 4, 8):
        k = 256 // world
        partial = [R.dequant_matmul_variant_a(x[:, r * k:(r + 1) * k], _shard_cols(w, r, world).numpy(), s) for r in range(world)]
        total = np.sum(np.stack(partial), axis=0, dtype=np.float32)  # rank-ordered f32 sum, as the all-reduce does
        assert np.abs(total - full).max() <= 1e-5 * np.abs(full).max()


def test_sharded_argmax_keeps_last_maximum():
    logits = np.array([1.0, 9.0, 3.0, 9.0, 2.0, 9.0, 0.0, 1.0], dtype=np.float32)
    for world in (2, 4):
        n = len(logits) // world
        pairs = []
        for r in range(world):
            shard = logits[r * n:(r + 1) * n]
            pairs.append((shard.max(), r * n + R.argmax_last(shard)))
        best = None
        for v, i in pairs:  # ascending shards, >= keeps the last
            if best is None or v >= best[0]:
                best = (v, i)
        assert best[1] == R.argmax_last(logits) == 5


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from my_nn_engine_b200.collective import env_rank_world, exchange_unique_id
    os.environ["MYNN_RANK"], os.environ["MYNN_WORLD_SIZE"] = str(rank), str(world)
    assert env_rank_world() == (rank, world)
    made = []

    def make_id():
        made.append(1)
        return bytes(range(128))

    uid = exchange_unique_id(rank, world, make_id)
    assert (len(made) == 1) == (rank == 0)
    # the all-reduce the ranks would then run on NVLink, restated on gloo: f32 sum of unequal partials
    t = torch.full((4,), float(rank + 1))
    dist.all_reduce(t)
    out.put((rank, uid, t.tolist()))
    dist.destroy_process_group()


def test_unique_id_exchange_two_ranks_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert res[0][1] == res[1][1] == bytes(range(128))
    assert res[0][2] == res[1][2] == [3.0] * 4
