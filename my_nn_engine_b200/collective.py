"""Process-global tensor-parallel communicator: the engine's ``collective::set_communicator`` /
``trait Communicator { rank, world_size, all_reduce, barrier }`` (src/collective.rs:1-20,
crates/comm/src/lib.rs:32-38) over NCCL on NVLink/NVSwitch, one process per GPU.

``torch.distributed`` is used only to hand the 128-byte NCCL unique id from rank 0 to the other ranks (any
process group works, including gloo); the collectives themselves are issued by the library on the caller's stream.
Environment variables follow the engine's (crates/comm/src/uds.rs:41-47): MYNN_RANK / MYNN_WORLD_SIZE override
RANK / WORLD_SIZE.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import ffi

_DT = {torch.float32: ffi.F32, torch.bfloat16: ffi.BF16, torch.float16: ffi.F16}


class Communicator:
    def __init__(self, rank: int, world_size: int):
        self._rank, self._world = rank, world_size

    def rank(self) -> int:
        return self._rank

    def world_size(self) -> int:
        return self._world

    def all_reduce(self, dst: torch.Tensor, src: torch.Tensor | None = None) -> torch.Tensor:
        """Sum over ranks, in place when ``src`` is None.  f32, bf16 or f16 CUDA tensors of equal length on every
        rank (a length mismatch is a protocol error in the engine; NCCL requires equal counts)."""
        src = dst if src is None else src
        if dst.numel() != src.numel() or dst.dtype != src.dtype:
            raise ValueError("all_reduce: dst and src differ in length or dtype")
        if not (dst.is_cuda and src.is_cuda and dst.is_contiguous() and src.is_contiguous()):
            raise ValueError("all_reduce needs contiguous CUDA tensors")
        ffi.check(ffi.lib().mynn_b200_all_reduce(torch.cuda.current_stream().cuda_stream, dst.data_ptr(), src.data_ptr(),
                                                 dst.numel(), _DT[dst.dtype]))
        return dst

    def barrier(self) -> None:
        ffi.check(ffi.lib().mynn_b200_comm_barrier(torch.cuda.current_stream().cuda_stream))


_COMM: Communicator | None = None


def env_rank_world():
    rank = int(os.environ.get("MYNN_RANK", os.environ.get("RANK", "0")))
    world = int(os.environ.get("MYNN_WORLD_SIZE", os.environ.get("WORLD_SIZE", "1")))
    return rank, world


def exchange_unique_id(rank: int, world: int, make_id, group=None) -> bytes:
    """Rank 0 creates the id with ``make_id()``; every rank returns the same 128 bytes (host-side broadcast)."""
    import torch.distributed as dist
    payload = [make_id() if rank == 0 else None]
    if world > 1:
        dist.broadcast_object_list(payload, src=0, group=group)
    return payload[0]


def set_communicator(rank: int | None = None, world_size: int | None = None, group=None) -> Communicator:
    """Create the process-global communicator (once).  With world_size > 1 a torch.distributed process group must
    already exist for the id exchange."""
    global _COMM
    if _COMM is not None:
        raise RuntimeError("communicator already set")
    if rank is None or world_size is None:
        rank, world_size = env_rank_world()
    lib = ffi.lib()
    if world_size == 1:
        ffi.check(lib.mynn_b200_comm_init(None, 0, 1))
    else:
        def make_id():
            buf = ctypes.create_string_buffer(128)
            ffi.check(lib.mynn_b200_comm_unique_id(buf))
            return buf.raw
        uid = exchange_unique_id(rank, world_size, make_id, group)
        if len(uid) != 128:
            raise RuntimeError("unique id must be 128 bytes")
        ffi.check(lib.mynn_b200_comm_init(ctypes.create_string_buffer(uid, 128), rank, world_size))
    _COMM = Communicator(rank, world_size)
    return _COMM


def communicator() -> Communicator:
    if _COMM is None:
        raise RuntimeError("communicator not set: call set_communicator first")
    return _COMM


def destroy_communicator() -> None:
    global _COMM
    ffi.lib().mynn_b200_comm_destroy()
    _COMM = None
