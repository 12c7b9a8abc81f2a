"""Tensor-parallel bootstrap: one process per GPU, `torch.distributed` for the plumbing only.

The data path is the library's own peer-memory exchange kernel (op codes 71 / 72); this
module just moves the 64-byte CUDA IPC handles of the ranks' exchange buffers between the
processes and keeps the ranks in step around set-up, timing and tear-down.
"""
from __future__ import annotations

import ctypes
import os
from typing import List

from . import _lib


def init_process_group():
    """Join the torchrun rendezvous (RANK / WORLD_SIZE / MASTER_* from the environment)."""
    import torch.distributed as dist
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend="gloo")
    return dist.get_rank(), dist.get_world_size()


def all_gather_bytes(blob: bytes) -> List[bytes]:
    """Every rank's blob (equal lengths), in rank order."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size()
    mine = torch.tensor(list(blob), dtype=torch.uint8)
    out = [torch.zeros(len(blob), dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(out, mine)
    return [bytes(t.tolist()) for t in out]


def max_over_ranks(value: float) -> float:
    import torch
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def barrier() -> None:
    import torch.distributed as dist
    dist.barrier()


def connect(rank: int, world: int, slot_floats: int, large_message_floats: int = 0) -> None:
    """Create this rank's exchange buffer, swap IPC handles, map the peers.  `large_message_floats` (the same on
    every rank; 0 = the library's default) is the message size above which an exchange takes the chunk-sized grid."""
    lib = _lib.load()
    _lib.check(lib.deepj_cuda_tp_configure(int(large_message_floats)))
    slot_floats = (int(slot_floats) + 3) // 4 * 4
    handle = ctypes.create_string_buffer(64)
    _lib.check(lib.deepj_cuda_tp_create(rank, world, slot_floats, handle))
    handles = all_gather_bytes(handle.raw)
    blob = b"".join(handles)
    _lib.check(lib.deepj_cuda_tp_connect(blob, world))
    barrier()


def disconnect() -> None:
    barrier()
    _lib.check(_lib.load().deepj_cuda_tp_destroy())
