"""Tensor-parallel bring-up of the native engine.

Each rank creates its engine, exports the CUDA IPC handle of its comm arena (all-reduce
slots, flags, sampler candidates), the handles travel through `torch.distributed`
(`all_gather_object`, the equivalent of the reference's handle exchange for its CUDA-IPC
all-reduce, src/models/deepseek_v4/runtime.py:206-289), and every rank maps its peers'
arenas. After that no host-side collective is on the token path: the kernels push
partial sums into peer memory and poll flags with bounded waits.
"""
from __future__ import annotations

import os
from typing import Sequence

import torch
import torch.distributed as dist


def env_rank_world() -> tuple[int, int, int]:
    """(rank, world, local_rank) from the torchrun environment; (0, 1, 0) when absent."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0")))


def exchange_handles(handle: bytes, group: dist.ProcessGroup | None = None) -> list[bytes]:
    world = dist.get_world_size(group)
    out: list[bytes | None] = [None] * world
    dist.all_gather_object(out, handle, group=group)
    if any(h is None or len(h) != 64 for h in out):
        raise RuntimeError("peer handle exchange was truncated")
    return [bytes(h) for h in out]  # type: ignore[arg-type]


def connect_engine(engine, group: dist.ProcessGroup | None = None) -> None:
    """Register every rank's comm arena with `engine` (collective call)."""
    if engine.tp_world == 1:
        return
    handles = exchange_handles(engine.export_arena(), group)
    engine.connect(handles)
    torch.cuda.synchronize()
    dist.barrier(group=group)


def shard_range(total: int, rank: int, world: int, align: int = 1) -> tuple[int, int]:
    """Contiguous [start, end) of `total` owned by `rank`; the shard size must be a multiple of `align`."""
    if total % world != 0 or (total // world) % align != 0:
        raise ValueError(f"{total} does not split into {world} shards aligned to {align}")
    n = total // world
    return rank * n, (rank + 1) * n
