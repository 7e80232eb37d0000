"""Sum of per-rank expert outputs: peer-memory all-reduce when the payload fits its arena (decode rows and
moderate prefill chunks), NCCL otherwise or when the peer path reported a timeout."""
from __future__ import annotations

import torch
import torch.distributed as dist

from .peer_allreduce import PeerAllReduce


class ExpertCombine:
    def __init__(self, world: int, group=None, capacity: int = 4 << 20, use_peer: bool = True):
        self.world, self.group = world, group
        self.peer: PeerAllReduce | None = None
        self.calls = {"peer": 0, "nccl": 0}
        if world > 1 and use_peer:
            self.peer = PeerAllReduce(capacity, group)

    def __call__(self, y: torch.Tensor) -> torch.Tensor:
        """In-place sum of contiguous fp32 `y` over the ranks."""
        if self.world == 1:
            return y
        if self.peer is not None and y.numel() <= self.peer.capacity and y.dtype == torch.float32 and y.is_contiguous():
            self.calls["peer"] += 1
            return self.peer.all_reduce(y)
        self.calls["nccl"] += 1
        dist.all_reduce(y, group=self.group)
        return y

    def check(self) -> None:
        """Raise if a peer wait ran out since the last check; the peer path is switched off after that."""
        if self.peer is not None and self.peer.status() != 0:
            self.peer.status(clear=True)
            self.peer = None
            raise TimeoutError("peer all-reduce timed out; falling back to NCCL for the following steps")
