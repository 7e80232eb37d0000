"""Sum of per-rank expert outputs: peer-memory all-reduce when the payload fits its arena (decode rows and
moderate prefill chunks), NCCL otherwise or after the peer path reported a timeout. With `multimem=True` (or
POCKET_MULTIMEM=1) and a machine that offers multicast, payloads from `multimem_min_floats` on go through the in-switch
all-reduce (`MultimemAllReduce`, two shot) instead: at eight ranks it moves each element over every link once, where
the unicast kernel stores it into seven peers.

A peer wait that runs out leaves a sticky status word on the rank that waited; later peer all-reduces of that rank
return without reducing, so the step's result is wrong on at least one rank. `check_step()` is therefore called by
the model runtimes once per forward, after the step's device synchronisation and before any token is returned: it
takes the MAX of the status words over the group, so every rank reaches the same verdict, and on a failure every
rank clears its word, drops the peer path (NCCL from then on) and raises `StepFailed`. Reference behaviour:
src/models/deepseek_v4/runtime.py:4191-4196 (custom all-reduce timeout -> NCCL)."""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


class StepFailed(TimeoutError):
    """The current step must be discarded: a peer all-reduce of some rank gave up waiting."""


class ExpertCombine:
    def __init__(self, world: int, group=None, capacity: int = 4 << 20, use_peer: bool = True, peer=None, multimem: bool | None = None,
                 multimem_min_floats: int | None = None, mm=None):
        """`peer` / `mm`: objects with `all_reduce`, `status(clear=False)` and `capacity` (tests inject them)."""
        self.world, self.group = world, group
        self.peer = peer
        self.mm = mm
        self.calls = {"peer": 0, "nccl": 0, "multimem": 0}
        self.fallbacks = 0
        if world > 1 and use_peer and peer is None:
            from .peer_allreduce import PeerAllReduce
            self.peer = PeerAllReduce(capacity, group)
        if multimem is None:
            multimem = os.environ.get("POCKET_MULTIMEM", "0") == "1"
        from .multimem_allreduce import TWO_SHOT_MIN_FLOATS
        self.mm_min = TWO_SHOT_MIN_FLOATS if multimem_min_floats is None else multimem_min_floats
        if world > 1 and use_peer and multimem and mm is None:
            from .multimem_allreduce import MulticastUnavailable, MultimemAllReduce
            try:
                self.mm = MultimemAllReduce(capacity, group)
            except (MulticastUnavailable, RuntimeError):     # collective probe: every rank takes the same branch
                self.mm = None

    def __call__(self, y: torch.Tensor) -> torch.Tensor:
        """In-place sum of contiguous fp32 `y` over the ranks."""
        if self.world == 1:
            return y
        if (self.mm is not None and self.mm_min <= y.numel() <= self.mm.capacity and y.dtype == torch.float32 and y.is_contiguous()):
            self.calls["multimem"] += 1
            return self.mm.all_reduce(y, two_shot=True)
        if self.peer is not None and y.numel() <= self.peer.capacity and y.dtype == torch.float32 and y.is_contiguous():
            self.calls["peer"] += 1
            return self.peer.all_reduce(y)
        self.calls["nccl"] += 1
        dist.all_reduce(y, group=self.group)
        return y

    def check_step(self, device: torch.device | str | None = None) -> None:
        """Collective over the group (every rank calls it once per forward, also ranks whose own word is clean).
        Raises `StepFailed` on every rank when any rank's peer wait ran out; the peer path is off afterwards."""
        if self.world == 1 or (self.peer is None and self.mm is None):
            return
        local = max(int(self.peer.status()) if self.peer is not None else 0, int(self.mm.status()) if self.mm is not None else 0)
        if device is None:
            device = "cuda" if dist.get_backend(self.group) == "nccl" else "cpu"
        word = torch.tensor([local], dtype=torch.int32, device=device)
        dist.all_reduce(word, op=dist.ReduceOp.MAX, group=self.group)
        worst = int(word.item())
        if worst == 0:
            return
        for path in (self.peer, self.mm):
            if path is not None:
                path.status(clear=True)
        self.peer = self.mm = None
        self.fallbacks += 1
        raise StepFailed(f"a peer all-reduce gave up waiting (status {worst}, this rank {local}): the step is discarded "
                         "and the following steps use NCCL")

    # kept for callers of the earlier, rank-local API
    def check(self) -> None:
        self.check_step()
