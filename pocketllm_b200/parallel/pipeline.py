"""Layer pipeline over `torch.distributed` point-to-point: each stage runs a contiguous layer
range, hands its activations to the next stage and the last stage broadcasts the sampled
token (the reference's layer-PP loop: src/models/deepseek_v4/runtime.py:4832-4838,4873).
On GPUs the transport is NCCL send/recv on a side stream; on CPU ranks it is gloo.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

from . import partition


class PipelineStage:
    def __init__(self, n_layers: int, *, group=None, side_stream: "torch.cuda.Stream | None" = None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.lo, self.hi = partition.layer_range(n_layers, self.world, self.rank)
        self.first, self.last = self.rank == 0, self.rank == self.world - 1
        self.side = side_stream

    def _p2p(self, fn, t: torch.Tensor, peer: int) -> None:
        if self.side is not None and t.is_cuda:
            self.side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.side):
                fn(t, peer, group=self.group)
            torch.cuda.current_stream().wait_stream(self.side)
        else:
            fn(t, peer, group=self.group)

    def step(self, tokens: torch.Tensor, embed: Callable, layers: Callable, head: Callable, act_shape: tuple[int, ...],
             act_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """Run one forward over all stages; every rank returns the next token(s).

        `embed(tokens)` runs on the first stage, `layers(x, lo, hi)` on each, `head(x)` (-> token ids)
        on the last."""
        dev = tokens.device
        if self.first:
            x = embed(tokens)
        else:
            x = torch.empty(act_shape, dtype=act_dtype, device=dev)
            self._p2p(dist.recv, x, self.rank - 1)
        x = layers(x, self.lo, self.hi)
        if not self.last:
            self._p2p(dist.send, x.contiguous(), self.rank + 1)
            nxt = torch.empty(tokens.shape[0], dtype=torch.long, device=dev)
        else:
            nxt = head(x).to(torch.long)
        dist.broadcast(nxt, src=self.world - 1, group=self.group)
        return nxt
