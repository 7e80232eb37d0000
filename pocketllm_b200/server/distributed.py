"""The Python server under several ranks (tensor- or expert-parallel engines started with torchrun).

Rank 0 runs the HTTP server; every request it serves is first broadcast to the other ranks over a CPU (gloo) control
group, and every rank then runs the same `backend.generate` call, so the collectives inside the model line up. The
other ranks sit in `worker_loop`. Stop conditions depend only on the tokens and the parameters, so all ranks leave a
request at the same step; a request that rank 0's client abandons is still run to its end on every rank.
Role of the reference's `_broadcast_payload` and `_worker_loop` (src/server/openai.py:717-720, 1050-1064).
"""
from __future__ import annotations

from datetime import timedelta
from typing import Iterator, Sequence

import torch.distributed as dist

from .engine import SamplingParams, TokenInfo

_SHUTDOWN = {"op": "shutdown"}


def control_group():
    """A gloo group over all ranks for request payloads (long timeout: workers wait for traffic)."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return None
    return dist.new_group(backend="gloo", timeout=timedelta(days=7))


def _stops(tokens: Sequence[int], params: SamplingParams) -> bool:
    return len(tokens) >= params.max_tokens or (len(tokens) > 0 and tokens[-1] in params.stop_token_ids)


class DistributedBackend:
    """Rank 0 side: announces each request, then generates; always runs the request to its end."""

    def __init__(self, backend, group):
        self.backend, self.group = backend, group
        self.max_batch_size = 1

    def generate(self, prompt_ids: Sequence[int], params: SamplingParams) -> Iterator[int]:
        dist.broadcast_object_list([{"op": "generate", "prompt": list(prompt_ids), "params": vars(params)}], src=0, group=self.group)
        produced: list[int] = []
        it = self.backend.generate(prompt_ids, params)
        try:
            for tok in it:
                produced.append(int(tok))
                yield tok if isinstance(tok, TokenInfo) else int(tok)      # log-probability reports pass through
        finally:
            # the consumer may have left early (client gone, stop string): the workers still run to the natural end
            if not _stops(produced, params):
                for tok in it:
                    produced.append(int(tok))

    def shutdown(self) -> None:
        dist.broadcast_object_list([_SHUTDOWN], src=0, group=self.group)


def worker_loop(backend, group) -> int:
    """Ranks > 0: follow rank 0's requests until it says shutdown. Returns the number of requests served."""
    served = 0
    while True:
        box = [None]
        dist.broadcast_object_list(box, src=0, group=group)
        msg = box[0]
        if not isinstance(msg, dict) or msg.get("op") == "shutdown":
            return served
        if msg.get("op") == "generate":
            p = msg["params"]
            p["stop_token_ids"] = tuple(p.get("stop_token_ids", ()))
            params = SamplingParams(**p)
            for _ in backend.generate(msg["prompt"], params):
                pass
            served += 1
