"""Serving engine: a request queue in front of one model worker thread.

The model runs one request at a time (single-request latency is what the engines are built
for); HTTP handler threads submit work and wait on a future, streaming requests receive
their tokens through a per-request queue. Same role as the reference's
`DeepSeekServingEngine` (src/server/engine.py: queue + one worker thread).
"""
from __future__ import annotations

import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Iterator, Protocol, Sequence


@dataclass
class SamplingParams:
    max_tokens: int = 512
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repetition_penalty: float = 1.0
    seed: int | None = None
    stop_token_ids: tuple[int, ...] = ()


class TokenBackend(Protocol):
    """What the server needs from a model: stream greedy/sampled tokens for a prompt."""

    def generate(self, prompt_ids: Sequence[int], params: SamplingParams) -> Iterator[int]: ...


@dataclass
class _Job:
    prompt_ids: list[int]
    params: SamplingParams
    out: "queue.Queue[object]" = field(default_factory=queue.Queue)
    submitted: float = field(default_factory=time.perf_counter)
    cancelled: threading.Event = field(default_factory=threading.Event)


_DONE = object()


class ServingEngine:
    def __init__(self, backend: TokenBackend, max_queue: int = 64):
        self.backend = backend
        self._q: "queue.Queue[_Job | None]" = queue.Queue(max_queue)
        self._thread = threading.Thread(target=self._loop, name="pocket-serving", daemon=True)
        self._thread.start()
        self.stats = {"requests": 0, "tokens": 0, "errors": 0}

    def _loop(self) -> None:
        while True:
            job = self._q.get()
            if job is None:
                return
            try:
                first = True
                for tok in self.backend.generate(job.prompt_ids, job.params):
                    if first:
                        job.out.put(("ttft", time.perf_counter() - job.submitted))
                        first = False
                    job.out.put(int(tok))
                    self.stats["tokens"] += 1
                    if job.cancelled.is_set():
                        break
                self.stats["requests"] += 1
            except Exception as e:  # the worker survives a failed request
                self.stats["errors"] += 1
                job.out.put(e)
            finally:
                job.out.put(_DONE)

    def stream(self, prompt_ids: Sequence[int], params: SamplingParams) -> Iterator[object]:
        """Yields ("ttft", seconds) once, then token ids; raises what the backend raised."""
        job = _Job(list(prompt_ids), params)
        try:
            self._q.put(job, timeout=1.0)
        except queue.Full:
            raise RuntimeError("server busy: request queue is full")
        try:
            while True:
                item = job.out.get()
                if item is _DONE:
                    return
                if isinstance(item, Exception):
                    raise item
                yield item
        finally:
            job.cancelled.set()

    def close(self) -> None:
        self._q.put(None)
        self._thread.join(timeout=5)


def apply_penalties(logits, generated: Sequence[int], p: SamplingParams):
    """Frequency / presence / repetition penalties on a 1-D torch logits tensor (in place)."""
    if not generated or (p.frequency_penalty == 0 and p.presence_penalty == 0 and p.repetition_penalty == 1.0):
        return logits
    import torch
    ids, counts = torch.unique(torch.tensor(list(generated), device=logits.device), return_counts=True)
    sel = logits[ids]
    if p.repetition_penalty != 1.0:
        sel = torch.where(sel > 0, sel / p.repetition_penalty, sel * p.repetition_penalty)
    sel = sel - p.frequency_penalty * counts.to(sel.dtype) - p.presence_penalty
    logits[ids] = sel
    return logits


def sample_token(logits, p: SamplingParams, generator=None) -> int:
    """temperature 0 -> argmax (lowest id on ties); else top-k / top-p / min-p filtering and a draw."""
    import torch
    if p.temperature <= 0:
        return int(torch.argmax(logits))
    z = logits.float() / p.temperature
    if p.top_k and p.top_k < z.numel():
        kth = torch.topk(z, p.top_k).values[-1]
        z = z.masked_fill(z < kth, float("-inf"))
    probs = torch.softmax(z, -1)
    if p.min_p > 0:
        probs = probs.masked_fill(probs < p.min_p * probs.max(), 0.0)
    if p.top_p < 1.0:
        sp, si = torch.sort(probs, descending=True)
        keep = torch.cumsum(sp, 0) - sp < p.top_p
        mask = torch.zeros_like(probs, dtype=torch.bool)
        mask[si[keep]] = True
        probs = probs.masked_fill(~mask, 0.0)
    probs = probs / probs.sum()
    return int(torch.multinomial(probs, 1, generator=generator))
