"""Serving engine: a request queue in front of one model worker thread.

HTTP handler threads submit work and read their tokens from a per-request queue. A backend that declares
`max_batch_size > 1` and implements `generate_batch` gets compatible non-streaming requests together: the worker
waits a short window (`batch_wait_ms`) for more requests with the same sampling parameters and runs them as one call;
every other request runs alone. Same role as the reference's `DeepSeekServingEngine` (src/server/engine.py:
queue + one worker thread, `_collect_batch`, `_is_batch_compatible`).
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
    logprobs: int = -1           # -1: off; k >= 0: log-probability of every generated token and of the k most likely ones


@dataclass
class TokenInfo:
    """A generated token with the model's log-probabilities at its step (backends yield these instead of plain ids when
    `SamplingParams.logprobs >= 0`)."""
    token: int
    logprob: float
    top: list[tuple[int, float]] = field(default_factory=list)

    def __int__(self) -> int:
        return self.token


def token_logprobs(logits, token: int, k: int) -> TokenInfo:
    """log-softmax of a 1-D logits tensor: the chosen token's entry and the k largest (the model's distribution, before
    temperature, penalties or filtering)."""
    import torch
    lp = torch.log_softmax(logits.float(), -1)
    top = []
    if k > 0:
        v, i = torch.topk(lp, min(k, lp.numel()))
        top = [(int(a), float(b)) for a, b in zip(i.tolist(), v.tolist())]
    return TokenInfo(int(token), float(lp[int(token)]), top)


class TokenBackend(Protocol):
    """What the server needs from a model: stream greedy/sampled tokens for a prompt. Optional: `max_batch_size` and
    `generate_batch(prompts, params_list) -> list[list[int]]` for backends that run several requests in one pass."""

    def generate(self, prompt_ids: Sequence[int], params: SamplingParams) -> Iterator[int]: ...


@dataclass
class _Job:
    prompt_ids: list[int]
    params: SamplingParams
    out: "queue.Queue[object]" = field(default_factory=queue.Queue)
    submitted: float = field(default_factory=time.perf_counter)
    cancelled: threading.Event = field(default_factory=threading.Event)
    batchable: bool = False      # the caller reads the whole completion at once (not a stream)


_DONE = object()


def batch_compatible(a: SamplingParams, b: SamplingParams) -> bool:
    """Requests share a batch when one sampler setting serves both (lengths and seeds may differ for greedy runs)."""
    same = (a.temperature, a.top_p, a.top_k, a.min_p, a.frequency_penalty, a.presence_penalty, a.repetition_penalty, a.stop_token_ids) == \
           (b.temperature, b.top_p, b.top_k, b.min_p, b.frequency_penalty, b.presence_penalty, b.repetition_penalty, b.stop_token_ids)
    return same and (a.temperature <= 0 or a.seed == b.seed)


class ServingEngine:
    def __init__(self, backend: TokenBackend, max_queue: int = 64, batch_wait_ms: float = 2.0):
        self.backend = backend
        self.batch_wait_ms = batch_wait_ms
        self.max_batch = int(getattr(backend, "max_batch_size", 1)) if hasattr(backend, "generate_batch") else 1
        self._q: "queue.Queue[_Job | None]" = queue.Queue(max_queue)
        self._held: list[_Job] = []          # taken off the queue while looking for batch partners, to run next
        self.stats = {"requests": 0, "tokens": 0, "errors": 0, "batches": 0, "batched_requests": 0}
        self._thread = threading.Thread(target=self._loop, name="pocket-serving", daemon=True)
        self._thread.start()

    def _collect_batch(self, first: _Job) -> list[_Job]:
        batch = [first]
        deadline = time.monotonic() + self.batch_wait_ms / 1000.0
        while len(batch) < self.max_batch:
            left = deadline - time.monotonic()
            try:
                cand = self._q.get(timeout=max(left, 0.0)) if left > 0 else self._q.get_nowait()
            except queue.Empty:
                break
            if cand is None:
                self._q.put(None)            # shutdown marker: leave it for the main loop
                break
            if cand.batchable and batch_compatible(first.params, cand.params):
                batch.append(cand)
            else:
                self._held.append(cand)      # runs right after this batch, in arrival order
                break
        return batch

    def _run_batch(self, batch: list[_Job]) -> None:
        try:
            outs = self.backend.generate_batch([j.prompt_ids for j in batch], [j.params for j in batch])
            if len(outs) != len(batch):
                raise RuntimeError("batched backend returned a result list of the wrong length")
            self.stats["batches"] += 1
            self.stats["batched_requests"] += len(batch)
            for job, toks in zip(batch, outs):
                job.out.put(("ttft", time.perf_counter() - job.submitted))
                for t in toks:
                    job.out.put(t if isinstance(t, TokenInfo) else int(t))
                self.stats["tokens"] += len(toks)
                self.stats["requests"] += 1
        except Exception as e:
            self.stats["errors"] += len(batch)
            for job in batch:
                job.out.put(e)
        finally:
            for job in batch:
                job.out.put(_DONE)

    def _loop(self) -> None:
        while True:
            job = self._held.pop(0) if self._held else self._q.get()
            if job is None:
                return
            if job.batchable and self.max_batch > 1:
                batch = self._collect_batch(job)
                if len(batch) > 1:
                    self._run_batch(batch)
                    continue
            try:
                first = True
                for tok in self.backend.generate(job.prompt_ids, job.params):
                    if first:
                        job.out.put(("ttft", time.perf_counter() - job.submitted))
                        first = False
                    job.out.put(tok if isinstance(tok, TokenInfo) else int(tok))
                    self.stats["tokens"] += 1
                    if job.cancelled.is_set():
                        break
                self.stats["requests"] += 1
            except Exception as e:  # the worker survives a failed request
                self.stats["errors"] += 1
                job.out.put(e)
            finally:
                job.out.put(_DONE)

    def stream(self, prompt_ids: Sequence[int], params: SamplingParams, batchable: bool = False) -> Iterator[object]:
        """Yields ("ttft", seconds) once, then token ids (`TokenInfo` objects when log-probabilities were asked for); raises what the backend raised. `batchable`: the caller does
        not need tokens one by one, so the request may share a pass with compatible ones."""
        job = _Job(list(prompt_ids), params, batchable=batchable)
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

    def queue_depth(self) -> int:
        """Requests waiting for the worker (not counting the one that runs)."""
        return self._q.qsize() + len(self._held)

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
