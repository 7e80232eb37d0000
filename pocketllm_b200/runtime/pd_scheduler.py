"""Prefill/decode scheduler for a single-stream engine.

Requests wait in two queues; a request whose prefill is done moves to the decode queue, and
decode work always runs before a new prefill (a started generation is never starved by
arriving prompts). Per-phase resource hints (CPU affinity, thread counts) are applied when
the phase changes. Counterpart of the reference's `PDScheduler`
(src/runtime/pd_scheduler.py:1-361) without its CPU-expert server control: experts live on
the GPUs here, so there is no process to stop and resume between phases.
"""
from __future__ import annotations

import heapq
import itertools
import os
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable


@dataclass
class PhaseResources:
    cpu_affinity: tuple[int, ...] | None = None
    threads: int | None = None
    env: dict[str, str] = field(default_factory=dict)


@dataclass(order=True)
class _Item:
    priority: int
    seq: int
    request: Any = field(compare=False)
    phase: str = field(compare=False, default="prefill")
    enqueued: float = field(compare=False, default_factory=time.perf_counter)


class PDScheduler:
    """`submit(request)` then repeatedly `next()` -> (request, phase); call `prefill_done(request)`
    to move it to the decode queue and `finish(request)` when it ends."""

    def __init__(self, prefill: PhaseResources | None = None, decode: PhaseResources | None = None, max_pending: int = 256,
                 decode_slice: int = 32):
        self.res = {"prefill": prefill or PhaseResources(), "decode": decode or PhaseResources()}
        self.max_pending, self.decode_slice = max_pending, decode_slice
        self._prefill: list[_Item] = []
        self._decode: list[_Item] = []
        self._seq = itertools.count()
        self._lock = threading.Condition()
        self.phase: str | None = None
        self.stats = {"submitted": 0, "prefills": 0, "decode_slices": 0, "phase_switches": 0, "rejected": 0,
                      "max_wait_s": 0.0}

    def submit(self, request: Any, priority: int = 0) -> bool:
        with self._lock:
            if len(self._prefill) + len(self._decode) >= self.max_pending:
                self.stats["rejected"] += 1
                return False
            heapq.heappush(self._prefill, _Item(priority, next(self._seq), request, "prefill"))
            self.stats["submitted"] += 1
            self._lock.notify()
            return True

    def prefill_done(self, request: Any, priority: int = 0) -> None:
        with self._lock:
            heapq.heappush(self._decode, _Item(priority, next(self._seq), request, "decode"))
            self._lock.notify()

    def requeue_decode(self, request: Any, priority: int = 0) -> None:
        """A decode slice ended without finishing the request."""
        self.prefill_done(request, priority)

    def finish(self, request: Any) -> None:
        pass

    def pending(self) -> tuple[int, int]:
        with self._lock:
            return len(self._prefill), len(self._decode)

    def next(self, timeout: float | None = None) -> tuple[Any, str] | None:
        """Decode first; a prefill only when no generation is waiting."""
        with self._lock:
            if not self._prefill and not self._decode:
                self._lock.wait(timeout)
            if self._decode:
                item = heapq.heappop(self._decode)
                self.stats["decode_slices"] += 1
            elif self._prefill:
                item = heapq.heappop(self._prefill)
                self.stats["prefills"] += 1
            else:
                return None
            self.stats["max_wait_s"] = max(self.stats["max_wait_s"], time.perf_counter() - item.enqueued)
        self.apply_phase_resources(item.phase)
        return item.request, item.phase

    def apply_phase_resources(self, phase: str) -> None:
        if phase == self.phase:
            return
        self.phase = phase
        self.stats["phase_switches"] += 1
        r = self.res[phase]
        for k, v in r.env.items():
            os.environ[k] = v
        if r.threads:
            try:
                import torch
                torch.set_num_threads(r.threads)
            except Exception:
                pass
        if r.cpu_affinity and hasattr(os, "sched_setaffinity"):
            try:
                os.sched_setaffinity(0, set(r.cpu_affinity))
            except OSError:
                pass
