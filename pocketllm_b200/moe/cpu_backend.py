"""Routed experts on the host CPU with an asynchronous submit / sync interface: a persistent worker thread runs the
native FP4 expert pass (`csrc/cpu/moe_cpu.cpp`) while the caller keeps the GPU busy with attention of the same layer
(reference: src/components/moe/cpu_backend.py - `_PersistentCPUWorker` 204-248, `CPURoutedExpertsBackend` 372-,
`dispatch_forward` 1095). On a 180 GB GPU the experts normally live in HBM; this backend serves checkpoints that do
not fit, and is the CPU oracle of the GPU expert kernels."""
from __future__ import annotations

import queue
import threading
import time

import torch

from . import cpu_oracle as co


class CPURoutedExpertsBackend:
    def __init__(self, layers: dict[int, co.Fp4MoEWeights], topk: int, *, score_func: str = "softmax", norm_topk: bool = True,
                 route_scale: float = 1.0, swiglu_limit: float = 0.0, pinned: bool = False):
        self.layers, self.topk = layers, topk
        self.kw = dict(score_func=score_func, norm_topk=norm_topk, route_scale=route_scale, swiglu_limit=swiglu_limit)
        self.pinned = pinned and torch.cuda.is_available()
        self._jobs: "queue.Queue[tuple | None]" = queue.Queue()
        self._done: "queue.Queue[tuple]" = queue.Queue()
        self._inflight = False
        self.stats = {"calls": 0, "tokens": 0, "expert_seconds": 0.0, "wait_seconds": 0.0}
        self._thread = threading.Thread(target=self._loop, name="cpu-moe-worker", daemon=True)
        self._thread.start()

    def _loop(self) -> None:
        while True:
            job = self._jobs.get()
            if job is None:
                return
            layer, x = job
            try:
                y, counts, dt = co.forward_native(x, self.layers[layer], self.topk, **self.kw)
                self._done.put((y, counts, dt, None))
            except Exception as e:                       # reported to the caller in sync()
                self._done.put((None, None, 0.0, e))

    def submit(self, layer: int, x: torch.Tensor) -> None:
        """Start the expert pass of `layer` for activations x [T, H] (any device; copied to the host)."""
        if self._inflight:
            raise RuntimeError("a CPU expert pass is already in flight; call sync() first")
        if layer not in self.layers:
            raise KeyError(f"no routed experts for layer {layer}")
        xh = x.detach().to("cpu", torch.float32, non_blocking=False).contiguous()
        self._inflight = True
        self._jobs.put((layer, xh))

    def sync(self, device: torch.device | str | None = None) -> torch.Tensor:
        """Wait for the submitted pass and return y [T, H] fp32 (moved to `device` when given)."""
        if not self._inflight:
            raise RuntimeError("sync() without submit()")
        t0 = time.perf_counter()
        y, counts, dt, err = self._done.get()
        self._inflight = False
        if err is not None:
            raise err
        self.stats["calls"] += 1
        self.stats["tokens"] += y.shape[0]
        self.stats["expert_seconds"] += dt
        self.stats["wait_seconds"] += time.perf_counter() - t0
        self.last_counts = counts
        if self.pinned:
            y = y.pin_memory()
        return y.to(device, non_blocking=self.pinned) if device is not None else y

    def forward(self, layer: int, x: torch.Tensor) -> torch.Tensor:
        self.submit(layer, x)
        return self.sync(x.device)

    def close(self) -> None:
        self._jobs.put(None)
        self._thread.join(timeout=10)
