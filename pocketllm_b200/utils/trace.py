"""Tracing helpers: device-timed sections (CUDA events, no host synchronisation inside the timed region, maximum
over ranks when a process group is up), NVTX ranges for external profilers, and the roofline arithmetic used in
the profile summaries (reference timers: the env-gated wall-clock sections of cpp_engine/src/dsv4_engine.cpp:4906-4988,
which synchronise the device around every stage; these do not)."""
from __future__ import annotations

import contextlib
import json
from collections import defaultdict
from pathlib import Path

import torch

_FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
NVLINK_GBS_MEASURED, NVLINK_GBS_NOMINAL = 770.0, 900.0


def measured_peaks(repo_root: str | Path | None = None) -> dict:
    """Copy bandwidth (GB/s) and bf16 GEMM throughput (TFLOP/s) measured on this pool, or the documented fallback."""
    root = Path(repo_root) if repo_root else Path(__file__).resolve().parents[2]
    p = root / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d.get("hbm_gbs", _FALLBACK_PEAKS["hbm_gbs"])), "bf16_tflops": float(d.get("bf16_tflops", _FALLBACK_PEAKS["bf16_tflops"])),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d.get("bf16_tflops", 0.0))), "source": "measured"}
    return dict(_FALLBACK_PEAKS)


def roofline(*, flops: float = 0.0, hbm_bytes: float = 0.0, nvlink_bytes: float = 0.0, seconds: float, peaks: dict | None = None) -> dict:
    """Bound time = the slowest of compute, HBM and NVLink at the measured peaks; fraction = bound / achieved."""
    pk = peaks or measured_peaks()
    t_compute = flops / (pk["bf16_tflops"] * 1e12) if flops else 0.0
    t_hbm = hbm_bytes / (pk["hbm_gbs"] * 1e9) if hbm_bytes else 0.0
    t_link = nvlink_bytes / (NVLINK_GBS_MEASURED * 1e9) if nvlink_bytes else 0.0
    bound = max(t_compute, t_hbm, t_link)
    limiter = "compute" if bound == t_compute and flops else "hbm" if bound == t_hbm and hbm_bytes else "nvlink"
    return {"bound_s": bound, "limiter": limiter, "fraction_of_" + pk.get("source", "measured"): bound / seconds if seconds > 0 else 0.0,
            "achieved_tflops": flops / seconds / 1e12 if seconds > 0 else 0.0, "achieved_gbs": hbm_bytes / seconds / 1e9 if seconds > 0 else 0.0}


class SectionTimer:
    """`with timer.section("attn"):` around device work; `summary()` after a single synchronise."""

    def __init__(self, enabled: bool = True, nvtx: bool = True):
        self.enabled, self.nvtx = enabled and torch.cuda.is_available(), nvtx and torch.cuda.is_available()
        self._events: dict[str, list[tuple[torch.cuda.Event, torch.cuda.Event]]] = defaultdict(list)

    @contextlib.contextmanager
    def section(self, name: str):
        if self.nvtx:
            torch.cuda.nvtx.range_push(name)
        if self.enabled:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
        try:
            yield
        finally:
            if self.enabled:
                b.record()
                self._events[name].append((a, b))
            if self.nvtx:
                torch.cuda.nvtx.range_pop()

    def summary(self, group=None) -> dict[str, dict[str, float]]:
        """Per section: calls, total and mean milliseconds (device time; maximum over the ranks of `group`)."""
        if not self.enabled:
            return {}
        torch.cuda.synchronize()
        out = {}
        for name, evs in self._events.items():
            total = sum(a.elapsed_time(b) for a, b in evs)
            if group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()):
                t = torch.tensor([total], device="cuda")
                torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX, group=group)
                total = float(t)
            out[name] = {"calls": len(evs), "total_ms": total, "mean_ms": total / len(evs)}
        return out

    def reset(self) -> None:
        self._events.clear()
