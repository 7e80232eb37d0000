"""Model-independent greedy generation over a token runtime, with the timing convention of
the reference (src/runtime/generation.py:74-126, docs/benchmarking.md:20-30): prefill time
covers the prompt and the first generated token, decode counts the later tokens; every
phase is bracketed by a device synchronise and, with several ranks, a barrier.
"""
from __future__ import annotations

import os
import struct
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Protocol, Sequence

import torch


class TokenRuntime(Protocol):
    """What a model must offer: `prefill` consumes the prompt and returns the first greedy
    token, `decode_one` feeds one token and returns the next, `reset` clears the caches."""

    def prefill(self, tokens: Sequence[int]) -> int: ...
    def decode_one(self, token: int) -> int: ...
    def reset(self) -> None: ...


@dataclass
class GenerationResult:
    tokens: list[int] = field(default_factory=list)
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    prompt_tokens: int = 0

    @property
    def prefill_tps(self) -> float:
        return self.prompt_tokens / self.prefill_seconds if self.prefill_seconds > 0 else 0.0

    @property
    def decode_tps(self) -> float:
        n = max(len(self.tokens) - 1, 0)
        return n / self.decode_seconds if self.decode_seconds > 0 and n else 0.0

    def result_line(self) -> str:
        return (f"RESULT prefill_seconds={self.prefill_seconds:.6f} prefill_tps={self.prefill_tps:.3f} "
                f"decode_seconds={self.decode_seconds:.6f} decode_tps={self.decode_tps:.3f}")


def setup_dist() -> tuple[int, int, int]:
    """(rank, world, local_rank) from the torchrun environment; initialises NCCL when world > 1."""
    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
    if world > 1 and not torch.distributed.is_initialized():
        backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {"device_id": torch.device("cuda", local)} if backend == "nccl" else {}
        torch.distributed.init_process_group(backend, **kw)
    return rank, world, local


def _sync() -> None:
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        torch.distributed.barrier()


def read_seed_tokens(path: str | Path) -> list[int]:
    """Raw little-endian token ids: int64 when the size is a multiple of 8 and the values are
    plausible, else int32 (same rule as the reference's seed-file reader, generation.py:53-64)."""
    data = Path(path).read_bytes()
    if len(data) % 8 == 0 and data:
        vals = list(struct.unpack(f"<{len(data) // 8}q", data))
        if all(0 <= v < (1 << 31) for v in vals):
            return vals
    if len(data) % 4:
        raise ValueError(f"{path}: size {len(data)} is not a multiple of 4")
    return list(struct.unpack(f"<{len(data) // 4}i", data))


def greedy_generate(rt: TokenRuntime, prompt: Sequence[int], max_new_tokens: int, eos: int | None = None) -> GenerationResult:
    res = GenerationResult(prompt_tokens=len(prompt))
    rt.reset()
    _sync()
    t0 = time.perf_counter()
    tok = rt.prefill(prompt)
    _sync()
    res.prefill_seconds = time.perf_counter() - t0
    res.tokens.append(tok)
    t0 = time.perf_counter()
    while len(res.tokens) < max_new_tokens and (eos is None or tok != eos):
        tok = rt.decode_one(tok)
        res.tokens.append(tok)
    _sync()
    res.decode_seconds = time.perf_counter() - t0
    return res
