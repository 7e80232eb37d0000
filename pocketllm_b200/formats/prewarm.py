"""Page-cache warm-up of checkpoint files before loading (sequential read with a read-ahead
hint), as the reference does for multi-hundred-GB GGUF bundles (src/loader/gguf/prewarm.py)."""
from __future__ import annotations

import os
import time
from pathlib import Path

from . import gguf


def prewarm(path: str | os.PathLike, chunk_mib: int = 64, max_bytes: int | None = None) -> dict:
    files = gguf.shard_paths(path) if str(path).endswith(".gguf") else [Path(path)]
    total, t0 = 0, time.perf_counter()
    for f in files:
        fd = os.open(f, os.O_RDONLY)
        try:
            size = os.fstat(fd).st_size
            if hasattr(os, "posix_fadvise"):
                os.posix_fadvise(fd, 0, 0, os.POSIX_FADV_SEQUENTIAL)
                os.posix_fadvise(fd, 0, 0, os.POSIX_FADV_WILLNEED)
            off = 0
            step = chunk_mib << 20
            while off < size and (max_bytes is None or total < max_bytes):
                n = len(os.pread(fd, step, off))
                if n == 0:
                    break
                off += n
                total += n
        finally:
            os.close(fd)
    dt = time.perf_counter() - t0
    return {"files": len(files), "bytes": total, "seconds": dt, "gib_per_s": total / dt / (1 << 30) if dt > 0 else 0.0}
