"""Host tier of a compressed KV cache (`csrc/engine/kv_swap.cpp`): all rows in pinned host memory, a fixed number of
device slots, the indexer's selection made resident per step (hits stay, misses arrive in one packed transfer and are
scattered into least-recently-used slots), selection rewritten to physical rows.

Reference counterpart: GgufKvSwapLayerState / gguf_kv_swap_in_selected (cpp_engine/src/dsv4_engine.cpp:5260-5434,
enabled by scripts/flashmemory_kv_swap_demo.sh).
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import lib as _lib


class KvSwapError(RuntimeError):
    pass


class KvSwapTier:
    """`capacity` logical rows of `row_bytes` on the host, `device_slots` of them resident in `pool` (a uint8 tensor
    [device_slots, row_bytes] owned here, or `pool=` a caller's view, e.g. the rows of a KV array behind its window),
    physical row of slot s = `window + s`. With `host_only` everything lives in host
    memory (tests without a GPU)."""

    def __init__(self, capacity: int, device_slots: int, row_bytes: int, window: int = 0, *, host_only: bool = False, device: str | torch.device = "cuda",
                 pool: torch.Tensor | None = None):
        self._L = _lib.engine()
        L = self._L
        L.pk_kvswap_create.restype = ctypes.c_void_p
        L.pk_engine_last_error.restype = ctypes.c_char_p
        self.host_only = host_only
        self.capacity, self.row_bytes, self.window = capacity, row_bytes, window
        self.device_slots = min(device_slots, capacity)
        h = L.pk_kvswap_create(capacity, device_slots, ctypes.c_ulonglong(row_bytes), window, int(host_only))
        if not h:
            raise KvSwapError(L.pk_engine_last_error().decode())
        self._h = ctypes.c_void_p(h)
        if pool is None:
            pool = torch.zeros(self.device_slots, row_bytes, dtype=torch.uint8, device="cpu" if host_only else device)
        elif not pool.is_contiguous() or pool.numel() * pool.element_size() != self.device_slots * row_bytes:
            raise ValueError("pool must be contiguous and hold device_slots rows of row_bytes")
        self.pool = pool          # may be a view into a larger KV array (the rows behind an attention window)

    def _ck(self, st: int) -> None:
        if st != 0:
            raise KvSwapError(self._L.pk_engine_last_error().decode())

    def _stream(self) -> ctypes.c_void_p:
        return ctypes.c_void_p(0 if self.host_only else torch.cuda.current_stream().cuda_stream)

    def store(self, first: int, rows: torch.Tensor) -> None:
        """Rows [count, row_bytes worth of elements] produced on the device become logical rows first .. first + count."""
        rows = rows.contiguous()
        count = rows.shape[0]
        if rows.numel() * rows.element_size() != count * self.row_bytes:
            raise ValueError("row size does not match the tier's row_bytes")
        self._ck(self._L.pk_kvswap_store(self._h, first, count, ctypes.c_void_p(rows.data_ptr()), self._stream()))

    def swap_in(self, selected: torch.Tensor) -> torch.Tensor:
        """selected int32 [...] logical ids (-1 = none) -> int32 tensor of the same shape with physical rows; afterwards
        `pool[physical - window]` holds every selected row."""
        sel = selected.contiguous()
        if sel.dtype != torch.int32:
            raise ValueError("selection must be int32")
        out = torch.empty_like(sel)
        self._ck(self._L.pk_kvswap_swap_in(self._h, ctypes.c_void_p(sel.data_ptr()), sel.numel(), ctypes.c_void_p(self.pool.data_ptr()),
                                           ctypes.c_void_p(out.data_ptr()), self._stream()))
        return out

    def reset(self) -> None:
        self._ck(self._L.pk_kvswap_reset(self._h))

    @property
    def stats(self) -> dict:
        buf = (ctypes.c_ulonglong * 8)()
        self._L.pk_kvswap_stats(self._h, buf)
        keys = ("hits", "misses", "h2d_bytes", "d2h_bytes", "evictions", "steps", "stored_rows", "host_bytes")
        return dict(zip(keys, (int(v) for v in buf)))

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._L.pk_kvswap_destroy(self._h)
            self._h = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass
