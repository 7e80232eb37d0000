"""Bindings of the native expert staging (csrc/engine/staging.*): the LRU slot bookkeeping, and the device arena that
brings host-resident experts in through page-locked bounce slots. Same decisions as `expert_cache.LRUSlots`; meant for
callers that drive the kernels from C++ or want the staging off the Python thread."""
from __future__ import annotations

import ctypes
from typing import Sequence

import torch

from ..ops import lib as _lib


class NativeError(RuntimeError):
    pass


def _engine() -> ctypes.CDLL:
    L = _lib.engine()
    L.pk_lru_create.restype = ctypes.c_void_p
    L.pk_expert_arena_create.restype = ctypes.c_void_p
    L.pk_engine_last_error.restype = ctypes.c_char_p
    return L


class NativeLruSlots:
    """`assign(needed)` -> (slot of every needed key, [(key, slot)] to load); keys of one call never evict one another."""

    def __init__(self, slots: int):
        self._L = _engine()
        h = self._L.pk_lru_create(slots)
        if not h:
            raise NativeError(self._L.pk_engine_last_error().decode())
        self._h = ctypes.c_void_p(h)
        self.stats = {"hits": 0, "misses": 0, "evictions": 0}

    def assign(self, needed: Sequence[int]) -> tuple[list[int], list[tuple[int, int]]]:
        n = len(needed)
        keys = (ctypes.c_longlong * max(n, 1))(*[int(k) for k in needed])
        slots = (ctypes.c_int * max(n, 1))()
        lk = (ctypes.c_longlong * max(n, 1))()
        ls = (ctypes.c_int * max(n, 1))()
        nl = ctypes.c_int(0)
        st = (ctypes.c_longlong * 3)()
        if self._L.pk_lru_assign(self._h, keys, n, slots, lk, ls, ctypes.byref(nl), st) != 0:
            raise NativeError(self._L.pk_engine_last_error().decode())
        self.stats = {"hits": int(st[0]), "misses": int(st[1]), "evictions": int(st[2])}
        return list(slots[:n]), [(int(lk[i]), int(ls[i])) for i in range(nl.value)]

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._L.pk_lru_destroy(self._h)
            self._h = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass


class NativeExpertArena:
    """Device slots for experts whose bytes stay in host memory (`store`: uint8 [n_experts, expert_bytes], any host
    tensor). `ensure(keys)` returns one uint8 device view per key, valid until a later `ensure` evicts it."""

    def __init__(self, store: torch.Tensor, device_slots: int, ring_slots: int = 4):
        if store.device.type != "cpu" or store.dtype != torch.uint8 or store.dim() != 2 or not store.is_contiguous():
            raise ValueError("store must be a contiguous uint8 host tensor [n_experts, expert_bytes]")
        self._L = _engine()
        self.store = store
        self.expert_bytes = store.shape[1]
        h = self._L.pk_expert_arena_create(device_slots, ctypes.c_ulonglong(self.expert_bytes), ring_slots)
        if not h:
            raise NativeError(self._L.pk_engine_last_error().decode())
        self._h = ctypes.c_void_p(h)
        if self._L.pk_expert_arena_set_host_store(self._h, ctypes.c_void_p(store.data_ptr()), ctypes.c_longlong(store.shape[0])) != 0:
            raise NativeError(self._L.pk_engine_last_error().decode())
        self.stats = {"hits": 0, "misses": 0, "evictions": 0, "bytes_copied": 0, "ring_waits": 0}

    def ensure_ptrs(self, keys: Sequence[int]) -> list[int]:
        n = len(keys)
        arr = (ctypes.c_longlong * max(n, 1))(*[int(k) for k in keys])
        out = (ctypes.c_void_p * max(n, 1))()
        st = (ctypes.c_longlong * 5)()
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        if self._L.pk_expert_arena_ensure(self._h, arr, n, out, stream, st) != 0:
            raise NativeError(self._L.pk_engine_last_error().decode())
        self.stats = dict(zip(("hits", "misses", "evictions", "bytes_copied", "ring_waits"), (int(v) for v in st)))
        return [int(out[i] or 0) for i in range(n)]

    def read_back(self, ptr: int) -> torch.Tensor:
        """Host copy of the expert-sized slot at device address `ptr` (synchronous; for checks)."""
        torch.cuda.current_stream().synchronize()
        out = torch.empty(self.expert_bytes, dtype=torch.uint8)
        if self._L.pk_device_read(ctypes.c_void_p(ptr), ctypes.c_void_p(out.data_ptr()), ctypes.c_ulonglong(self.expert_bytes)) != 0:
            raise NativeError(self._L.pk_engine_last_error().decode())
        return out

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._L.pk_expert_arena_destroy(self._h)
            self._h = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass
