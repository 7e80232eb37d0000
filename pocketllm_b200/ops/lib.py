"""Loader of the in-tree native libraries.

The CUDA path is the only path: when a GPU is present and the libraries are missing or
stale, importing an op raises instead of falling back to PyTorch.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_DIR = Path(__file__).resolve().parent.parent / "_C"
_libs: dict[str, ctypes.CDLL] = {}


class NativeLibraryMissing(RuntimeError):
    pass


def lib_path(name: str) -> Path:
    return _DIR / f"libpocket_{name}.so"


def load(name: str) -> ctypes.CDLL:
    """Load `libpocket_<name>.so` from `pocketllm_b200/_C` (built by `python -m pocketllm_b200.build`)."""
    if name in _libs:
        return _libs[name]
    path = lib_path(name)
    if not path.exists():
        raise NativeLibraryMissing(
            f"{path} not found: run `python -m pocketllm_b200.build` (nvcc cross-compiles sm_100a without a GPU)")
    mode = ctypes.RTLD_GLOBAL if name.startswith("kernels") else ctypes.DEFAULT_MODE
    if name == "engine":
        load("kernels")
    lib = ctypes.CDLL(str(path), mode=mode)
    _libs[name] = lib
    return lib


def available(name: str = "kernels") -> bool:
    return lib_path(name).exists()


def kernels() -> ctypes.CDLL:
    """The kernel library; with POCKET_KERNELS_DEBUG=1 its twin compiled with index checks that record a bad KV position or
    route id in a status word and skip the access (`debug_bounds()` reads it)."""
    if os.environ.get("POCKET_KERNELS_DEBUG", "0") not in ("", "0"):
        return load("kernels_debug")
    return load("kernels")


def debug_bounds(clear: bool = True) -> dict:
    """What the debug kernel library recorded since the last clear: {"code", "index", "limit", "skipped"}; code 0 = nothing
    (101 KV-cache position, 102 routed expert id). Raises when the loaded library is the release build."""
    k = kernels()
    if not k.pk_debug_bounds_enabled():
        raise RuntimeError("the release kernel library is loaded: set POCKET_KERNELS_DEBUG=1 before the first op")
    out = (ctypes.c_uint * 4)()
    if k.pk_debug_bounds_read(out) != 0:
        raise RuntimeError("pk_debug_bounds_read failed")
    if clear and k.pk_debug_bounds_clear() != 0:
        raise RuntimeError("pk_debug_bounds_clear failed")
    return {"code": int(out[0]), "index": ctypes.c_int32(out[1]).value, "limit": int(out[2]), "skipped": int(out[3])}


def engine() -> ctypes.CDLL:
    return load("engine")


def cpu() -> ctypes.CDLL:
    return load("cpu")


def loaded_library_paths() -> list[str]:
    """Paths of the native libraries this process actually mapped (from /proc/self/maps)."""
    out = set()
    try:
        with open("/proc/self/maps") as f:
            for line in f:
                if "libpocket_" in line:
                    out.add(line.split()[-1])
    except OSError:
        pass
    return sorted(out)
