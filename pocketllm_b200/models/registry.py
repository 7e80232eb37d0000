"""Architecture registry: `general.architecture` of a GGUF file -> model runtime builder
(reference: src/components/moe/registry.py `detect_spec`)."""
from __future__ import annotations

from typing import Callable

_BUILDERS: dict[str, Callable] = {}


def register(arch: str):
    def deco(fn):
        _BUILDERS[arch] = fn
        return fn
    return deco


def architectures() -> list[str]:
    _load()
    return sorted(_BUILDERS)


def build_runtime(path, architecture: str | None = None, **kw):
    """Open `path`, pick the builder for its architecture and return a token runtime."""
    from ..formats import gguf
    _load()
    arch = architecture or gguf.GGUFFile(gguf.shard_paths(path)[0]).architecture()
    if arch not in _BUILDERS:
        raise KeyError(f"no runtime for GGUF architecture {arch!r}; known: {sorted(_BUILDERS)}")
    return _BUILDERS[arch](path, **kw)


def _load() -> None:
    if _BUILDERS:
        return
    from . import minimax_m2, glm_dsa  # noqa: F401

    @register("minimax-m2")
    def _mm(path, **kw):
        return minimax_m2.MiniMaxM2Model(path, **kw)

    @register("glm-dsa")
    def _glm(path, **kw):
        return glm_dsa.GLMDSAModel(path, **kw)
