"""Safetensors reader and writer in plain Python + torch (FP8 E4M3 / E8M0 / bf16 aware).

File layout: 8-byte little-endian header length, JSON header
`{name: {"dtype", "shape", "data_offsets"}, "__metadata__": {...}}`, then the raw tensors.
Directory layout: shards plus `model.safetensors.index.json` with a `weight_map`.
Counterpart of the reference's `src/loader/safetensors.py` (index + shard reader); the
reference has no writer, this one exists so that random-init checkpoints of any shape can
be produced in the exact on-disk format.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from pathlib import Path
from typing import Iterable, Mapping

import torch

_DTYPES = {
    "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I8": torch.int8, "U8": torch.uint8,
    "I32": torch.int32, "I64": torch.int64, "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2,
}
if hasattr(torch, "float8_e8m0fnu"):
    _DTYPES["F8_E8M0"] = torch.float8_e8m0fnu
_NAMES = {v: k for k, v in _DTYPES.items()}


def dtype_name(dt: torch.dtype) -> str:
    return _NAMES[dt]


def write_file(path: str | os.PathLike, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] | None = None) -> None:
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    off = 0
    order = list(tensors.keys())
    for name in order:
        t = tensors[name]
        n = t.numel() * t.element_size()
        header[name] = {"dtype": dtype_name(t.dtype), "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")


def write_sharded(directory: str | os.PathLike, tensors: Mapping[str, torch.Tensor], max_shard_bytes: int = 4 << 30,
                  metadata: Mapping[str, str] | None = None) -> list[str]:
    """Write `model-0000i-of-0000n.safetensors` shards and the index file."""
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    shards: list[dict[str, torch.Tensor]] = [{}]
    size = 0
    for name, t in tensors.items():
        n = t.numel() * t.element_size()
        if size and size + n > max_shard_bytes:
            shards.append({})
            size = 0
        shards[-1][name] = t
        size += n
    files, weight_map, total = [], {}, 0
    for i, sh in enumerate(shards):
        fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        write_file(d / fn, sh, metadata)
        files.append(fn)
        for name, t in sh.items():
            weight_map[name] = fn
            total += t.numel() * t.element_size()
    with open(d / "model.safetensors.index.json", "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f)
    return files


class SafetensorsFile:
    """mmap-backed reader of one file; tensors are materialised on access."""

    def __init__(self, path: str | os.PathLike):
        self.path = str(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if hlen > len(self._mm) - 8:
            raise ValueError(f"{self.path}: header length {hlen} exceeds the file")
        header = json.loads(self._mm[8:8 + hlen].decode())
        self.metadata = header.pop("__metadata__", {})
        self.entries = header
        self._base = 8 + hlen

    def keys(self) -> Iterable[str]:
        return self.entries.keys()

    def info(self, name: str) -> tuple[str, list[int]]:
        e = self.entries[name]
        return e["dtype"], list(e["shape"])

    def raw(self, name: str) -> memoryview:
        b, e = self.entries[name]["data_offsets"]
        return memoryview(self._mm)[self._base + b:self._base + e]

    def get(self, name: str) -> torch.Tensor:
        dt, shape = self.info(name)
        buf = bytearray(self.raw(name))
        t = torch.frombuffer(buf, dtype=torch.uint8) if buf else torch.empty(0, dtype=torch.uint8)
        return t.view(_DTYPES[dt]).reshape(shape)

    def close(self) -> None:
        self._mm.close()
        self._f.close()


class SafetensorsModel:
    """A checkpoint directory (index + shards) or a single file."""

    def __init__(self, path: str | os.PathLike):
        p = Path(path)
        files: list[Path]
        if p.is_dir():
            idx = p / "model.safetensors.index.json"
            if idx.exists():
                wm = json.loads(idx.read_text())["weight_map"]
                files = [p / f for f in sorted(set(wm.values()))]
            else:
                files = sorted(p.glob("*.safetensors"))
        else:
            files = [p]
        if not files:
            raise FileNotFoundError(f"no safetensors files under {path}")
        self.files = [SafetensorsFile(f) for f in files]
        self._where = {k: sf for sf in self.files for k in sf.keys()}

    def keys(self) -> list[str]:
        return sorted(self._where)

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def info(self, name: str) -> tuple[str, list[int]]:
        return self._where[name].info(name)

    def get(self, name: str) -> torch.Tensor:
        return self._where[name].get(name)
