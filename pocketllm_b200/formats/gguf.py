"""GGUF v3 container: reader (mmap), writer, multi-shard bundles.

Layout: magic `GGUF`, version, tensor count, metadata count; typed metadata key/values;
tensor table (name, dims innermost-first, ggml type, offset); padding to
`general.alignment` (32 by default); tensor data. Multi-shard files are named
`<stem>-0000i-of-0000n.gguf`.

Covers the reference's readers (src/loader/gguf/reader.py:27-57, bundle.py,
cpp_engine/src/gguf_reader.cpp) and adds what the reference lacks: a writer, so that
random-init checkpoints with REAL quantised payloads can be produced for tests and
benchmarks (the reference's test helper writes zero payloads, tests/gguf_test_utils.py:52-107).
"""
from __future__ import annotations

import mmap
import os
import re
import struct
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Iterable, Mapping

import numpy as np

GGUF_MAGIC = 0x46554747  # "GGUF" little endian
GGUF_VERSION = 3
DEFAULT_ALIGNMENT = 32

# ggml type id -> (name, weights per block, bytes per block)
GGML_TYPES: dict[int, tuple[str, int, int]] = {
    0: ("f32", 1, 4), 1: ("f16", 1, 2), 2: ("q4_0", 32, 18), 3: ("q4_1", 32, 20), 6: ("q5_0", 32, 22),
    7: ("q5_1", 32, 24), 8: ("q8_0", 32, 34), 9: ("q8_1", 32, 36), 10: ("q2_k", 256, 84), 11: ("q3_k", 256, 110),
    12: ("q4_k", 256, 144), 13: ("q5_k", 256, 176), 14: ("q6_k", 256, 210), 15: ("q8_k", 256, 292),
    16: ("iq2_xxs", 256, 66), 17: ("iq2_xs", 256, 74), 18: ("iq3_xxs", 256, 98), 19: ("iq1_s", 256, 50),
    20: ("iq4_nl", 32, 18), 21: ("iq3_s", 256, 110), 22: ("iq2_s", 256, 82), 23: ("iq4_xs", 256, 136),
    24: ("i8", 1, 1), 25: ("i16", 1, 2), 26: ("i32", 1, 4), 27: ("i64", 1, 8), 28: ("f64", 1, 8),
    29: ("iq1_m", 256, 56), 30: ("bf16", 1, 2),
}
GGML_TYPE_IDS = {name: tid for tid, (name, _, _) in GGML_TYPES.items()}

# metadata value types
T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)
_SCALAR_FMT = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f", T_BOOL: "<?",
               T_U64: "<Q", T_I64: "<q", T_F64: "<d"}


def tensor_nbytes(type_id: int, shape: Iterable[int]) -> int:
    """Bytes of a tensor with logical `shape` (row-major, last dim quantised in blocks)."""
    name, qk, bs = GGML_TYPES[type_id]
    shape = list(shape)
    n = int(np.prod(shape)) if shape else 1
    if shape and shape[-1] % qk != 0:
        raise ValueError(f"last dim {shape[-1]} is not a multiple of the {name} block ({qk})")
    return n // qk * bs


@dataclass
class GGUFTensorInfo:
    name: str
    shape: tuple[int, ...]   # logical shape, outermost first (the file stores it reversed)
    type_id: int
    offset: int              # relative to the data section
    nbytes: int

    @property
    def type_name(self) -> str:
        return GGML_TYPES[self.type_id][0]


class _Cursor:
    def __init__(self, buf, pos: int = 0):
        self.buf, self.pos = buf, pos

    def take(self, fmt: str):
        v = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += struct.calcsize(fmt)
        return v[0] if len(v) == 1 else v

    def string(self) -> str:
        n = self.take("<Q")
        if n > len(self.buf) - self.pos:
            raise ValueError("gguf: string length exceeds the file")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, vt: int):
        if vt in _SCALAR_FMT:
            return self.take(_SCALAR_FMT[vt])
        if vt == T_STR:
            return self.string()
        if vt == T_ARR:
            it = self.take("<I")
            n = self.take("<Q")
            if it in _SCALAR_FMT and it != T_BOOL:
                dt = np.dtype(_SCALAR_FMT[it])
                arr = np.frombuffer(self.buf, dtype=dt, count=n, offset=self.pos)
                self.pos += n * dt.itemsize
                return arr.tolist()
            return [self.value(it) for _ in range(n)]
        raise ValueError(f"gguf: unknown metadata type {vt}")


class GGUFFile:
    """One GGUF file, memory mapped. `metadata` is a dict, `tensors` maps names to infos."""

    def __init__(self, path: str | os.PathLike):
        self.path = str(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        c = _Cursor(self._mm)
        if c.take("<I") != GGUF_MAGIC:
            raise ValueError(f"{self.path}: not a GGUF file")
        self.version = c.take("<I")
        if self.version not in (2, 3):
            raise ValueError(f"{self.path}: unsupported GGUF version {self.version}")
        n_tensors, n_kv = c.take("<Q"), c.take("<Q")
        self.metadata: dict[str, Any] = {}
        self.metadata_types: dict[str, int] = {}
        for _ in range(n_kv):
            key = c.string()
            vt = c.take("<I")
            self.metadata[key] = c.value(vt)
            self.metadata_types[key] = vt
        self.alignment = int(self.metadata.get("general.alignment", DEFAULT_ALIGNMENT))
        self.tensors: dict[str, GGUFTensorInfo] = {}
        for _ in range(n_tensors):
            name = c.string()
            nd = c.take("<I")
            dims = [c.take("<Q") for _ in range(nd)]
            tid = c.take("<I")
            off = c.take("<Q")
            if tid not in GGML_TYPES:
                raise ValueError(f"{self.path}: tensor {name} has unknown ggml type {tid}")
            shape = tuple(reversed(dims))
            self.tensors[name] = GGUFTensorInfo(name, shape, tid, off, tensor_nbytes(tid, shape))
        self.data_offset = (c.pos + self.alignment - 1) // self.alignment * self.alignment
        for t in self.tensors.values():
            if self.data_offset + t.offset + t.nbytes > len(self._mm):
                raise ValueError(f"{self.path}: tensor {t.name} runs past the end of the file")

    def raw(self, name: str) -> np.ndarray:
        """The tensor's bytes as a uint8 view of the mapping (no copy)."""
        t = self.tensors[name]
        return np.frombuffer(self._mm, dtype=np.uint8, count=t.nbytes, offset=self.data_offset + t.offset)

    def blocks(self, name: str) -> np.ndarray:
        """Raw blocks as uint8 [rows..., blocks_per_row, bytes_per_block]."""
        t = self.tensors[name]
        _, qk, bs = GGML_TYPES[t.type_id]
        return self.raw(name).reshape(*t.shape[:-1], t.shape[-1] // qk, bs)

    def architecture(self) -> str:
        return str(self.metadata.get("general.architecture", ""))

    def close(self) -> None:
        try:
            self._mm.close()
        except BufferError:
            pass  # numpy views of the mapping are still alive; the OS frees it with them
        self._f.close()


_SHARD_RE = re.compile(r"^(?P<stem>.*)-(?P<idx>\d{5})-of-(?P<n>\d{5})\.gguf$")


def shard_paths(path: str | os.PathLike) -> list[Path]:
    """All shards of the bundle that `path` belongs to (or just `path`)."""
    p = Path(path)
    m = _SHARD_RE.match(p.name)
    if not m:
        return [p]
    n = int(m.group("n"))
    out = [p.with_name(f"{m.group('stem')}-{i:05d}-of-{n:05d}.gguf") for i in range(1, n + 1)]
    missing = [str(q) for q in out if not q.exists()]
    if missing:
        raise FileNotFoundError(f"missing GGUF shards: {missing}")
    return out


class GGUFBundle:
    """A single- or multi-shard GGUF model: metadata of the first shard, tensors of all."""

    def __init__(self, path: str | os.PathLike):
        self.files = [GGUFFile(p) for p in shard_paths(path)]
        self.metadata = self.files[0].metadata
        self._where: dict[str, GGUFFile] = {}
        for f in self.files:
            for name in f.tensors:
                if name in self._where:
                    raise ValueError(f"tensor {name} appears in two shards")
                self._where[name] = f

    @property
    def tensors(self) -> dict[str, GGUFTensorInfo]:
        return {n: f.tensors[n] for n, f in self._where.items()}

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def info(self, name: str) -> GGUFTensorInfo:
        return self._where[name].tensors[name]

    def raw(self, name: str) -> np.ndarray:
        return self._where[name].raw(name)

    def blocks(self, name: str) -> np.ndarray:
        return self._where[name].blocks(name)

    def architecture(self) -> str:
        return self.files[0].architecture()

    def total_bytes(self) -> int:
        return sum(t.nbytes for t in self.tensors.values())

    def close(self) -> None:
        for f in self.files:
            f.close()


# --------------------------------------------------------------------------------------
# writer

def _infer_type(v: Any) -> int:
    if isinstance(v, bool):
        return T_BOOL
    if isinstance(v, int):
        return T_U32 if 0 <= v < 2 ** 32 else T_I64
    if isinstance(v, float):
        return T_F32
    if isinstance(v, str):
        return T_STR
    if isinstance(v, (list, tuple)):
        return T_ARR
    raise TypeError(f"gguf: cannot infer the metadata type of {type(v)}")


def _pack_string(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _pack_value(v: Any, vt: int) -> bytes:
    if vt in _SCALAR_FMT:
        return struct.pack(_SCALAR_FMT[vt], v)
    if vt == T_STR:
        return _pack_string(v)
    if vt == T_ARR:
        items = list(v)
        it = _infer_type(items[0]) if items else T_U32
        if it == T_U32 and any(isinstance(x, int) and x < 0 for x in items):
            it = T_I32
        out = struct.pack("<IQ", it, len(items))
        return out + b"".join(_pack_value(x, it) for x in items)
    raise TypeError(f"gguf: unknown metadata type {vt}")


@dataclass
class GGUFWriter:
    """Collect metadata and tensors, then `write(path)`.

    `add_tensor(name, data, type_name, shape)`: `data` is the raw payload (uint8 blocks for
    quantised types, or an ndarray of the matching dtype for f32/f16/i32...)."""
    metadata: dict[str, tuple[Any, int]] = field(default_factory=dict)
    tensors: list[tuple[str, tuple[int, ...], int, np.ndarray]] = field(default_factory=list)
    alignment: int = DEFAULT_ALIGNMENT

    def add_meta(self, key: str, value: Any, vtype: int | None = None) -> None:
        self.metadata[key] = (value, _infer_type(value) if vtype is None else vtype)

    def add_tensor(self, name: str, data: np.ndarray, type_name: str, shape: Iterable[int] | None = None) -> None:
        tid = GGML_TYPE_IDS[type_name]
        raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        shape = tuple(int(s) for s in (shape if shape is not None else data.shape))
        if raw.size != tensor_nbytes(tid, shape):
            raise ValueError(f"{name}: payload has {raw.size} bytes, {type_name}{list(shape)} needs {tensor_nbytes(tid, shape)}")
        self.tensors.append((name, shape, tid, raw))

    def write(self, path: str | os.PathLike) -> None:
        head = struct.pack("<IIQQ", GGUF_MAGIC, GGUF_VERSION, len(self.tensors), len(self.metadata) + 1)
        meta = dict(self.metadata)
        meta["general.alignment"] = (self.alignment, T_U32)
        for k, (v, vt) in meta.items():
            head += _pack_string(k) + struct.pack("<I", vt) + _pack_value(v, vt)
        off = 0
        offsets = []
        for name, shape, tid, raw in self.tensors:
            offsets.append(off)
            off = (off + raw.size + self.alignment - 1) // self.alignment * self.alignment
        for (name, shape, tid, raw), o in zip(self.tensors, offsets):
            head += _pack_string(name) + struct.pack("<I", len(shape))
            head += b"".join(struct.pack("<Q", d) for d in reversed(shape))
            head += struct.pack("<IQ", tid, o)
        pad = (-len(head)) % self.alignment
        with open(path, "wb") as f:
            f.write(head + b"\0" * pad)
            for (name, shape, tid, raw), o in zip(self.tensors, offsets):
                f.write(raw.tobytes())
                f.write(b"\0" * ((-raw.size) % self.alignment))
