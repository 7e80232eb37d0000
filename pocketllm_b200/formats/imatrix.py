"""Importance matrices: per-input-channel sums of squared activations collected while a
model runs, stored as a GGUF file (`<tensor>.in_sum2` f32 vectors and `<tensor>.counts`),
and merged across runs. Format and merge rule of the reference's imatrix tools
(src/loader/gguf/imatrix.py, src/cli/merge_imatrix.py): sums add, counts add.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np

from . import gguf


class IMatrixCollector:
    def __init__(self) -> None:
        self.sum2: dict[str, np.ndarray] = {}
        self.counts: dict[str, int] = {}

    def observe(self, tensor_name: str, activations: np.ndarray) -> None:
        """activations: [rows, in_features] inputs of the linear layer `tensor_name`."""
        a = np.asarray(activations, dtype=np.float32).reshape(-1, activations.shape[-1])
        s = (a * a).sum(0)
        if tensor_name in self.sum2:
            self.sum2[tensor_name] += s
            self.counts[tensor_name] += a.shape[0]
        else:
            self.sum2[tensor_name] = s
            self.counts[tensor_name] = a.shape[0]

    def save(self, path: str | Path, dataset: str = "") -> None:
        w = gguf.GGUFWriter()
        w.add_meta("general.type", "imatrix")
        w.add_meta("imatrix.datasets", [dataset] if dataset else ["unknown"])
        w.add_meta("imatrix.chunk_count", int(max(self.counts.values(), default=0)))
        for name in sorted(self.sum2):
            w.add_tensor(name + ".in_sum2", self.sum2[name].astype(np.float32), "f32")
            w.add_tensor(name + ".counts", np.array([self.counts[name]], dtype=np.float32), "f32")
        w.write(path)


def load(path: str | Path) -> IMatrixCollector:
    f = gguf.GGUFFile(path)
    if f.metadata.get("general.type") != "imatrix":
        raise ValueError(f"{path} is not an imatrix GGUF")
    c = IMatrixCollector()
    for name in f.tensors:
        if name.endswith(".in_sum2"):
            base = name[: -len(".in_sum2")]
            c.sum2[base] = f.raw(name).view(np.float32).copy()
            c.counts[base] = int(f.raw(base + ".counts").view(np.float32)[0])
    return c


def merge(paths: list[str | Path], out: str | Path) -> IMatrixCollector:
    acc = IMatrixCollector()
    for p in paths:
        c = load(p)
        for k, v in c.sum2.items():
            if k in acc.sum2:
                if acc.sum2[k].shape != v.shape:
                    raise ValueError(f"{k}: shapes differ between imatrix files")
                acc.sum2[k] += v
                acc.counts[k] += c.counts[k]
            else:
                acc.sum2[k], acc.counts[k] = v.copy(), c.counts[k]
    acc.save(out, dataset="merged")
    return acc


def importance(c: IMatrixCollector, tensor_name: str) -> np.ndarray:
    """Mean squared activation per input channel (the weighting a quantiser would use)."""
    return c.sum2[tensor_name] / max(c.counts[tensor_name], 1)
