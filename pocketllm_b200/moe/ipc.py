"""Shared-memory channel between model ranks and a CPU expert server process, and a shared read-only weight arena.

Channel layout (one per client rank; reference: src/components/moe/ipc.py:1-130): an int64 header
`[req_seq, resp_seq, layer_id, tokens, stop, ready]` followed by an input area [max_tokens, hidden] fp32 and an output
area of the same size. The client writes the input, then `layer_id`, `tokens`, then bumps `req_seq`; the server answers
by writing the output and setting `resp_seq = req_seq`. Both sides poll with `time.sleep(0)` and a deadline: a stopped or
dead peer turns into an exception, never into an endless wait.

Weight arena (reference: src/components/moe/shared_weights.py): named tensors packed into one shared-memory segment
with a JSON directory, created once and attached read-only by any number of processes; `wait_until_ready` bounds the
attach.
"""
from __future__ import annotations

import json
import time
from multiprocessing import shared_memory

import numpy as np
import torch

_HDR = 6                     # int64 words
REQ, RESP, LAYER, TOKENS, STOP, READY = range(_HDR)


class ServerStopped(RuntimeError):
    pass


def _unregister(shm: shared_memory.SharedMemory) -> None:
    """Attached (not created) segments must not be unlinked by this process's resource tracker at exit."""
    try:
        from multiprocessing import resource_tracker
        resource_tracker.unregister(shm._name, "shared_memory")
    except Exception:
        pass


class MoEChannel:
    def __init__(self, name: str, max_tokens: int, hidden: int, create: bool):
        self.name, self.max_tokens, self.hidden = name, max_tokens, hidden
        nbytes = _HDR * 8 + 2 * max_tokens * hidden * 4
        if create:
            self.shm = shared_memory.SharedMemory(name=name, create=True, size=nbytes)
            self.shm.buf[:nbytes] = bytes(nbytes)
        else:
            self.shm = shared_memory.SharedMemory(name=name)
            _unregister(self.shm)
        self.created = create
        self.hdr = np.ndarray((_HDR,), dtype=np.int64, buffer=self.shm.buf)
        off = _HDR * 8
        self.inp = np.ndarray((max_tokens, hidden), dtype=np.float32, buffer=self.shm.buf, offset=off)
        self.out = np.ndarray((max_tokens, hidden), dtype=np.float32, buffer=self.shm.buf, offset=off + max_tokens * hidden * 4)

    # -- client ------------------------------------------------------------------------
    def wait_until_ready(self, timeout_s: float = 600.0) -> None:
        deadline = time.monotonic() + timeout_s
        while self.hdr[READY] == 0:
            if time.monotonic() > deadline:
                raise TimeoutError(f"CPU MoE server did not become ready within {timeout_s:.0f} s")
            time.sleep(0.002)

    def request(self, layer: int, x: torch.Tensor, timeout_s: float = 120.0) -> torch.Tensor:
        T = x.shape[0]
        if T > self.max_tokens or x.shape[1] != self.hidden:
            raise ValueError("request does not fit the channel")
        if self.hdr[STOP]:
            raise ServerStopped("CPU MoE server stopped")
        self.inp[:T] = x.detach().to("cpu", torch.float32).numpy()
        self.hdr[LAYER], self.hdr[TOKENS] = layer, T
        seq = int(self.hdr[REQ]) + 1
        self.hdr[REQ] = seq                                # publish last
        deadline = time.monotonic() + timeout_s
        while self.hdr[RESP] != seq:
            if self.hdr[STOP]:
                raise ServerStopped("CPU MoE server stopped")
            if time.monotonic() > deadline:
                raise TimeoutError(f"CPU MoE server did not answer request {seq} within {timeout_s:.0f} s")
            time.sleep(0)
        return torch.from_numpy(self.out[:T].copy())

    # -- server ------------------------------------------------------------------------
    def poll(self, last_seq: int) -> tuple[int, int, np.ndarray] | None:
        seq = int(self.hdr[REQ])
        if seq == last_seq:
            return None
        T = int(self.hdr[TOKENS])
        return seq, int(self.hdr[LAYER]), self.inp[:T]

    def respond(self, seq: int, y: np.ndarray) -> None:
        self.out[: y.shape[0]] = y
        self.hdr[RESP] = seq

    def close(self, unlink: bool | None = None) -> None:
        del self.hdr, self.inp, self.out
        self.shm.close()
        if self.created if unlink is None else unlink:
            try:
                self.shm.unlink()
            except FileNotFoundError:
                pass


class SharedWeightArena:
    """One shared-memory segment holding named uint8 / fp32 tensors; `create` packs, `attach` maps them without a copy."""

    def __init__(self, shm: shared_memory.SharedMemory, directory: dict, created: bool):
        self.shm, self.directory, self.created = shm, directory, created

    @classmethod
    def create(cls, name: str, tensors: dict[str, torch.Tensor]) -> "SharedWeightArena":
        directory, off = {}, 0
        for k, t in tensors.items():
            n = t.numel() * t.element_size()
            directory[k] = {"offset": off, "shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", "")}
            off += (n + 63) // 64 * 64
        blob = json.dumps(directory).encode()
        head = 16 + (len(blob) + 63) // 64 * 64
        shm = shared_memory.SharedMemory(name=name, create=True, size=head + max(off, 64))
        shm.buf[8:16] = len(blob).to_bytes(8, "little")
        shm.buf[16:16 + len(blob)] = blob
        for k, t in tensors.items():
            d = directory[k]
            raw = t.detach().contiguous().view(torch.uint8).numpy().reshape(-1)
            shm.buf[head + d["offset"]: head + d["offset"] + raw.size] = raw.tobytes()
        shm.buf[0:8] = (1).to_bytes(8, "little")                    # ready flag last
        return cls(shm, directory, True)

    @classmethod
    def attach(cls, name: str, timeout_s: float = 600.0) -> "SharedWeightArena":
        deadline = time.monotonic() + timeout_s
        while True:
            try:
                shm = shared_memory.SharedMemory(name=name)
                if int.from_bytes(shm.buf[0:8], "little") == 1:
                    break
                shm.close()
            except FileNotFoundError:
                pass
            if time.monotonic() > deadline:
                raise TimeoutError(f"shared weight arena {name!r} was not ready within {timeout_s:.0f} s")
            time.sleep(0.01)
        _unregister(shm)
        n = int.from_bytes(shm.buf[8:16], "little")
        return cls(shm, json.loads(bytes(shm.buf[16:16 + n]).decode()), False)

    def tensor(self, name: str) -> torch.Tensor:
        d = self.directory[name]
        n = int.from_bytes(self.shm.buf[8:16], "little")
        head = 16 + (n + 63) // 64 * 64
        dt = getattr(torch, d["dtype"])
        count = int(np.prod(d["shape"])) if d["shape"] else 1
        arr = np.frombuffer(self.shm.buf, dtype=np.uint8, count=count * torch.empty(0, dtype=dt).element_size(), offset=head + d["offset"])
        return torch.from_numpy(arr).view(dt).reshape(d["shape"])

    def close(self) -> None:
        """Unmap (and remove, for the creator). Tensors handed out by `tensor()` alias the mapping: while any of them
        is alive the mapping stays until they are collected; the name is removed right away."""
        try:
            self.shm.close()
        except BufferError:
            pass
        if self.created:
            try:
                self.shm.unlink()
            except FileNotFoundError:
                pass
