"""All-reduce over peer memory for Python-level runtimes (expert-parallel combines, small tensor-parallel
reductions): one kernel per rank pushes its data into every peer, signals, waits and sums
(`csrc/comm/peer_allreduce.cu`). Arenas are plain device allocations shared through CUDA IPC handles that
travel over the `torch.distributed` group. Falls back to nothing: a wait that runs out sets a status word
which `check()` turns into an exception, and the caller decides (the models fall back to NCCL)."""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_size_t, c_uint, c_void_p

import torch
import torch.distributed as dist

from ..ops import lib as _lib
from .tp import exchange_handles


class PeerAllReduce:
    def __init__(self, capacity: int, group=None, timeout_us: int = 2_000_000, _solo_world: int | None = None):
        """capacity: floats per call (rounded up to a multiple of 4). `_solo_world` builds a context whose peers
        are this rank's own arena and never answer: only for testing the bounded wait on one GPU."""
        self.K, self.E = _lib.kernels(), _lib.engine()
        self.K.pk_par_arena_bytes.restype = c_size_t
        self.E.pk_ipc_open.restype = c_void_p
        self.group = group
        self.capacity = (capacity + 3) // 4 * 4
        self.timeout_us = timeout_us
        self.world = _solo_world or dist.get_world_size(group)
        self.rank = 0 if _solo_world else dist.get_rank(group)
        self.K.pk_par_alloc.restype = c_void_p
        torch.cuda.current_device()                      # make sure the context of this rank's device is current
        self.arena = self.K.pk_par_alloc(c_int(self.world), c_size_t(self.capacity))
        if not self.arena:
            raise RuntimeError("could not allocate the peer all-reduce arena")
        self._opened: list[int] = []
        ptrs = [0] * self.world
        ptrs[self.rank] = self.arena
        if _solo_world:
            ptrs = [self.arena] * self.world
        elif self.world > 1:
            handle = ctypes.create_string_buffer(64)
            if self.E.pk_ipc_export(c_void_p(self.arena), handle) != 0:
                raise RuntimeError("cudaIpcGetMemHandle failed")
            handles = exchange_handles(handle.raw, group)
            for r, h in enumerate(handles):
                if r == self.rank:
                    continue
                p = self.E.pk_ipc_open(ctypes.c_char_p(h))
                if not p:
                    raise RuntimeError(f"cudaIpcOpenMemHandle failed for rank {r}")
                ptrs[r] = p
                self._opened.append(p)
        self._ptrs = (c_void_p * self.world)(*ptrs)
        self._sm = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        if self.world > 1 and not _solo_world:
            torch.cuda.synchronize()
            dist.barrier(group=group)

    def all_reduce(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Sum of `x` (fp32, contiguous, numel <= capacity) over the group; in place unless `out` is given."""
        if x.dtype != torch.float32 or not x.is_contiguous():
            raise ValueError("peer all-reduce takes contiguous fp32 tensors")
        out = x if out is None else out
        st = self.K.pk_par_allreduce(self._ptrs, c_int(self.world), c_int(self.rank), c_size_t(self.capacity), c_void_p(x.data_ptr()),
                                     c_void_p(out.data_ptr()), c_size_t(x.numel()), c_uint(self.timeout_us), c_int(self._sm),
                                     c_void_p(torch.cuda.current_stream().cuda_stream))
        if st != 0:
            raise RuntimeError(f"pk_par_allreduce: status {st}")
        return out

    def moe_combine(self, ybuf: torch.Tensor, route_w: torch.Tensor, route_pos: torch.Tensor, seg: torch.Tensor, expert_offset: int,
                    local_experts: int, T: int, topk: int, out: torch.Tensor) -> torch.Tensor:
        """MoE combine as peer stores from the per-token reduce: out [T, H] fp32 = sum over ranks of every rank's weighted sum
        of the token's routes through its own experts (ybuf [routes, H] per-route outputs and route_w [routes] in expert
        order, route_pos [T * topk] the sorted position of route (t, k)). One launch per rank: reduce, stores into every
        rank, signal, bounded wait, sum."""
        H = ybuf.shape[1]
        if T * H > self.capacity or out.dtype != torch.float32 or not out.is_contiguous():
            raise ValueError("moe_combine: payload exceeds the arena or the output is not contiguous fp32")
        st = self.K.pk_par_moe_combine(self._ptrs, c_int(self.world), c_int(self.rank), c_size_t(self.capacity), c_void_p(ybuf.data_ptr()),
                                       c_void_p(route_w.data_ptr()), c_void_p(route_pos.data_ptr()), c_void_p(seg.data_ptr()), c_int(expert_offset),
                                       c_int(local_experts), c_int(T), c_int(topk), c_int(H), c_void_p(out.data_ptr()), c_uint(self.timeout_us),
                                       c_int(self._sm), c_void_p(torch.cuda.current_stream().cuda_stream))
        if st != 0:
            raise RuntimeError(f"pk_par_moe_combine: status {st}")
        return out

    def status(self, clear: bool = False) -> int:
        return int(self.K.pk_par_status(c_void_p(self.arena), c_int(self.world), c_size_t(self.capacity), c_int(int(clear))))

    def check(self) -> None:
        s = self.status(clear=True)
        if s != 0:
            raise TimeoutError(f"peer all-reduce gave up waiting (status {s}); a rank is missing or late")

    def close(self) -> None:
        for p in self._opened:
            self.E.pk_ipc_close(c_void_p(p))
        self._opened = []
        if self.arena:
            torch.cuda.synchronize()
            self.K.pk_par_free(c_void_p(self.arena))
            self.arena = None
