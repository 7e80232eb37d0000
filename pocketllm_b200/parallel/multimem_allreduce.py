"""All-reduce with the sum done inside NVSwitch (`csrc/comm/multimem_allreduce.cu`): every rank writes its data once
into its own symmetric buffer and reads the sum of all ranks' buffers through a multicast address
(`multimem.ld_reduce`); large payloads are reduced slice by slice and broadcast with `multimem.st`.

The symmetric buffer, its peer mappings and the multicast mapping come from `torch.distributed._symmetric_memory`
(driver multicast objects bound to every rank's allocation); the kernel and its bounded waits are this package's.
`MulticastUnavailable` is raised where the machine or the driver offers no multicast (no NVSwitch, one GPU): callers
keep the unicast `PeerAllReduce` then. Same contract as `PeerAllReduce`: fp32, contiguous, `numel <= capacity`, a wait
that runs out sets a status word which `check()` turns into an exception.

Never use this class in a test that lets a rank die or leave early: a process that exits while its memory is bound to
a multicast object can raise NVLink errors on the surviving ranks' GPUs. Failure-handling tests use the unicast path."""
from __future__ import annotations

from ctypes import c_int, c_size_t, c_uint, c_void_p

import torch
import torch.distributed as dist

from ..ops import lib as _lib

TWO_SHOT_MIN_FLOATS = 64 * 1024     # from 256 KiB on, each element should cross every link once, not world times


class MulticastUnavailable(RuntimeError):
    pass


class MultimemAllReduce:
    def __init__(self, capacity: int, group=None, timeout_us: int = 2_000_000):
        """capacity: floats per call (rounded up to a multiple of 4)."""
        import torch.distributed._symmetric_memory as symm_mem
        self.K = _lib.kernels()
        self.K.pk_mm_buffer_bytes.restype = c_size_t
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.capacity = (capacity + 3) // 4 * 4
        self.timeout_us = timeout_us
        dev = torch.device("cuda", torch.cuda.current_device())
        nbytes = int(self.K.pk_mm_buffer_bytes(c_int(self.world), c_size_t(self.capacity)))
        self.buf = symm_mem.empty((nbytes + 15) // 16 * 16, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        self._hdl = symm_mem.rendezvous(self.buf, self.group)
        mc = int(getattr(self._hdl, "multicast_ptr", 0) or 0)
        if mc == 0:
            raise MulticastUnavailable("no multicast mapping for symmetric memory on this machine")
        off = int(getattr(self._hdl, "offset", 0) or 0)
        ptrs = [int(p) + off for p in self._hdl.buffer_ptrs]
        if ptrs[self.rank] != self.buf.data_ptr():
            raise MulticastUnavailable("symmetric memory handle does not describe the buffer that was allocated")
        self._ptrs = (c_void_p * self.world)(*ptrs)
        self._mc = c_void_p(mc + off)
        self._sm = torch.cuda.get_device_properties(dev).multi_processor_count
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def all_reduce(self, x: torch.Tensor, out: torch.Tensor | None = None, two_shot: bool | None = None) -> torch.Tensor:
        """Sum of `x` (fp32, contiguous, numel <= capacity) over the group; in place unless `out` is given."""
        if x.dtype != torch.float32 or not x.is_contiguous():
            raise ValueError("multimem all-reduce takes contiguous fp32 tensors")
        out = x if out is None else out
        if two_shot is None:
            two_shot = x.numel() >= TWO_SHOT_MIN_FLOATS
        st = self.K.pk_mm_allreduce(self._ptrs, self._mc, c_int(self.world), c_int(self.rank), c_size_t(self.capacity), c_void_p(x.data_ptr()),
                                    c_void_p(out.data_ptr()), c_size_t(x.numel()), c_int(int(two_shot)), c_uint(self.timeout_us), c_int(self._sm),
                                    c_void_p(torch.cuda.current_stream().cuda_stream))
        if st != 0:
            raise RuntimeError(f"pk_mm_allreduce: status {st}")
        return out

    def status(self, clear: bool = False) -> int:
        return int(self.K.pk_mm_status(c_void_p(self.buf.data_ptr()), c_int(self.world), c_size_t(self.capacity), c_int(int(clear))))

    def check(self) -> None:
        s = self.status(clear=True)
        if s != 0:
            raise TimeoutError(f"multimem all-reduce gave up waiting (status {s}); a rank is missing or late")
