"""Host-staged routed experts: every expert of a layer sits in pinned host memory in its stored (quantised) form, a
device slab holds a few of them, and the experts a step needs are copied in on a side stream while an LRU policy
picks the slots to overwrite. For checkpoints whose experts do not fit in HBM next to everything else.

Roles in the reference: `GPUPrefillMoEBackend` with its pinned workspaces, copy stream, hot-expert cache and slab
budget (src/components/moe/gpu_prefill_backend.py:11-39,41-103,105-), `MiniMaxM2DeviceResidentCache`
(src/models/minimax_m2/moe_runtime.py:191-339), and the native `DeviceFp4ActiveArena` / `GgufPinnedStagingRing`
(cpp_engine/src/dsv4_engine.cpp:1432-1569).
"""
from __future__ import annotations

from collections import OrderedDict

import torch


class LRUSlots:
    """Which expert occupies which slot. `assign(needed)` returns (slot of every needed expert, list of (expert, slot)
    copies to make); experts of the current request are never evicted for one another."""

    def __init__(self, slots: int):
        self.n = slots
        self.where: "OrderedDict[int, int]" = OrderedDict()          # expert -> slot, least recently used first
        self.free = list(range(slots - 1, -1, -1))
        self.stats = {"hits": 0, "misses": 0, "evictions": 0}

    def assign(self, needed: list[int]) -> tuple[dict[int, int], list[tuple[int, int]]]:
        uniq = list(dict.fromkeys(int(e) for e in needed))
        if len(uniq) > self.n:
            raise ValueError(f"{len(uniq)} distinct experts do not fit in {self.n} slots; split the step into waves")
        copies = []
        for e in uniq:
            if e in self.where:
                self.where.move_to_end(e)
                self.stats["hits"] += 1
        for e in uniq:
            if e in self.where:
                continue
            self.stats["misses"] += 1
            if self.free:
                slot = self.free.pop()
            else:
                victim = next(v for v in self.where if v not in uniq)        # oldest resident that this step does not need
                slot = self.where.pop(victim)
                self.stats["evictions"] += 1
            self.where[e] = slot
            copies.append((e, slot))
        return {e: self.where[e] for e in uniq}, copies


def slots_for_budget(budget_bytes: int, per_expert_bytes: int, n_layers: int, n_experts: int, top_k: int) -> int | None:
    """Device slots per layer that `budget_bytes` of expert memory allow (every MoE layer gets the same number): None when
    all experts fit (no staging needed); never fewer than `top_k + 1`, so that one token's experts are resident
    together and one slot is free for a prefetch. Reference counterpart: the per-GPU expert budget of
    src/runtime/generation.py (`--gpu-memory-gib`) and src/moe/planning.py."""
    if per_expert_bytes <= 0 or n_layers <= 0:
        raise ValueError("per_expert_bytes and n_layers must be positive")
    fit = int(budget_bytes // (per_expert_bytes * n_layers))
    if fit >= n_experts:
        return None
    return max(min(top_k + 1, n_experts), fit)


def waves(ids: torch.Tensor, slots: int) -> list[tuple[int, int]]:
    """Split rows [0, T) of routed ids [T, k] into consecutive ranges whose distinct experts fit into `slots`."""
    out, start, seen = [], 0, set()
    rows = ids.tolist()
    for t, row in enumerate(rows):
        if len(set(row)) > slots:
            raise ValueError("one token routes to more experts than there are slots")
        if len(seen | set(row)) > slots:
            out.append((start, t))
            start, seen = t, set()
        seen |= set(row)
    out.append((start, len(rows)))
    return out


class ExpertStagingCache:
    def __init__(self, host: dict[str, torch.Tensor], slots: int, device: str | torch.device = "cuda"):
        """host[name]: uint8 [E, bytes_per_expert] (moved to pinned memory here); one device slab [slots, bytes] per name."""
        self.device = torch.device(device)
        self.host = {k: (v if v.is_pinned() else v.contiguous().pin_memory()) for k, v in host.items()}
        self.n_experts = next(iter(self.host.values())).shape[0]
        self.slab = {k: torch.empty(slots, v.shape[1], dtype=torch.uint8, device=self.device) for k, v in self.host.items()}
        self.lru = LRUSlots(slots)
        self.copy_stream = torch.cuda.Stream(device=self.device)
        self.table = torch.full((self.n_experts,), -1, dtype=torch.int32, device=self.device)
        self.bytes_staged = 0
        self._pending: torch.cuda.Event | None = None

    def _stage(self, copies: list[tuple[int, int]]) -> None:
        if not copies:
            return
        # the slots being overwritten may still be read by kernels already queued on the compute stream
        self.copy_stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.copy_stream):
            for e, slot in copies:
                for k, h in self.host.items():
                    self.slab[k][slot].copy_(h[e], non_blocking=True)
                    self.bytes_staged += h.shape[1]
            ev = torch.cuda.Event()
            ev.record(self.copy_stream)
        self._pending = ev

    def prefetch(self, experts: list[int]) -> None:
        """Start copying experts that a later step is predicted to need; the compute stream does not wait."""
        fit = list(dict.fromkeys(int(e) for e in experts))[: self.lru.n]
        _, copies = self.lru.assign(fit)
        self._stage(copies)
        self._update_table()

    def _update_table(self) -> None:
        t = torch.full((self.n_experts,), -1, dtype=torch.int32)
        for e, s in self.lru.where.items():
            t[e] = s
        self.table.copy_(t, non_blocking=False)

    def ensure(self, experts: list[int]) -> None:
        """Make `experts` resident and make the current stream wait for their copies."""
        _, copies = self.lru.assign(experts)
        self._stage(copies)
        if copies:
            self._update_table()
        if self._pending is not None:
            torch.cuda.current_stream(self.device).wait_event(self._pending)
            self._pending = None

    def remap(self, ids: torch.Tensor) -> torch.Tensor:
        """Expert ids [T, k] -> slot ids (int32)."""
        return self.table[ids.long()].contiguous()


def staged_moe_forward(cache: ExpertStagingCache, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, type13: str, type2: str,
                       inter: int, *, limit: float = 0.0, w13: str = "w13", w2: str = "w2") -> torch.Tensor:
    """Routed experts through the staging cache: y [T, H] fp32. Steps whose distinct experts exceed the slots run in waves."""
    from ..ops import gguf_ops as go
    T, H = x.shape
    y = torch.zeros(T, H, device=x.device, dtype=torch.float32)
    ids_host = ids.cpu()
    for lo, hi in waves(ids_host, cache.lru.n):
        cache.ensure(ids_host[lo:hi].flatten().tolist())
        slot_ids = cache.remap(ids[lo:hi])
        routes = go.group_routes(slot_ids, weights[lo:hi].contiguous(), cache.lru.n)
        seg, tok, rw = routes
        go.gguf_moe_forward(x[lo:hi].contiguous(), cache.slab[w13].view(-1), cache.slab[w2].view(-1), type13, type2, cache.lru.n, inter, seg, tok, rw,
                            limit=limit, out=y[lo:hi], routes=routes)
    return y
