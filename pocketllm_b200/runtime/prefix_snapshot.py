"""Prefix snapshot cache: reuse of model state across requests that share a prompt prefix.

Prompts are hashed in blocks of 256 tokens with a rolling blake2b chain, so a lookup walks
the chain of a new prompt and finds the deepest stored snapshot whose chain hash matches.
Entries are kept in LRU order (8 by default). The state itself is opaque to the cache: the
model hands over whatever `capture` should keep (for the hybrid decoder: DeltaNet states and
conv tails; KV rows are position indexed and only need the length).
Same contract as the reference's `PrefixSnapshotCache` (src/runtime/prefix_snapshot.py) and
the Qwen engine's snapshot policy (cpp_engine/src/qwen_engine.cpp:1979-2149).
"""
from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict
from dataclasses import dataclass
from typing import Any, Callable, Sequence

BLOCK = 256


def chain_hashes(tokens: Sequence[int], block: int = BLOCK) -> list[bytes]:
    """Hash of every full block prefix: out[i] covers tokens[: (i + 1) * block]."""
    out, prev = [], b""
    for i in range(0, len(tokens) - len(tokens) % block, block):
        h = hashlib.blake2b(prev, digest_size=16)
        h.update(struct.pack(f"<{block}q", *tokens[i:i + block]))
        prev = h.digest()
        out.append(prev)
    return out


@dataclass
class Snapshot:
    length: int          # tokens covered (a multiple of the block size)
    state: Any
    result: Any = None   # optional: model output at exactly this prefix


class PrefixSnapshotCache:
    def __init__(self, capacity: int = 8, block: int = BLOCK, on_evict: Callable[[Snapshot], None] | None = None):
        self.capacity, self.block, self.on_evict = capacity, block, on_evict
        self._lru: "OrderedDict[bytes, Snapshot]" = OrderedDict()
        self.stats = {"lookups": 0, "hits": 0, "reused_tokens": 0, "captures": 0, "evictions": 0}

    def __len__(self) -> int:
        return len(self._lru)

    def lookup_hint(self, tokens: Sequence[int]) -> int:
        """Length of the deepest cached prefix of `tokens` (0 when none); does not touch LRU order."""
        best = 0
        for i, h in enumerate(chain_hashes(tokens, self.block)):
            if h in self._lru:
                best = (i + 1) * self.block
        return best

    def restore(self, tokens: Sequence[int], leave_at_least: int = 1) -> Snapshot | None:
        """Deepest snapshot that is a prefix of `tokens` and leaves at least `leave_at_least`
        tokens to compute (a model needs a forward to produce logits)."""
        self.stats["lookups"] += 1
        hit = None
        for i, h in enumerate(chain_hashes(tokens, self.block)):
            n = (i + 1) * self.block
            if h in self._lru and len(tokens) - n >= leave_at_least:
                hit = h
        if hit is None:
            return None
        self._lru.move_to_end(hit)
        snap = self._lru[hit]
        self.stats["hits"] += 1
        self.stats["reused_tokens"] += snap.length
        return snap

    def capture(self, tokens: Sequence[int], state: Any, result: Any = None) -> bool:
        """Store `state` for the prefix tokens[:n], n = the largest block multiple <= len(tokens)
        (the caller captures at block boundaries while it prefills). Returns False when the
        prompt is shorter than one block."""
        hashes = chain_hashes(tokens, self.block)
        if not hashes:
            return False
        key = hashes[-1]
        if key in self._lru:
            old = self._lru.pop(key)
            if self.on_evict:
                self.on_evict(old)
        self._lru[key] = Snapshot(len(hashes) * self.block, state, result)
        self.stats["captures"] += 1
        while len(self._lru) > self.capacity:
            _, ev = self._lru.popitem(last=False)
            self.stats["evictions"] += 1
            if self.on_evict:
                self.on_evict(ev)
        return True

    def clear(self) -> None:
        while self._lru:
            _, ev = self._lru.popitem(last=False)
            if self.on_evict:
                self.on_evict(ev)
