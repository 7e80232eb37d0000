"""Native expert staging: LRU decisions equal the Python cache's; the arena brings the right bytes to the device."""
import random

import pytest
import torch

from pocketllm_b200.moe.expert_cache import LRUSlots
from pocketllm_b200.ops import lib

pytestmark = pytest.mark.skipif(not lib.available("engine"), reason="libpocket_engine.so not built")


def test_native_lru_matches_python_lru():
    from pocketllm_b200.moe.native_staging import NativeError, NativeLruSlots
    rnd = random.Random(0)
    py, nat = LRUSlots(6), NativeLruSlots(6)
    for _ in range(300):
        need = [rnd.randrange(20) for _ in range(rnd.randint(1, 6))]
        where, copies = py.assign(need)
        slots, loads = nat.assign(need)
        assert slots == [where[e] for e in need] and loads == copies
    assert nat.stats == py.stats and nat.stats["evictions"] > 0
    with pytest.raises(NativeError):
        nat.assign(list(range(7)))                     # seven distinct keys, six slots
    nat.close()


@pytest.mark.gpu
def test_native_arena_stages_the_right_bytes():
    from pocketllm_b200.moe.native_staging import NativeExpertArena
    g = torch.Generator().manual_seed(0)
    E, B = 12, 96 * 1024
    store = torch.randint(0, 256, (E, B), dtype=torch.uint8, generator=g)
    arena = NativeExpertArena(store, device_slots=4, ring_slots=2)
    rnd = random.Random(1)
    torch.zeros(1, device="cuda")                       # a CUDA context on the current device
    for step in range(40):
        keys = rnd.sample(range(E), rnd.randint(1, 4))
        ptrs = arena.ensure_ptrs(keys)
        assert len(set(ptrs)) == len(keys)
        for k, p in zip(keys, ptrs):
            assert torch.equal(arena.read_back(p), store[k]), (step, k)
    st = arena.stats
    assert st["misses"] * B == st["bytes_copied"] and st["hits"] > 0 and st["evictions"] > 0
    arena.close()
