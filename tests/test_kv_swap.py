"""KV swap tier: host store, device slots with LRU reuse, selection rewritten to physical rows. The bookkeeping and the
copies run in host-only mode here; the GPU test moves real rows through pinned memory and the scatter kernel."""
import pytest
import torch


def _rows(n, row_elems, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, row_elems, generator=g)


def _check_resident(tier, rows, selected, physical, window):
    pool = tier.pool.cpu().contiguous().view(torch.uint8).view(tier.device_slots, -1).view(torch.float32)
    for lid, ph in zip(selected.flatten().tolist(), physical.flatten().tolist()):
        if lid < 0:
            assert ph == -1
        else:
            assert window <= ph < window + tier.device_slots
            assert torch.equal(pool[ph - window], rows[lid])


def test_host_only_swap_in_hits_misses_and_eviction():
    from pocketllm_b200.runtime.kv_swap import KvSwapTier, KvSwapError
    rows = _rows(40, 8)
    t = KvSwapTier(capacity=64, device_slots=6, row_bytes=32, window=128, host_only=True)
    t.store(0, rows[:25])
    t.store(25, rows[25:])
    sel = torch.tensor([3, 7, -1, 3, 11], dtype=torch.int32)
    ph = t.swap_in(sel)
    _check_resident(t, rows, sel, ph, 128)
    assert ph[0] == ph[3] and t.stats["misses"] == 3 and t.stats["hits"] == 0 and t.stats["h2d_bytes"] == 3 * 32
    ph2 = t.swap_in(torch.tensor([7, 11, 20, 21, 22], dtype=torch.int32))       # 2 hits, 3 misses, slots now full
    assert t.stats["hits"] == 2 and t.stats["misses"] == 6 and t.stats["evictions"] == 0
    sel3 = torch.tensor([[30, 31], [7, 32]], dtype=torch.int32)                  # 3 misses evict the oldest rows, never row 7
    ph3 = t.swap_in(sel3)
    _check_resident(t, rows, sel3, ph3, 128)
    assert t.stats["evictions"] == 3 and ph3[1, 0] == ph2[0]
    assert t.stats["stored_rows"] == 40 and t.stats["d2h_bytes"] == 40 * 32 and t.stats["host_bytes"] == 64 * 32
    with pytest.raises(KvSwapError, match="never stored"):
        t.swap_in(torch.tensor([50], dtype=torch.int32))
    with pytest.raises(KvSwapError, match="do not fit"):
        t.swap_in(torch.arange(7, dtype=torch.int32))
    with pytest.raises(KvSwapError, match="resident"):
        t.store(7, rows[:1])
    t.reset()
    assert t.stats["stored_rows"] == 0 and t.stats["hits"] == 0
    with pytest.raises(KvSwapError):
        KvSwapTier(capacity=4, device_slots=2, row_bytes=24, host_only=True)       # not a multiple of 16
    t.close()


def test_host_only_random_walk_matches_a_plain_lookup():
    from pocketllm_b200.runtime.kv_swap import KvSwapTier
    rows = _rows(200, 16, seed=1)
    t = KvSwapTier(capacity=200, device_slots=32, row_bytes=64, window=0, host_only=True)
    t.store(0, rows)
    g = torch.Generator().manual_seed(2)
    for _ in range(50):
        sel = torch.randint(-1, 200, (24,), generator=g, dtype=torch.int32)
        ph = t.swap_in(sel)
        _check_resident(t, rows, sel, ph, 0)
    s = t.stats
    assert s["hits"] + s["misses"] > 0 and s["steps"] == 50 and s["h2d_bytes"] == s["misses"] * 64


@pytest.mark.gpu
def test_gpu_rows_travel_through_pinned_memory_and_the_scatter_kernel():
    from pocketllm_b200.runtime.kv_swap import KvSwapTier
    rows = _rows(3000, 128, seed=3).cuda()                                         # 512-byte rows
    t = KvSwapTier(capacity=4096, device_slots=600, row_bytes=512, window=128)
    t.store(0, rows[:1000])
    t.store(1000, rows[1000:])
    g = torch.Generator().manual_seed(4)
    for step in range(6):
        sel = torch.randint(0, 3000, (4, 128), generator=g, dtype=torch.int32).cuda()
        sel[0, :5] = -1
        ph = t.swap_in(sel)
        torch.cuda.synchronize()
        _check_resident(t, rows.cpu(), sel.cpu(), ph.cpu(), 128)
    s = t.stats
    assert s["misses"] > 600 and s["evictions"] > 0 and s["hits"] > 0
    t.close()


@pytest.mark.gpu
def test_sparse_attention_over_swapped_slots_equals_attention_over_the_full_cache():
    """DSV4 compressed attention (window rows + selected compressed rows): the KV array holds the window and 64 slots; the
    tier makes each step's selection resident and rewrites it to slot rows. Same output as with the whole cache resident."""
    from pocketllm_b200.ops import dsv4_ops as dk
    from pocketllm_b200.runtime.kv_swap import KvSwapTier
    torch.manual_seed(0)
    H, hd, rd, win, ncomp, slots, ksel = 8, 128, 64, 16, 400, 64, 48
    full = (torch.randn(win + ncomp, hd, device="cuda") * 0.5).to(torch.bfloat16)
    small = torch.zeros(win + slots, hd, device="cuda", dtype=torch.bfloat16)
    small[:win] = full[:win]
    tier = KvSwapTier(capacity=ncomp, device_slots=slots, row_bytes=hd * 2, window=0, pool=small[win:])
    tier.store(0, full[win:])
    ang = torch.outer(torch.arange(4096).double(), 1.0 / (10000.0 ** (torch.arange(0, rd, 2).double() / rd)))
    cos_t, sin_t = torch.cos(ang).float().cuda(), torch.sin(ang).float().cuda()
    sink = torch.zeros(H, device="cuda")
    for step in range(5):
        q = torch.randn(2, H, hd, device="cuda").to(torch.bfloat16)
        pos = torch.tensor([1700 + step, 1701 + step], device="cuda", dtype=torch.int32)
        sel = torch.stack([torch.randperm(ncomp, device="cuda")[:ksel] for _ in range(2)]).to(torch.int32)
        sel[1, -3:] = -1
        want = dk.sparse_attn(q, full, pos, sink, cos_t, sin_t, win=win, ring=win, ratio=4, rd=rd, sel=sel)
        # two rows of 48 share the 64 slots: swap in row by row, attend row by row
        for m in range(2):
            phys = tier.swap_in(sel[m:m + 1])
            got = dk.sparse_attn(q[m:m + 1], small, pos[m:m + 1], sink, cos_t, sin_t, win=win, ring=win, ratio=4, rd=rd, sel=phys)
            assert torch.equal(got, want[m:m + 1])
    assert tier.stats["evictions"] > 0
    tier.close()
