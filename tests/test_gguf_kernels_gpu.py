"""Raw-GGUF-block kernels against the numpy dequantisers (B200 only)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TYPES = ["iq2_xxs", "q2_k", "iq1_m", "q4_k", "q5_k", "iq2_xs", "iq3_xxs", "q8_0"]


def _quant(w, name):
    from pocketllm_b200.formats import gguf_quants as gq
    blocks = gq.quantize(w, name)
    deq = gq.dequantize(blocks, name)
    return torch.from_numpy(blocks.reshape(w.shape[0], -1).copy()).cuda(), torch.from_numpy(deq).cuda()


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm()).item()


@pytest.mark.parametrize("name", TYPES)
@pytest.mark.parametrize("M", [1, 5])
def test_gguf_linear(name, M):
    from pocketllm_b200.ops import gguf_ops as go
    rng = np.random.default_rng(3)
    N, K = 96, 768
    raw, wd = _quant((rng.standard_normal((N, K)) * 0.02).astype(np.float32), name)
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    y = go.gguf_linear(x, raw, name, N, epi=2)
    assert _rel(y, x.float() @ wd.t()) < 2e-3


def test_gguf_linear_norm_swiglu_and_many_rows():
    from pocketllm_b200.ops import gguf_ops as go
    rng = np.random.default_rng(4)
    N, K, M = 128, 512, 19
    raw, wd = _quant((rng.standard_normal((N, K)) * 0.02).astype(np.float32), "q4_k")
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    gamma = 1 + torch.randn(K, device="cuda") * 0.1
    y = go.gguf_linear(x, raw, "q4_k", N, gamma=gamma, epi=1)
    xf = x.float()
    xn = (xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + 1e-6) * gamma).to(torch.bfloat16).float()
    gu = xn @ wd.t()
    assert _rel(y, torch.nn.functional.silu(gu[:, :64]) * gu[:, 64:]) < 1e-2


@pytest.mark.parametrize("name,M,N,K,epi", [("q4_k", 64, 384, 768, 2), ("iq2_xxs", 200, 512, 1024, 1), ("q8_0", 33, 96, 512, 0),
                                             ("q5_k", 130, 256, 2048, 2)])
def test_gguf_linear_tensor_core_path_for_many_rows(name, M, N, K, epi):
    """From 32 rows on the weight is decoded once to bf16 and the product runs on the tcgen05 GEMM; it agrees with the
    8-rows-at-a-time streaming path and with the dequantised fp32 reference."""
    from pocketllm_b200.ops import gguf_ops as go
    rng = np.random.default_rng(M + N)
    raw, wd = _quant((rng.standard_normal((N, K)) * 0.02).astype(np.float32), name)
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    gamma = 1 + torch.randn(K, device="cuda") * 0.1
    assert M >= go.TENSOR_CORE_MIN_ROWS
    y = go.gguf_linear(x, raw, name, N, gamma=gamma, epi=epi)
    keep = go.TENSOR_CORE_MIN_ROWS
    go.TENSOR_CORE_MIN_ROWS = 1 << 30
    try:
        y_stream = go.gguf_linear(x, raw, name, N, gamma=gamma, epi=epi)
    finally:
        go.TENSOR_CORE_MIN_ROWS = keep
    xf = x.float()
    xn = (xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + 1e-6) * gamma).to(torch.bfloat16).float()
    ref = xn @ wd.t()
    if epi == 1:
        ref = torch.nn.functional.silu(ref[:, : N // 2]) * ref[:, N // 2:]
    tol = 1.5e-2 if epi == 1 else 6e-3
    assert y.shape == y_stream.shape and y.dtype == y_stream.dtype
    assert _rel(y, ref) < tol and _rel(y, y_stream) < tol


@pytest.mark.parametrize("score,norm", [("sigmoid", True), ("softmax", False), ("sqrtsoftplus", True)])
def test_router_topk(score, norm):
    from pocketllm_b200.ops import gguf_ops as go
    T, H, E, k = 7, 512, 64, 8
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    rw = torch.randn(E, H, device="cuda") * 0.05
    bias = torch.randn(E, device="cuda") * 0.01
    ids, w = go.router_topk(x, rw, k, bias=bias, score_func=score, norm_topk=norm, route_scale=1.5)
    logits = x.float() @ rw.t()
    sc = {"sigmoid": torch.sigmoid, "softmax": lambda z: torch.softmax(z, -1),
          "sqrtsoftplus": lambda z: torch.sqrt(torch.nn.functional.softplus(z))}[score](logits)
    ref_ids = torch.topk(sc + bias, k, dim=-1).indices
    assert torch.equal(ids.long().sort(-1).values, ref_ids.sort(-1).values)
    ref_w = torch.gather(sc, 1, ids.long())
    if norm:
        ref_w = ref_w / ref_w.sum(-1, keepdim=True)
    assert torch.allclose(w, ref_w * 1.5, rtol=2e-3, atol=1e-5)


@pytest.mark.parametrize("t13,t2,T", [("iq2_xxs", "q2_k", 1), ("iq2_xxs", "iq2_xxs", 40), ("iq1_m", "iq1_m", 9)])
def test_moe_forward_matches_dequantised_reference(t13, t2, T):
    from pocketllm_b200.ops import gguf_ops as go
    rng = np.random.default_rng(5)
    E, H, I, k = 8, 512, 256, 2
    w13 = (rng.standard_normal((E * 2 * I, H)) * 0.02).astype(np.float32)
    w2 = (rng.standard_normal((E * H, I)) * 0.02).astype(np.float32)
    raw13, d13 = _quant(w13, t13)
    raw2, d2 = _quant(w2, t2)
    d13, d2 = d13.view(E, 2 * I, H), d2.view(E, H, I)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    rw = torch.randn(E, H, device="cuda") * 0.05
    ids, w = go.router_topk(x, rw, k, score_func="sigmoid")
    seg, tok, rwt = go.group_routes(ids, w, E)
    assert int(seg[-1]) == T * k
    counts = torch.bincount(ids.reshape(-1).long(), minlength=E)
    assert torch.equal((seg[1:] - seg[:-1]).long(), counts)
    y = go.gguf_moe_forward(x, raw13, raw2, t13, t2, E, I, seg, tok, rwt)
    ref = torch.zeros(T, H, device="cuda")
    xf = x.float()
    for t in range(T):
        for j in range(k):
            e = int(ids[t, j])
            gu = d13[e] @ xf[t]
            ref[t] += w[t, j] * (d2[e] @ (torch.nn.functional.silu(gu[:I]) * gu[I:]))
    assert _rel(y, ref) < 3e-3
    # expert-parallel halves add up to the whole
    lo = go.gguf_moe_forward(x, raw13[: E // 2 * 2 * I], raw2[: E // 2 * H], t13, t2, E, I, seg, tok, rwt, local_experts=E // 2)
    hi = go.gguf_moe_forward(x, raw13[E // 2 * 2 * I:], raw2[E // 2 * H:], t13, t2, E, I, seg, tok, rwt,
                             expert_offset=E // 2, local_experts=E // 2)
    assert _rel(lo + hi, ref) < 3e-3


@pytest.mark.parametrize("T,E,topk", [(300, 8, 3), (64, 16, 2), (700, 4, 2)])
def test_grouped_tensor_core_experts_match_the_route_kernels(T, E, topk):
    """Prefill-sized steps: experts decoded once to bf16, rows gathered in expert order, two grouped tcgen05 GEMMs (SwiGLU,
    then down) over the (expert, row tile, column block) list built from the route segments on the device; ragged groups
    (some empty, some longer than one tile), expert-parallel halves, bitwise reproducible."""
    import numpy as np
    from pocketllm_b200.formats import gguf_quants as gq
    from pocketllm_b200.ops import gguf_ops as go
    torch.manual_seed(T)
    H, I = 512, 256
    rng = np.random.default_rng(T)
    w13 = torch.from_numpy(gq.quantize((rng.standard_normal((E * 2 * I, H)) * 0.05).astype(np.float32), "q4_k")).cuda().view(-1)
    w2 = torch.from_numpy(gq.quantize((rng.standard_normal((E * H, I)) * 0.05).astype(np.float32), "iq2_xxs")).cuda().view(-1)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E - 1)[:topk] for _ in range(T)]).int().cuda()      # the last expert gets no route
    ids[: T // 2] = torch.where(ids[: T // 2] == 1, torch.zeros_like(ids[: T // 2]), ids[: T // 2]) if topk == 1 else ids[: T // 2]
    wts = torch.rand(T, topk, device="cuda")
    routes = go.group_routes(ids, wts, E)
    seg, tok, rw = routes
    want = go.gguf_moe_forward(x, w13, w2, "q4_k", "iq2_xxs", E, I, seg, tok, rw, routes=routes)
    got = [go.gguf_moe_forward_grouped(x, w13, w2, "q4_k", "iq2_xxs", E, I, routes) for _ in range(2)]
    assert torch.equal(got[0], got[1])
    assert _rel(got[0], want) < 6e-3                       # hidden activations pass through bf16 between the two GEMMs
    half = E // 2
    lo = go.gguf_moe_forward_grouped(x, w13[: w13.numel() // 2], w2[: w2.numel() // 2], "q4_k", "iq2_xxs", E, I, routes, expert_offset=0,
                                     local_experts=half)
    hi = go.gguf_moe_forward_grouped(x, w13[w13.numel() // 2:], w2[w2.numel() // 2:], "q4_k", "iq2_xxs", E, I, routes, expert_offset=half,
                                     local_experts=half)
    assert _rel(lo + hi, got[0]) < 1e-5


def test_moe_forward_fixed_order_reduce_is_bitwise_reproducible():
    """Per-route outputs summed in route order: two runs agree bit for bit and match the atomic path closely."""
    import numpy as np
    from pocketllm_b200.formats import gguf_quants as gq
    from pocketllm_b200.ops import gguf_ops as go
    torch.manual_seed(0)
    E, H, I, T, topk = 8, 512, 256, 37, 3
    rng = np.random.default_rng(0)
    w13 = torch.from_numpy(gq.quantize((rng.standard_normal((E * 2 * I, H)) * 0.05).astype(np.float32), "q4_k")).cuda().view(-1)
    w2 = torch.from_numpy(gq.quantize((rng.standard_normal((E * H, I)) * 0.05).astype(np.float32), "q4_k")).cuda().view(-1)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E)[:topk] for _ in range(T)]).int().cuda()
    wts = torch.rand(T, topk, device="cuda")
    routes = go.group_routes(ids, wts, E)
    seg, tok, rw = routes
    runs = [go.gguf_moe_forward(x, w13, w2, "q4_k", "q4_k", E, I, seg, tok, rw, routes=routes) for _ in range(3)]
    assert torch.equal(runs[0], runs[1]) and torch.equal(runs[0], runs[2])
    atomic = go.gguf_moe_forward(x, w13, w2, "q4_k", "q4_k", E, I, seg, tok, rw)
    assert ((runs[0] - atomic).norm() / atomic.norm()).item() < 1e-5
    # expert-parallel halves add up to the whole
    lo = go.gguf_moe_forward(x, w13[: w13.numel() // 2], w2[: w2.numel() // 2], "q4_k", "q4_k", E, I, seg, tok, rw, expert_offset=0, local_experts=4, routes=routes)
    hi = go.gguf_moe_forward(x, w13[w13.numel() // 2:], w2[w2.numel() // 2:], "q4_k", "q4_k", E, I, seg, tok, rw, expert_offset=4, local_experts=4, routes=routes)
    assert ((lo + hi - runs[0]).norm() / runs[0].norm()).item() < 1e-6


def test_staged_experts_match_resident_experts():
    """Experts staged from pinned host memory through a 3-slot device cache give the resident result."""
    import numpy as np
    from pocketllm_b200.formats import gguf_quants as gq
    from pocketllm_b200.moe.expert_cache import ExpertStagingCache, staged_moe_forward
    from pocketllm_b200.ops import gguf_ops as go
    torch.manual_seed(1)
    E, H, I, T, topk = 8, 256, 256, 21, 2
    rng = np.random.default_rng(1)
    w13 = torch.from_numpy(gq.quantize((rng.standard_normal((E * 2 * I, H)) * 0.05).astype(np.float32), "q4_k")).reshape(E, -1)
    w2 = torch.from_numpy(gq.quantize((rng.standard_normal((E * H, I)) * 0.05).astype(np.float32), "q4_k")).reshape(E, -1)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E)[:topk] for _ in range(T)]).int().cuda()
    wts = torch.rand(T, topk, device="cuda")
    routes = go.group_routes(ids, wts, E)
    want = go.gguf_moe_forward(x, w13.cuda().view(-1), w2.cuda().view(-1), "q4_k", "q4_k", E, I, *routes, routes=routes)
    cache = ExpertStagingCache({"w13": w13, "w2": w2}, slots=3)
    got = staged_moe_forward(cache, x, ids, wts, "q4_k", "q4_k", I)
    assert ((got - want).norm() / want.norm()).item() < 1e-6
    assert cache.lru.stats["misses"] >= E - 1 and cache.bytes_staged > 0
    again = staged_moe_forward(cache, x[:1], ids[:1], wts[:1], "q4_k", "q4_k", I)            # decode-like step
    assert ((again - want[:1]).norm() / want[:1].norm()).item() < 1e-6
    cache.prefetch([0, 1, 2])
    assert all(int(cache.table[e]) >= 0 for e in (0, 1, 2))
