"""Numerics of the hand-written kernels against plain PyTorch fp32 references (B200 only)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda:0")


def _fp8_weight(n, k, seed=0, sigma=0.02):
    from pocketllm_b200.formats import fp8
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * sigma
    q, s = fp8.quantize_block128(w)
    return q.cuda(), s.float().cuda(), fp8.dequantize_block128(q, s).cuda()


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def test_native_library_is_loaded():
    from pocketllm_b200.ops import lib
    lib.kernels()
    assert any("libpocket_kernels.so" in p for p in lib.loaded_library_paths())


@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("N,K", [(256, 512), (1024, 5120), (384, 2176)])
def test_matvec_fp8(M, N, K):
    from pocketllm_b200 import ops
    q, s, wd = _fp8_weight(N, K, seed=N + K)
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    y = ops.matvec(x, q, s, epi=2)
    ref = x.float() @ wd.t()
    assert _rel_err(y, ref) < 2e-3


def test_matvec_chunked_k_and_bf16_rows():
    from pocketllm_b200 import ops
    N, Nb, K, M = 256, 64, 17408, 8
    q, s, wd = _fp8_weight(N, K, seed=5)
    wb = (torch.randn(Nb, K, device="cuda") * 0.02).to(torch.bfloat16)
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    y = ops.matvec(x, q, s, wb, epi=2)
    ref = torch.cat([x.float() @ wd.t(), x.float() @ wb.float().t()], dim=1)
    assert _rel_err(y, ref) < 2e-3


def test_matvec_fused_norm_parts_swiglu():
    from pocketllm_b200 import ops
    inter, K, M, R = 512, 1024, 2, 3
    q, s, wd = _fp8_weight(2 * inter, K, seed=9)
    x = (torch.randn(M, K, device="cuda")).to(torch.bfloat16)
    parts = torch.randn(R, M, K, device="cuda") * 0.3
    gamma = torch.randn(K, device="cuda") * 0.1
    hidden_out = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
    y = ops.matvec(x, q, s, gamma=gamma, parts=parts, hidden_out=hidden_out, epi=1)
    h = x.float()
    for r in range(R):                                       # the kernel adds the partial sums one after the other
        h = h + parts[r]
    h = h.to(torch.bfloat16)
    assert torch.equal(h, hidden_out)
    hf = h.float()
    xn = (hf * torch.rsqrt((hf * hf).mean(-1, keepdim=True) + 1e-6) * (1 + gamma)).to(torch.bfloat16).float()
    gu = xn @ wd.t()
    ref = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
    assert _rel_err(y, ref) < 1e-2


@pytest.mark.parametrize("M", [1, 2])
@pytest.mark.parametrize("N,Nb,K,epi,norm", [(4096, 0, 5120, 1, True), (2048, 0, 17408, 0, False), (3072, 64, 5120, 0, True),
                                             (640, 0, 2176, 2, True), (1024, 0, 6144, 0, False), (130, 0, 512, 2, False)])
def test_matvec_ring_matches_register_path(M, N, Nb, K, epi, norm):
    """Decode shapes go through the shared-memory ring (bulk asynchronous copies); they agree with the
    register-streaming kernel up to the fp32 summation order, repeat exactly, and match fp32 torch within the FP8 tolerance."""
    import os
    from pocketllm_b200 import ops
    q, s, wd = _fp8_weight(N, K, seed=N + K + epi)
    wb = (torch.randn(Nb, K, device="cuda") * 0.02).to(torch.bfloat16) if Nb else None
    x = (torch.randn(M, K, device="cuda") * 0.7).to(torch.bfloat16)
    kw = {}
    if norm:
        kw = dict(gamma=torch.randn(K, device="cuda") * 0.1, parts=torch.randn(2, M, K, device="cuda") * 0.3,
                  hidden_out=torch.empty(M, K, device="cuda", dtype=torch.bfloat16))
    y = ops.matvec(x, q, s, wb, epi=epi, **kw)
    assert ops.matvec_ring_status() == 0
    os.environ["POCKET_MATVEC_RING"] = "0"
    try:
        y0 = ops.matvec(x, q, s, wb, epi=epi, **kw)
    finally:
        del os.environ["POCKET_MATVEC_RING"]
    assert _rel_err(y, y0) < 1e-3          # the two kernels cut K differently among warps: fp32 sums in another order
    assert torch.equal(y, ops.matvec(x, q, s, wb, epi=epi, **kw))
    h = x.float()
    if norm:
        for r in range(kw["parts"].shape[0]):                    # same order as the kernel: fp32 sums round differently otherwise
            h = h + kw["parts"][r]
        h = h.to(torch.bfloat16)
        assert torch.equal(h, kw["hidden_out"])
        hf = h.float()
        h = (hf * torch.rsqrt((hf * hf).mean(-1, keepdim=True) + 1e-6) * (1 + kw["gamma"])).to(torch.bfloat16).float()
    w_all = wd if wb is None else torch.cat([wd, wb.float()], 0)
    ref = h @ w_all.t()
    if epi == 1:
        ref = torch.nn.functional.silu(ref[:, : N // 2]) * ref[:, N // 2:]
    assert _rel_err(y, ref) < (1e-2 if epi == 1 else 3e-3)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (512, 1024, 5120), (200, 384, 256), (64, 256, 2176), (1000, 640, 512)])
def test_gemm_umma_fp8(M, N, K):
    from pocketllm_b200 import ops
    q, s, wd = _fp8_weight(N, K, seed=M + N)
    a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    c = ops.gemm_umma(a, q, s, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    ref = a.float() @ wd.t()
    assert _rel_err(c, ref) < 6e-3


def test_gemm_umma_bf16_and_epilogues():
    from pocketllm_b200 import ops
    M, N, K = 300, 512, 1024
    a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    wb = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
    c = ops.gemm_umma(a, wb, epi=ops.EPI_F32)
    ref = a.float() @ wb.float().t()
    assert _rel_err(c, ref) < 2e-3
    # residual add
    q, s, wd = _fp8_weight(N, K, seed=3)
    resid = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    c2 = ops.gemm_umma(a, q, s, epi=ops.EPI_RESID, resid=resid)
    assert _rel_err(c2, resid.float() + a.float() @ wd.t()) < 6e-3
    # SwiGLU: rows = gate then up
    c3 = ops.gemm_umma(a, q, s, epi=ops.EPI_SWIGLU)
    gu = a.float() @ wd.t()
    ref3 = torch.nn.functional.silu(gu[:, : N // 2]) * gu[:, N // 2:]
    assert c3.shape == (M, N // 2)
    assert _rel_err(c3, ref3) < 1.5e-2


def test_gemm_umma_narrow_n():
    from pocketllm_b200 import ops
    M, N, K = 130, 64, 256
    a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    wb = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
    c = ops.gemm_umma(a, wb)
    assert _rel_err(c, a.float() @ wb.float().t()) < 6e-3


@pytest.mark.parametrize("M,N,K", [(512, 1024, 512), (300, 768, 1024), (130, 64, 256), (1, 256, 64), (700, 2304, 320)])
def test_gemm_bf16_persistent_tiles(M, N, K):
    """128x256 tiles, several tiles per CTA (double-buffered accumulator), ragged M and N edges."""
    from pocketllm_b200 import ops
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    ref = a.float() @ w.float().t()
    c = ops.gemm_bf16(a, w, epi=ops.EPI_F32, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0 and _rel_err(c, ref) < 2e-3
    assert _rel_err(ops.gemm_bf16(a, w), ref) < 6e-3
    resid = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    assert _rel_err(ops.gemm_bf16(a, w, epi=ops.EPI_RESID, resid=resid), resid.float() + ref) < 6e-3
    if (N // 2) % 128 == 0:
        got = ops.gemm_bf16(a, w, epi=ops.EPI_SWIGLU)
        want = torch.nn.functional.silu(ref[:, : N // 2]) * ref[:, N // 2:]
        assert got.shape == (M, N // 2) and _rel_err(got, want) < 1.5e-2


@pytest.mark.parametrize("M,N,K,epi", [(512, 5120, 1024, 0), (512, 5120, 1024, 2), (384, 5120, 2048, 1), (512, 1536, 4096, 3), (200, 2304, 3072, 0)])
def test_gemm_bf16_stream_k(M, N, K, epi):
    """Tile counts that would idle most SMs: the k-steps are cut into equal ranges per CTA and partial tiles are
    combined by the owner; the result must agree with the whole-tile schedule and with fp32 torch."""
    import os
    from pocketllm_b200 import ops
    torch.manual_seed(M + N + K + epi)
    a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    resid = torch.randn(M, N, device="cuda").to(torch.bfloat16) if epi == ops.EPI_RESID else None
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    os.environ["POCKET_GEMM_STREAMK"] = "1"
    try:
        got = [ops.gemm_bf16(a, w, epi=epi, resid=resid, status=status) for _ in range(3)]
        torch.cuda.synchronize()
    finally:
        del os.environ["POCKET_GEMM_STREAMK"]
    assert status.item() == 0
    os.environ["POCKET_GEMM_NO_STREAMK"] = "1"
    try:
        plain = ops.gemm_bf16(a, w, epi=epi, resid=resid)
    finally:
        del os.environ["POCKET_GEMM_NO_STREAMK"]
    ref = a.float() @ w.float().t()
    if epi == ops.EPI_RESID:
        ref = ref + resid.float()
    if epi == ops.EPI_SWIGLU:
        ref = torch.nn.functional.silu(ref[:, : N // 2]) * ref[:, N // 2:]
    assert _rel_err(got[0], ref) < (1.5e-2 if epi == 1 else 6e-3)
    assert _rel_err(got[0], plain) < 4e-3                      # fp32 sums in a different order, then one bf16 rounding
    assert torch.equal(got[0], got[1]) and torch.equal(got[1], got[2])


def test_gemm_bf16_many_tiles_per_cta():
    """More tiles than SMs: every CTA walks several tiles and both accumulators are reused."""
    from pocketllm_b200 import ops
    torch.manual_seed(5)
    M, N, K = 1024, 12288, 256                # 8 x 48 = 384 tiles
    a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    c = ops.gemm_bf16(a, w)
    assert _rel_err(c, a.float() @ w.float().t()) < 6e-3
    assert torch.equal(c, ops.gemm_bf16(a, w))


def _fp8_gemm_inputs(M, N, K, seed):
    from pocketllm_b200.formats import fp8 as f8
    torch.manual_seed(seed)
    a = (torch.randn(M, K, device="cuda") * torch.rand(M, 1, device="cuda") * 2).to(torch.bfloat16)
    a[:, ::37] *= 8                                                     # outliers that set the block scale
    wq, ws = f8.quantize_block128(torch.randn(N, K) * 0.05, scale_dtype=torch.float32)
    wq, ws = wq.cuda(), ws.cuda().contiguous()
    return a, wq, ws, f8.dequantize_block128(wq, ws)


@pytest.mark.parametrize("terms", [1, 2])
@pytest.mark.parametrize("M,N,K", [(512, 1024, 512), (300, 768, 1024), (130, 256, 256), (1, 256, 128), (700, 2304, 384)])
def test_gemm_fp8_native_tiles(M, N, K, terms):
    """Weights stay E4M3 codes; activations are one or two E4M3 terms with a scale per row and k block. The kernel must
    reproduce (sum of the terms * scale) @ dequantised weights to fp32 accuracy, and with two terms the bf16 product."""
    from pocketllm_b200 import ops
    a, wq, ws, wd = _fp8_gemm_inputs(M, N, K, M + N + K)
    aq, asc = ops.quant_act_fp8(a, terms)
    m_pad = aq.shape[1]
    planes = aq.view(torch.float8_e4m3fn).float().sum(0)[:M]             # [M, K]
    a_deq = planes * asc.t()[:M].repeat_interleave(128, 1)
    # quantiser: scale = amax / 448 per (row, block), first term is the nearest code
    blocks = a.float().view(M, K // 128, 128)
    want_s = blocks.abs().amax(-1) / 448.0
    want_s = torch.where(want_s > 0, want_s, torch.ones_like(want_s))
    assert torch.allclose(asc.t()[:M], want_s, rtol=1e-6, atol=0)
    assert aq[:, M:].abs().sum() == 0 and m_pad % 128 == 0
    assert _rel_err(a_deq, a.float()) < (4e-2 if terms == 1 else 3e-3)
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    c = ops.gemm_fp8(aq, asc, M, wq, ws, epi=ops.EPI_F32, status=status)
    torch.cuda.synchronize()
    exact = a_deq @ wd.t()
    assert status.item() == 0 and _rel_err(c, exact) < 2e-5
    ref = a.float() @ wd.t()
    assert _rel_err(c, ref) < (4e-2 if terms == 1 else 3e-3)
    assert _rel_err(ops.gemm_fp8(aq, asc, M, wq, ws), exact) < 6e-3
    resid = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    assert _rel_err(ops.gemm_fp8(aq, asc, M, wq, ws, epi=ops.EPI_RESID, resid=resid), resid.float() + exact) < 6e-3
    if (N // 2) % 128 == 0:
        got = ops.gemm_fp8(aq, asc, M, wq, ws, epi=ops.EPI_SWIGLU)
        want = torch.nn.functional.silu(exact[:, : N // 2]) * exact[:, N // 2:]
        assert got.shape == (M, N // 2) and _rel_err(got, want) < 1.5e-2


@pytest.mark.parametrize("M,N,K,epi", [(512, 5120, 1024, 0), (384, 5120, 2048, 1), (512, 1536, 4096, 3), (200, 2304, 3072, 2)])
def test_gemm_fp8_stream_k_and_many_tiles(M, N, K, epi):
    import os
    from pocketllm_b200 import ops
    a, wq, ws, wd = _fp8_gemm_inputs(M, N, K, M + N + K + epi)
    aq, asc = ops.quant_act_fp8(a, 2)
    resid = torch.randn(M, N, device="cuda").to(torch.bfloat16) if epi == ops.EPI_RESID else None
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    os.environ["POCKET_GEMM_STREAMK"] = "1"
    try:
        got = [ops.gemm_fp8(aq, asc, M, wq, ws, epi=epi, resid=resid, status=status) for _ in range(3)]
        torch.cuda.synchronize()
    finally:
        del os.environ["POCKET_GEMM_STREAMK"]
    assert status.item() == 0
    ref = a.float() @ wd.t()
    if epi == ops.EPI_RESID:
        ref = ref + resid.float()
    if epi == ops.EPI_SWIGLU:
        ref = torch.nn.functional.silu(ref[:, : N // 2]) * ref[:, N // 2:]
    assert _rel_err(got[0], ref) < (1.5e-2 if epi == 1 else 6e-3)
    assert torch.equal(got[0], got[1]) and torch.equal(got[1], got[2])
    # more tiles than SMs: both accumulators and every stage are reused many times
    a2, wq2, ws2, wd2 = _fp8_gemm_inputs(1024, 12288, 256, 9)
    aq2, asc2 = ops.quant_act_fp8(a2, 1)
    c2 = ops.gemm_fp8(aq2, asc2, 1024, wq2, ws2)
    planes = aq2.view(torch.float8_e4m3fn).float().sum(0) * asc2.t().repeat_interleave(128, 1)
    assert _rel_err(c2, planes @ wd2.t()) < 6e-3


def test_rmsnorm_embedding_argmax():
    from pocketllm_b200 import ops
    x = torch.randn(5, 640, device="cuda").to(torch.bfloat16)
    g = torch.randn(640, device="cuda") * 0.1
    y = ops.rmsnorm(x, g, mode=1)
    xf = x.float()
    ref = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + 1e-6) * (1 + g)
    assert _rel_err(y, ref) < 5e-3
    table = torch.randn(100, 64, device="cuda").to(torch.bfloat16)
    tok = torch.tensor([3, 99, 0], device="cuda", dtype=torch.int32)
    assert torch.equal(ops.embedding(tok, table), table[tok.long()])
    logits = torch.randn(4, 5000, device="cuda")
    logits[1, 77] = logits[1, 4000] = 50.0   # tie: lowest index wins
    am = ops.argmax(logits, id_offset=10)
    exp = logits.argmax(-1)
    exp[1] = 77
    assert am.tolist() == (exp + 10).tolist()


def _deltanet_ref(proj, Hk, Hv, conv_w, conv_state, A_log, dt_bias, norm_w, eps, S):
    """Serial recurrence in fp32 (cpp_engine/cuda/qwen_half_ops.cu:746-930 semantics)."""
    T = proj.shape[0]
    KD, VD = Hk * 128, Hv * 128
    outs = []
    tail = conv_state.clone()
    S = S.clone()
    rep = Hv // Hk
    for t in range(T):
        row = proj[t].float()
        packed, z = row[: 2 * KD + VD], row[2 * KD + VD: 2 * KD + 2 * VD]
        a, b = row[2 * KD + 2 * VD: 2 * KD + 2 * VD + Hv], row[2 * KD + 2 * VD + Hv: 2 * KD + 2 * VD + 2 * Hv]
        win = torch.cat([tail, packed[:, None]], 1)
        y = torch.nn.functional.silu((win * conv_w).sum(-1)).to(torch.bfloat16).float()
        tail = win[:, 1:]
        q, k, v = y[:KD].view(Hk, 128), y[KD:2 * KD].view(Hk, 128), y[2 * KD:].view(Hv, 128)
        q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6)
        k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        q, k = q.repeat_interleave(rep, 0), k.repeat_interleave(rep, 0)
        g = -torch.exp(A_log) * torch.nn.functional.softplus(a + dt_bias)
        beta = torch.sigmoid(b)
        S = S * torch.exp(g)[:, None, None]
        kv = torch.einsum("hkv,hk->hv", S, k)
        delta = (v - kv) * beta[:, None]
        S = S + torch.einsum("hk,hv->hkv", k, delta)
        o = torch.einsum("hkv,hk->hv", S, q) * (128 ** -0.5)
        o = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * norm_w * torch.nn.functional.silu(z.view(Hv, 128))
        outs.append(o.reshape(VD))
    return torch.stack(outs), S, tail


@pytest.mark.parametrize("Hk,Hv,T", [(2, 4, 1), (2, 4, 9), (1, 1, 5), (2, 2, 40)])
def test_deltanet_seq(Hk, Hv, T):
    from pocketllm_b200 import ops
    torch.manual_seed(Hk * 10 + T)
    KD, VD = Hk * 128, Hv * 128
    ld = 2 * KD + 2 * VD + 2 * Hv
    ld = (ld + 7) // 8 * 8
    proj = (torch.randn(T, ld, device="cuda")).to(torch.bfloat16)
    conv_w = torch.randn(2 * KD + VD, 4, device="cuda") * 0.3
    conv_state = torch.randn(2 * KD + VD, 3, device="cuda")
    A_log, dt_bias = torch.randn(Hv, device="cuda") * 0.5, torch.randn(Hv, device="cuda") * 0.5
    norm_w = 1 + torch.randn(128, device="cuda") * 0.05
    S = torch.randn(Hv, 128, 128, device="cuda") * 0.1
    ref_o, ref_S, ref_tail = _deltanet_ref(proj, Hk, Hv, conv_w, conv_state, A_log, dt_bias, norm_w, 1e-6, S)
    S2, cs2 = S.clone(), conv_state.clone()
    out = ops.deltanet_seq(proj, Hk, Hv, conv_w, cs2, A_log, dt_bias, norm_w, 1e-6, S2)
    assert _rel_err(out, ref_o) < 1e-2
    assert _rel_err(S2, ref_S) < 1e-3
    assert torch.allclose(cs2, ref_tail, atol=1e-6)


@pytest.mark.parametrize("Hk,Hv,T", [(2, 4, 64), (1, 2, 100), (2, 2, 33), (1, 1, 200)])
def test_deltanet_chunked_matches_serial_recurrence(Hk, Hv, T):
    from pocketllm_b200 import ops
    torch.manual_seed(Hv * 100 + T)
    KD, VD = Hk * 128, Hv * 128
    ld = (2 * KD + 2 * VD + 2 * Hv + 7) // 8 * 8
    proj = (torch.randn(T, ld, device="cuda")).to(torch.bfloat16)
    conv_w = torch.randn(2 * KD + VD, 4, device="cuda") * 0.3
    conv_state = torch.randn(2 * KD + VD, 3, device="cuda")
    A_log, dt_bias = torch.randn(Hv, device="cuda") * 0.5, torch.randn(Hv, device="cuda") * 0.5
    norm_w = 1 + torch.randn(128, device="cuda") * 0.05
    S = torch.randn(Hv, 128, 128, device="cuda") * 0.1
    ref_o, ref_S, ref_tail = _deltanet_ref(proj, Hk, Hv, conv_w, conv_state, A_log, dt_bias, norm_w, 1e-6, S)
    S2, cs2 = S.clone(), conv_state.clone()
    out = ops.deltanet_chunked(proj, Hk, Hv, conv_w, cs2, A_log, dt_bias, norm_w, 1e-6, S2)
    assert _rel_err(out, ref_o) < 1e-2
    assert _rel_err(S2, ref_S) < 2e-3
    assert torch.allclose(cs2, ref_tail, atol=1e-6)
    # and against the serial kernel, continuing from the produced state
    S3, cs3 = S.clone(), conv_state.clone()
    out3 = ops.deltanet_seq(proj, Hk, Hv, conv_w, cs3, A_log, dt_bias, norm_w, 1e-6, S3)
    assert _rel_err(out, out3) < 1e-2 and _rel_err(S2, S3) < 2e-3


@pytest.mark.parametrize("M,ctx,Hq,Hkv,nsplit", [(1, 1, 4, 2, 4), (1, 700, 10, 2, 8), (5, 300, 5, 1, 3), (8, 64, 8, 8, 2)])
def test_gqa_append_and_decode(M, ctx, Hq, Hkv, nsplit):
    from pocketllm_b200 import ops
    torch.manual_seed(ctx)
    D, cap, rd, theta = 128, 1024, 32, 1e6
    ld = Hq * 2 * D + 2 * Hkv * D
    kc = torch.zeros(Hkv, cap, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    base = ctx - 1                          # rows occupy positions base .. base+M-1
    kc[:, :base] = torch.randn(Hkv, base, D, device="cuda").to(torch.bfloat16)
    vc[:, :base] = torch.randn(Hkv, base, D, device="cuda").to(torch.bfloat16)
    proj = torch.randn(M, ld, device="cuda").to(torch.bfloat16)
    pos = torch.arange(base, base + M, device="cuda", dtype=torch.int32)
    qg, kg = torch.randn(D, device="cuda") * 0.1, torch.randn(D, device="cuda") * 0.1
    q = ops.qk_norm_rope_append(proj, Hq, Hkv, pos, qg, kg, 1e-6, rd, theta, kc, vc)
    out = ops.gqa_decode(q, kc, vc, pos, nsplit=nsplit, gate_proj=proj)

    def rope(x, p):
        half = rd // 2
        inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / rd)
        ang = (p * inv)
        cs, sn = torch.cos(ang).float().cuda(), torch.sin(ang).float().cuda()
        x1, x2 = x[..., :half], x[..., half:rd]
        return torch.cat([x1 * cs - x2 * sn, x2 * cs + x1 * sn, x[..., rd:]], -1)

    def rms(x, g):
        return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6) * (1 + g)

    pf = proj.float()
    for m in range(M):
        p = base + m
        qm = pf[m, : Hq * 2 * D].view(Hq, 2 * D)
        qh, gate = qm[:, :D], qm[:, D:]
        kh = pf[m, Hq * 2 * D: Hq * 2 * D + Hkv * D].view(Hkv, D)
        vh = pf[m, Hq * 2 * D + Hkv * D:].view(Hkv, D)
        qr = rope(rms(qh, qg).to(torch.bfloat16).float(), p).to(torch.bfloat16).float()
        kr = rope(rms(kh, kg).to(torch.bfloat16).float(), p).to(torch.bfloat16)
        assert _rel_err(q[m], qr) < 1e-2
        assert _rel_err(kc[:, p], kr) < 1e-2
        assert torch.equal(vc[:, p], vh.to(torch.bfloat16))
        K = kc[:, : p + 1].float().repeat_interleave(Hq // Hkv, 0)
        V = vc[:, : p + 1].float().repeat_interleave(Hq // Hkv, 0)
        sc = torch.einsum("hd,htd->ht", q[m].float(), K) * D ** -0.5
        o = torch.einsum("ht,htd->hd", torch.softmax(sc, -1), V) * torch.sigmoid(gate)
        assert _rel_err(out[m].view(Hq, D), o) < 1e-2


def test_gqa_fp8_kv_cache_append_and_decode():
    """FP8 KV cache: E4M3 codes with one scale per 64 channels (amax / 448). The appended rows must be the quantised
    keys / values, and attention over the cache must equal attention over its dequantised contents."""
    from pocketllm_b200 import ops
    torch.manual_seed(5)
    M, ctx, Hq, Hkv, D, cap, rd, theta, nsplit = 3, 200, 8, 2, 128, 512, 32, 1e6, 4
    ld = Hq * 2 * D + 2 * Hkv * D
    base = ctx - 1

    def quant(x):                                   # [..., 128] -> codes uint8, scales [..., 2]
        g = x.float().view(*x.shape[:-1], 2, 64)
        sc = g.abs().amax(-1) / 448.0
        sc = torch.where(sc > 0, sc, torch.ones_like(sc))
        codes = (g / sc.unsqueeze(-1)).to(torch.float8_e4m3fn)
        return codes.view(torch.uint8).view(*x.shape), sc

    def dequant(codes, sc):
        return (codes.view(torch.float8_e4m3fn).float().view(*codes.shape[:-1], 2, 64) * sc.unsqueeze(-1)).view(*codes.shape)

    kc = torch.zeros(Hkv, cap, D, device="cuda", dtype=torch.uint8)
    vc = torch.zeros_like(kc)
    ks = torch.ones(Hkv, cap, 2, device="cuda")
    vs = torch.ones_like(ks)
    kc[:, :base], ks[:, :base] = quant(torch.randn(Hkv, base, D, device="cuda").to(torch.bfloat16))
    vc[:, :base], vs[:, :base] = quant(torch.randn(Hkv, base, D, device="cuda").to(torch.bfloat16))
    proj = torch.randn(M, ld, device="cuda").to(torch.bfloat16)
    pos = torch.arange(base, base + M, device="cuda", dtype=torch.int32)
    qg, kg = torch.randn(D, device="cuda") * 0.1, torch.randn(D, device="cuda") * 0.1
    # the same rows through the bf16 cache give the unquantised keys to compare with
    kb = torch.zeros(Hkv, cap, D, device="cuda", dtype=torch.bfloat16)
    vb = torch.zeros_like(kb)
    ops.qk_norm_rope_append(proj, Hq, Hkv, pos, qg, kg, 1e-6, rd, theta, kb, vb)
    q = ops.qk_norm_rope_append(proj, Hq, Hkv, pos, qg, kg, 1e-6, rd, theta, kc, vc, ks, vs)
    for m in range(M):
        p = base + m
        # scales to the last bit or one apart (the framework divides by multiplying with 1/448), codes at most one apart
        wc, ws_ = quant(kb[:, p])
        assert torch.allclose(ks[:, p], ws_, rtol=1e-6, atol=0) and (kc[:, p].int() - wc.int()).abs().max() <= 1
        wc, ws_ = quant(vb[:, p])
        assert torch.allclose(vs[:, p], ws_, rtol=1e-6, atol=0) and (vc[:, p].int() - wc.int()).abs().max() <= 1
    out = ops.gqa_decode(q, kc, vc, pos, nsplit=nsplit, gate_proj=proj, kscale=ks, vscale=vs)
    Kd, Vd = dequant(kc, ks), dequant(vc, vs)
    for m in range(M):
        p = base + m
        gate = proj[m, : Hq * 2 * D].float().view(Hq, 2 * D)[:, D:]
        K = Kd[:, : p + 1].repeat_interleave(Hq // Hkv, 0)
        V = Vd[:, : p + 1].repeat_interleave(Hq // Hkv, 0)
        sc = torch.einsum("hd,htd->ht", q[m].float(), K) * D ** -0.5
        o = torch.einsum("ht,htd->hd", torch.softmax(sc, -1), V) * torch.sigmoid(gate)
        assert _rel_err(out[m].view(Hq, D), o) < 1e-2


@pytest.mark.parametrize("M,n,k", [(3, 5000, 512), (2, 70000, 2048), (4, 300, 64), (1, 40, 64)])
def test_topk_select_matches_torch_topk(M, n, k):
    from pocketllm_b200.ops import dsv4_ops as dk
    torch.manual_seed(n)
    score = torch.randn(M, n, device="cuda")
    score[0, ::7] = float("-inf")                       # entries a row cannot see
    score[-1, :n // 2] = score[-1, n // 2: 2 * (n // 2)]   # many exact ties
    lengths = torch.tensor([n, max(n - 17, 1), n, n][:M], device="cuda", dtype=torch.int32)
    got = dk.topk_select(score, k, lengths)
    for m in range(M):
        row = score[m, : int(lengths[m])]
        finite = int((~torch.isinf(row)).sum())
        want_n = min(k, finite)
        g = got[m]
        sel = g[g >= 0]
        assert sel.numel() == want_n and (g[want_n:] == -1).all()
        assert torch.equal(sel, torch.sort(sel).values) and sel.unique().numel() == want_n       # ascending, no repeats
        if want_n:
            kth = torch.topk(row, want_n).values[-1]
            assert (row[sel.long()] >= kth).all()                         # nothing below the k-th largest
            assert int((row > kth).sum()) == int((row[sel.long()] > kth).sum())   # everything above it is in
            ties = torch.nonzero(row == kth).flatten()
            taken = sel[row[sel.long()] == kth]
            assert torch.equal(taken.long(), ties[: taken.numel()])      # lowest indices win ties
    all_rows = dk.topk_select(score, k)
    assert all_rows.shape == (M, k)


@pytest.mark.parametrize("fp8_kv", [False, True])
def test_verify_rows_equal_single_row_decode_bit_for_bit(fp8_kv):
    """Exact-order verify: M draft rows through one call == M single-row calls at the same positions, bitwise, with and
    without the output gate, for the bf16 and the FP8 cache."""
    from pocketllm_b200 import ops
    torch.manual_seed(11)
    M, Hq, Hkv, D, cap, nsplit = 5, 8, 2, 128, 1024, 8
    base = 700
    q = torch.randn(M, Hq, D, device="cuda").to(torch.bfloat16)
    pos = torch.arange(base, base + M, device="cuda", dtype=torch.int32)
    proj = torch.randn(M, Hq * 2 * D + 2 * Hkv * D, device="cuda").to(torch.bfloat16)
    if fp8_kv:
        kc = torch.randint(0, 120, (Hkv, cap, D), device="cuda", dtype=torch.uint8)
        vc = torch.randint(0, 120, (Hkv, cap, D), device="cuda", dtype=torch.uint8)
        ks, vs = torch.rand(Hkv, cap, 2, device="cuda") * 0.02, torch.rand(Hkv, cap, 2, device="cuda") * 0.02
        kw = dict(kscale=ks, vscale=vs)
    else:
        kc = torch.randn(Hkv, cap, D, device="cuda").to(torch.bfloat16)
        vc = torch.randn(Hkv, cap, D, device="cuda").to(torch.bfloat16)
        kw = {}
    for gate in (None, proj):
        for window, sink in ((0, 0), (256, 4)):
            rows = ops.gqa_decode(q, kc, vc, pos, nsplit=nsplit, gate_proj=gate, window=window, sink=sink, **kw)
            for m in range(M):
                one = ops.gqa_decode(q[m:m + 1], kc, vc, pos[m:m + 1], nsplit=nsplit, gate_proj=None if gate is None else gate[m:m + 1],
                                     window=window, sink=sink, **kw)
                assert torch.equal(rows[m:m + 1], one), (m, window)


@pytest.mark.parametrize("M,pos0,Hq,Hkv", [(128, 0, 4, 2), (200, 77, 5, 1), (512, 1000, 8, 2), (37, 300, 6, 6), (300, 0, 2, 1)])
def test_gqa_prefill_tensor_core_attention_matches_fp32(M, pos0, Hq, Hkv):
    """tcgen05 flash attention of a prefill chunk against fp32 softmax attention, ragged chunk lengths, chunk offsets
    that are not multiples of the tile, with and without the output gate; and against the split-context SIMT kernel."""
    from pocketllm_b200 import ops
    torch.manual_seed(M + pos0)
    D, cap = 128, 2048
    ctx = pos0 + M
    kc = torch.zeros(Hkv, cap, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    kc[:, :ctx] = torch.randn(Hkv, ctx, D, device="cuda").to(torch.bfloat16)
    vc[:, :ctx] = torch.randn(Hkv, ctx, D, device="cuda").to(torch.bfloat16)
    kc[:, ctx:ctx + 64] = 7.0                       # rows behind the chunk: read by the last tile, must be masked
    vc[:, ctx:ctx + 64] = -9.0
    q = torch.randn(M, Hq, D, device="cuda").to(torch.bfloat16)
    proj = torch.randn(M, Hq * 2 * D + 2 * Hkv * D, device="cuda").to(torch.bfloat16)
    pos = torch.arange(pos0, pos0 + M, device="cuda", dtype=torch.int32)
    rep = Hq // Hkv
    K, V = kc[:, :ctx].float().repeat_interleave(rep, 0), vc[:, :ctx].float().repeat_interleave(rep, 0)
    sc = torch.einsum("mhd,htd->mht", q.float(), K) * D ** -0.5
    mask = torch.arange(ctx, device="cuda")[None, None, :] > pos[:, None, None]
    want = torch.einsum("mht,htd->mhd", torch.softmax(sc.masked_fill(mask, float("-inf")), -1), V)
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    got = ops.gqa_prefill(q, kc, vc, pos, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert _rel_err(got.view(M, Hq, D), want) < 1e-2
    gated = ops.gqa_prefill(q, kc, vc, pos, gate_proj=proj)
    gate = proj[:, : Hq * 2 * D].float().view(M, Hq, 2 * D)[:, :, D:]
    assert _rel_err(gated.view(M, Hq, D), want * torch.sigmoid(gate)) < 1e-2
    simt = ops.gqa_decode(q, kc, vc, pos, nsplit=1, gate_proj=proj)
    assert _rel_err(gated, simt) < 1e-2


def test_full_qk_norm_rope_append_matches_torch():
    """Whole-vector RMS (one gamma per element) + half-split rotation from tables + KV append, against plain PyTorch."""
    from pocketllm_b200 import ops
    from pocketllm_b200.models.minimax_m2 import _rms, _rope, _rope_tables
    torch.manual_seed(0)
    T, Hq, Hkv, D, rope_dim, ctx = 5, 6, 2, 128, 64, 40
    q = torch.randn(T, Hq * D, device="cuda").to(torch.bfloat16)
    k = torch.randn(T, Hkv * D, device="cuda").to(torch.bfloat16)
    v = torch.randn(T, Hkv * D, device="cuda").to(torch.bfloat16)
    gq, gk = 1 + torch.randn(Hq * D, device="cuda") * 0.1, 1 + torch.randn(Hkv * D, device="cuda") * 0.1
    pos = torch.tensor([3, 4, 5, 17, 39], device="cuda", dtype=torch.int32)
    cos_t, sin_t = _rope_tables(ctx, rope_dim, 5e6, "cuda")
    kc = torch.zeros(Hkv, ctx, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    out = ops.full_qk_norm_rope_append(q, k, v, pos, gq, gk, cos_t, sin_t, kc, vc, n_heads=Hq, n_kv_heads=Hkv, rope_dim=rope_dim, eps=1e-6)
    want_q = _rope(_rms(q.float(), gq, 1e-6).view(T, Hq, D), pos, rope_dim, 5e6).to(torch.bfloat16)
    want_k = _rope(_rms(k.float(), gk, 1e-6).view(T, Hkv, D), pos, rope_dim, 5e6).to(torch.bfloat16)
    assert _rel_err(out, want_q) < 4e-3 and (out.float() - want_q.float()).abs().max() < 0.05
    idx = pos.long()
    assert _rel_err(kc[:, idx], want_k.transpose(0, 1)) < 4e-3
    assert torch.equal(vc[:, idx], v.view(T, Hkv, D).transpose(0, 1))
    untouched = torch.ones(ctx, dtype=torch.bool, device="cuda")
    untouched[idx] = False
    assert kc[:, untouched].abs().sum() == 0 and vc[:, untouched].abs().sum() == 0
