"""Allocation-free GQA decode entry point (`pk_gqa_decode_static`), called through its exported C
symbol and checked against `pk_gqa_decode` with a caller-provided workspace. This file sorts
last on purpose: the check must hold both in a fresh process and after every other test has
used the library."""
from ctypes import c_char_p, c_float, c_int, c_void_p

import pytest
import torch

STATIC_WS_FLOATS = 8 * 64 * 8 * 130


def _lib():
    from pocketllm_b200.ops import lib
    L = lib.kernels()
    L.pk_gqa_decode_static_error.restype = c_char_p
    return L


def _call_static(L, q, kc, vc, pos, nsplit, gate_proj, out):
    M, Hq, D = q.shape
    Hkv, cap, _ = kc.shape
    return L.pk_gqa_decode_static(
        c_void_p(q.data_ptr()), c_void_p(kc.data_ptr()), c_void_p(vc.data_ptr()), c_void_p(pos.data_ptr()), c_int(M), c_int(Hq),
        c_int(Hkv), c_int(D), c_int(cap), c_float(D ** -0.5), c_int(nsplit), c_int(0), c_int(0),
        c_void_p(gate_proj.data_ptr()), c_int(gate_proj.stride(0)), c_void_p(out.data_ptr()),
        c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.gpu
def test_static_scratch_matches_workspace_variant_twice():
    from pocketllm_b200 import ops
    L = _lib()
    D, cap = 128, 2048
    # two different problems back to back: the second call finds the first one's partials in the scratch
    for seed, (M, ctx, Hq, Hkv, nsplit) in enumerate([(4, 900, 16, 4, 8), (8, 1500, 24, 4, 5)]):
        torch.manual_seed(seed)
        kc = torch.randn(Hkv, cap, D, device="cuda").to(torch.bfloat16)
        vc = torch.randn(Hkv, cap, D, device="cuda").to(torch.bfloat16)
        q = torch.randn(M, Hq, D, device="cuda").to(torch.bfloat16)
        gate = torch.randn(M, Hq * 2 * D, device="cuda").to(torch.bfloat16)
        pos = torch.arange(ctx - M, ctx, device="cuda", dtype=torch.int32)
        want = ops.gqa_decode(q, kc, vc, pos, nsplit=nsplit, gate_proj=gate)
        got = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        assert _call_static(L, q, kc, vc, pos, nsplit, gate, got) == 0, L.pk_gqa_decode_static_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.isfinite(got.float()).all()
        torch.testing.assert_close(got.float(), want.float(), rtol=1e-2, atol=1e-3)


@pytest.mark.gpu
def test_static_scratch_rejects_oversize_problem():
    L = _lib()
    M, Hq, D, nsplit = 8, 64, 128, 9                     # one split more than the fixed array holds
    assert M * Hq * nsplit * (D + 2) > STATIC_WS_FLOATS
    q = torch.zeros(M, Hq, D, device="cuda", dtype=torch.bfloat16)
    kc = torch.zeros(8, 64, D, device="cuda", dtype=torch.bfloat16)
    pos = torch.zeros(M, device="cuda", dtype=torch.int32)
    gate = torch.zeros(M, Hq * 2 * D, device="cuda", dtype=torch.bfloat16)
    out = torch.full((M, Hq * D), 7.0, device="cuda", dtype=torch.bfloat16)
    assert _call_static(L, q, kc, kc, pos, nsplit, gate, out) == 1        # PK_ERR_BAD_ARG, nothing launched
    msg = L.pk_gqa_decode_static_error().decode()
    assert "exceeds the fixed scratch" in msg and str(STATIC_WS_FLOATS) in msg
    torch.cuda.synchronize()
    assert (out == 7.0).all()
    # a kv head count of zero (or one that does not divide the q heads) is refused the same way, before any launch
    for bad_hkv in (0, -3, 5):
        kc_bad = torch.zeros(max(bad_hkv, 1), 64, D, device="cuda", dtype=torch.bfloat16)
        rc = L.pk_gqa_decode_static(
            c_void_p(q.data_ptr()), c_void_p(kc_bad.data_ptr()), c_void_p(kc_bad.data_ptr()), c_void_p(pos.data_ptr()), c_int(M), c_int(Hq),
            c_int(bad_hkv), c_int(D), c_int(64), c_float(D ** -0.5), c_int(2), c_int(0), c_int(0), c_void_p(gate.data_ptr()),
            c_int(gate.stride(0)), c_void_p(out.data_ptr()), c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 1 and "Hkv" in L.pk_gqa_decode_static_error().decode()
    torch.cuda.synchronize()
    assert (out == 7.0).all()
