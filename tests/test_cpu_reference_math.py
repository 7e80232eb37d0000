"""Native host reference math of the DeepSeek-V4 block glue against the Python definitions; CPU dot microbenchmark."""
import ctypes
import subprocess
from pathlib import Path

import pytest
import torch

from pocketllm_b200.models import deepseek_v4 as d4
from pocketllm_b200.ops import lib

ROOT = Path(__file__).resolve().parent.parent


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.fixture(scope="module")
def cpu():
    if not lib.available("cpu"):
        pytest.skip("libpocket_cpu.so not built")
    return lib.cpu()


def test_hyper_connection_mixes_match_python(cpu):
    cfg = d4.DSV4Config.tiny()
    g = torch.Generator().manual_seed(0)
    T, hc, dim = 5, cfg.hc_mult, 96
    h = torch.randn(T, hc, dim, generator=g)
    fn = torch.randn((2 + hc) * hc, hc * dim, generator=g) * 0.05
    scale, base = torch.rand(3, generator=g) + 0.5, torch.randn((2 + hc) * hc, generator=g) * 0.3
    x_ref, post_ref, comb_ref = d4.hc_pre(h, fn, scale, base, cfg)
    x, post, comb = torch.empty(T, dim), torch.empty(T, hc), torch.empty(T, hc, hc)
    rc = cpu.pk_cpu_hc_pre(_p(h), T, hc, dim, _p(fn), _p(scale), _p(base), cfg.hc_sinkhorn_iters, ctypes.c_float(cfg.hc_eps),
                           ctypes.c_float(cfg.norm_eps), _p(x), _p(post), _p(comb))
    assert rc == 0
    assert torch.allclose(x, x_ref, atol=2e-5, rtol=1e-4) and torch.allclose(post, post_ref, atol=1e-5) and torch.allclose(comb, comb_ref, atol=1e-5)
    assert torch.allclose(comb.sum(-2), torch.ones(T, hc), atol=1e-3)          # Sinkhorn: columns sum to one
    y = torch.randn(T, dim, generator=g)
    out = torch.empty(T, hc, dim)
    assert cpu.pk_cpu_hc_post(_p(y), _p(h), _p(post), _p(comb), T, hc, dim, _p(out)) == 0
    assert torch.allclose(out, d4.hc_post(y, h, post_ref, comb_ref), atol=2e-5, rtol=1e-4)
    hfn, hscale, hbase = torch.randn(hc, hc * dim, generator=g) * 0.05, torch.rand(1, generator=g) + 0.5, torch.randn(hc, generator=g) * 0.3
    xh = torch.empty(T, dim)
    assert cpu.pk_cpu_hc_head(_p(h), T, hc, dim, _p(hfn), _p(hscale), _p(hbase), ctypes.c_float(cfg.hc_eps), ctypes.c_float(cfg.norm_eps), _p(xh)) == 0
    assert torch.allclose(xh, d4.hc_head(h, hfn, hscale, hbase, cfg), atol=2e-5, rtol=1e-4)


def test_rmsnorm_and_bf16_matvec_match_python(cpu):
    g = torch.Generator().manual_seed(1)
    T, K, N = 3, 320, 70
    x = torch.randn(T, K, generator=g)
    gamma = 1 + torch.randn(K, generator=g) * 0.1
    y = torch.empty(T, K)
    assert cpu.pk_cpu_rmsnorm(_p(x), T, K, _p(gamma), ctypes.c_float(1e-6), _p(y)) == 0
    assert torch.allclose(y, d4.rmsnorm(x, gamma, 1e-6), atol=1e-5, rtol=1e-5)
    assert cpu.pk_cpu_rmsnorm(_p(x), T, K, None, ctypes.c_float(1e-6), _p(y)) == 0
    assert torch.allclose(y, d4.rmsnorm(x, None, 1e-6), atol=1e-5, rtol=1e-5)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    out = torch.empty(T, N)
    assert cpu.pk_cpu_bf16_matvec(_p(x), T, K, _p(w.view(torch.int16)), N, _p(out)) == 0
    assert torch.allclose(out, x @ w.float().T, atol=1e-4, rtol=1e-4)


def test_dot_microbench_runs():
    exe = ROOT / "pocketllm_b200" / "_C" / "dot_microbench"
    if not exe.exists():
        pytest.skip("dot_microbench not built")
    r = subprocess.run([str(exe), "--k", "512", "--rows", "64", "--iters", "2", "--threads", "2"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    lines = r.stdout.strip().splitlines()
    assert lines[0].startswith("check=dot_f32") and lines[0].endswith("ok=1")
    formats = {l.split("format=")[1].split()[0] for l in lines[1:]}
    assert formats == {"f32", "bf16", "int8", "fp4_e2m1"}
    assert subprocess.run([str(exe), "--k", "100"], capture_output=True).returncode == 2


def test_int8_routed_experts_match_dequantised_reference(cpu):
    """INT8 experts with one scale per weight row: the native loop against fp32 math on the dequantised weights."""
    g = torch.Generator().manual_seed(4)
    T, H, I, E, k = 6, 96, 64, 5, 2
    x = torch.randn(T, H, generator=g)
    w13, w2 = torch.randn(E, 2 * I, H, generator=g) * 0.05, torch.randn(E, H, I, generator=g) * 0.05
    q13, s13 = torch.empty(E, 2 * I, H, dtype=torch.int8), torch.empty(E, 2 * I)
    q2, s2 = torch.empty(E, H, I, dtype=torch.int8), torch.empty(E, H)
    cpu.pk_cpu_quantize_int8_rows(_p(w13), ctypes.c_long(E * 2 * I), H, _p(q13), _p(s13))
    cpu.pk_cpu_quantize_int8_rows(_p(w2), ctypes.c_long(E * H), I, _p(q2), _p(s2))
    d13, d2 = q13.float() * s13.unsqueeze(-1), q2.float() * s2.unsqueeze(-1)
    assert (d13 - w13).abs().max() <= s13.max() * 0.5 + 1e-7
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, k, generator=g)
    y, counts = torch.empty(T, H), torch.zeros(E, dtype=torch.int32)
    rc = cpu.pk_cpu_moe_int8_forward(_p(x), T, H, I, E, k, _p(ids), _p(wts), _p(q13), _p(s13), _p(q2), _p(s2), ctypes.c_float(7.0), _p(y), _p(counts))
    assert rc == 0
    ref = torch.zeros(T, H)
    for t in range(T):
        for j in range(k):
            e = int(ids[t, j])
            gate, up = d13[e, :I] @ x[t], d13[e, I:] @ x[t]
            ref[t] += wts[t, j] * (d2[e] @ d4.swiglu(gate, up, 7.0))
    assert torch.allclose(y, ref, atol=1e-4, rtol=1e-4)
    assert counts.tolist() == torch.bincount(ids.flatten().long(), minlength=E).tolist()
    bad = ids.clone()
    bad[0, 0] = E
    assert cpu.pk_cpu_moe_int8_forward(_p(x), T, H, I, E, k, _p(bad), _p(wts), _p(q13), _p(s13), _p(q2), _p(s2), ctypes.c_float(0.0), _p(y), None) == 2
