"""The RMSNorm kernel that quantises its output rows for the native FP8 GEMM in the same pass (`ops.rmsnorm_quant`)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("terms", [1, 2])
@pytest.mark.parametrize("M,K", [(512, 5120), (77, 1024), (1, 128), (300, 2176)])
def test_rmsnorm_quant_equals_norm_then_quantise(M, K, terms):
    """The norm kernel that quantises on the way out: its bf16 rows follow the fp32 definition and equal the plain norm
    kernel's, and its codes and scales are exactly what the quantiser makes of those rows."""
    from pocketllm_b200 import ops
    torch.manual_seed(M + K + terms)
    x = (torch.randn(M, K, device="cuda") * 1.7).to(torch.bfloat16)
    gamma = torch.randn(K, device="cuda") * 0.2
    y, q, sc = ops.rmsnorm_quant(x, gamma, mode=1, eps=1e-6, terms=terms)
    xf = x.float()
    want = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + 1e-6) * (1 + gamma)
    assert _rel_err(y, want) < 5e-3
    # the two norm kernels add the squares in different orders: rows may differ by a bf16 rounding step here and there
    assert _rel_err(y, ops.rmsnorm(x, gamma, mode=1, eps=1e-6)) < 1e-3
    q_ref, sc_ref = ops.quant_act_fp8(y, terms)
    assert q.shape == q_ref.shape and sc.shape == sc_ref.shape
    assert torch.equal(q, q_ref) and torch.equal(sc, sc_ref)
    y2, _, _ = ops.rmsnorm_quant(x, gamma, mode=2, eps=1e-6, terms=terms)
    assert _rel_err(y2, ops.rmsnorm(x, gamma, mode=2, eps=1e-6)) < 1e-3
