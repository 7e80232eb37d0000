"""The CPU FP4 MoE block: native oracle vs dequantised fp32 PyTorch, and token counts."""
import pytest
import torch

from pocketllm_b200.formats import fp4
from pocketllm_b200.ops import lib

pytestmark = pytest.mark.skipif(not lib.available("cpu"), reason="libpocket_cpu.so not built")


def test_fp4_roundtrip():
    torch.manual_seed(0)
    w = torch.randn(4, 256) * 0.02
    q, s = fp4.quantize_e2m1(w)
    assert q.shape == (4, 128) and s.shape == (4, 8) and q.dtype == torch.uint8
    back = fp4.dequantize_e2m1(q, s)
    assert ((back - w).norm() / w.norm()) < 0.2
    # codes decode to the value table times a power of two
    q2, s2 = fp4.quantize_e2m1(back)
    assert torch.equal(fp4.dequantize_e2m1(q2, s2), back)


def test_benchmark_block_parity_and_counts():
    from pocketllm_b200.moe import cpu_oracle as co
    w = co.random_fp4_moe(hidden=1024, inter=512, experts=8, shared=True, seed=0)
    torch.manual_seed(0)
    x = torch.randn(16, 1024).to(torch.bfloat16)
    y_ref, counts_ref = co.forward_torch(x, w, topk=2)
    y, counts, secs = co.forward_native(x, w, topk=2)
    assert counts.tolist() == counts_ref.tolist() and int(counts.sum()) == 32
    assert ((y - y_ref).norm() / y_ref.norm()) < 1e-4
    assert secs > 0


@pytest.mark.parametrize("score,norm", [("sigmoid", True), ("sqrtsoftplus", True), ("softmax", False)])
def test_routing_variants(score, norm):
    from pocketllm_b200.moe import cpu_oracle as co
    w = co.random_fp4_moe(hidden=256, inter=64, experts=16, shared=False, seed=3)
    w.bias = torch.randn(16) * 0.01
    x = torch.randn(5, 256)
    y_ref, c_ref = co.forward_torch(x, w, topk=4, score_func=score, norm_topk=norm, route_scale=1.5)
    y, c, _ = co.forward_native(x, w, topk=4, score_func=score, norm_topk=norm, route_scale=1.5)
    assert c.tolist() == c_ref.tolist()
    assert ((y - y_ref).norm() / y_ref.norm()) < 1e-4
