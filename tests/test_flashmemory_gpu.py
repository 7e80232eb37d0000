"""Chunk scorer of the long-context retriever against its fp32 definition (the reference tests the same path with a
fixture exported from its retriever: cpp_engine/tests/test_flashmemory_scorer.cpp)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _weights(heads=64, rank=384, hidden=1024, rope_dim=64, seed=0):
    from pocketllm_b200.ops import flashmemory as fm
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s, sd: (torch.randn(*s, generator=g) * sd).cuda()
    return fm.ScorerWeights(wq_a=mk(rank, hidden, sd=hidden ** -0.5), wq_b=mk(heads * 128, rank, sd=rank ** -0.5),
                            q_norm=(1 + 0.1 * torch.randn(rank, generator=g)).cuda(), weights_proj=mk(heads, hidden, sd=hidden ** -0.5),
                            inv_freqs=fm.yarn_inv_freqs(rope_dim, 160000.0, 16.0, 65536, 32.0, 1.0).cuda(), eps=1e-6)


@pytest.mark.parametrize("heads,n_chunks,position", [(64, 5000, 123456), (128, 300, 7), (16, 129, 1_000_000)])
def test_scorer_matches_fp32_definition(heads, n_chunks, position):
    from pocketllm_b200.ops import flashmemory as fm
    torch.manual_seed(heads + n_chunks)
    w = _weights(heads=heads)
    hidden = torch.randn(1024, device="cuda")
    keys = torch.randn(n_chunks, 128, device="cuda") * torch.rand(n_chunks, 1, device="cuda") * 3
    codes, scale = fm.quantize_keys(keys)
    deq = codes.view(torch.float8_e4m3fn).float() * scale[:, None]
    assert torch.allclose(scale, keys.abs().amax(-1) / 448.0, rtol=1e-6) and ((deq - keys).norm() / keys.norm()).item() < 4e-2
    # query side
    qcodes, head_w, q = fm.build_query(w, hidden, position, want_q=True)
    q_ref, hw_ref = fm.reference_query(w, hidden, position)
    assert ((q - q_ref).norm() / q_ref.norm()).item() < 1e-2           # bf16 rounding points may flip on the last bit
    planes = qcodes.view(torch.float8_e4m3fn).float()
    assert planes[heads:128].abs().sum() == 0 and planes[128 + heads:].abs().sum() == 0
    # scores against the definition evaluated on the dequantised keys (what the cache holds)
    for sig in (False, True):
        got = fm.score_chunks(codes, scale, qcodes, head_w, sigmoid=sig)
        want = fm.reference_scores(w, hidden, deq, position, sigmoid=sig)
        assert ((got - want).norm() / want.norm()).item() < 1.5e-2
    # layer call = the two steps
    assert torch.equal(fm.score_layer(w, hidden, codes, scale, position), fm.score_chunks(codes, scale, qcodes, head_w))


def test_packed_keys_ensemble_topk_and_offsets():
    from pocketllm_b200.ops import flashmemory as fm
    torch.manual_seed(3)
    n = 777
    keys = torch.randn(n, 128, device="cuda")
    codes, scale = fm.quantize_keys(keys)
    packed = torch.cat([codes, scale.view(torch.uint8).view(n, 4)], 1)         # the reference's row layout
    c2, s2 = fm.unpack_keys(packed)
    assert torch.equal(c2, codes) and torch.equal(s2, scale)
    layers = torch.rand(3, 1024, device="cuda")
    assert torch.equal(fm.ensemble(layers, n, use_max=True), layers[:, :n].amax(0))
    assert torch.allclose(fm.ensemble(layers, n, use_max=False), layers[:, :n].mean(0), rtol=1e-6)
    ens = fm.ensemble(layers, n)
    idx, val = fm.topk(ens, 50)
    want = torch.topk(ens, 50)
    assert torch.equal(val, want.values) and set(idx.tolist()) == set(want.indices.tolist())
    phys = fm.write_global_indices(torch.cat([idx, torch.full((3,), -1, device="cuda", dtype=torch.int32)]), 128)
    assert torch.equal(phys[:50], idx + 128) and (phys[50:] == -1).all()


def test_yarn_frequencies():
    from pocketllm_b200.ops import flashmemory as fm
    plain = fm.yarn_inv_freqs(64, 10000.0, 1.0, 0, 32, 1)
    assert torch.allclose(plain, 1.0 / (10000.0 ** (torch.arange(0, 64, 2).float() / 64)))
    y = fm.yarn_inv_freqs(64, 10000.0, 16.0, 4096, 32, 1)
    assert torch.allclose(y[0], plain[0]) and torch.allclose(y[-1], plain[-1] / 16) and (y <= plain + 1e-12).all()


def test_retrieval_attention_chain_scores_selects_swaps_and_attends(capsys):
    """The whole long-context chain (three scorer layers -> ensemble -> top-k -> KV swap -> sparse attention over window +
    slots) gives exactly the attention over a fully resident cache, while only the slots live on the device."""
    import json
    from pocketllm_b200.cli import flashmemory_kv_swap as demo
    assert demo.main(["--context", "8192", "--gpu-chunks", "320", "--keep", "256", "--steps", "6", "--heads", "16", "--hidden", "1024",
                      "--q-lora-rank", "256", "--check"]) == 0
    res = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert res["max_abs_diff_vs_resident"] == 0.0
    assert res["kv_swap"]["misses"] >= 256 and res["kv_swap"]["hits"] + res["kv_swap"]["misses"] == 6 * 256
    assert res["kv_swap"]["device_mib"] < res["resident_cache_mib"]
