"""GLM-DSA on a tiny synthetic GGUF: raw-block GPU runtime vs the fp32 oracle, with the
DSA indexer on (top-k smaller than the context) and off (dense attention)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny_gguf(tmp_path_factory):
    from pocketllm_b200.models import glm_dsa as glm
    p = tmp_path_factory.mktemp("glm") / "tiny.gguf"
    glm.write_random_gguf(p, glm.GLMDSAConfig.tiny(), seed=0)
    return p


@pytest.mark.parametrize("topk", [0, 8])
def test_forward_matches_oracle(tiny_gguf, topk):
    from pocketllm_b200.models import glm_dsa as glm
    ref = glm.ReferenceModel(tiny_gguf, dsa_topk=topk)
    model = glm.GLMDSAModel(tiny_gguf, max_context=128, dsa_topk=topk)
    prompt = [3, 77, 140, 9, 255, 31, 8, 500, 64, 2, 19, 33, 21, 400]
    lr = ref.forward(prompt)
    lg = model.forward(prompt).cpu()
    assert ((lg - lr).norm() / lr.norm()) < 4e-2
    nxt = int(lr.argmax())
    lr2, lg2 = ref.forward([nxt]), model.forward([nxt]).cpu()
    assert ((lg2 - lr2).norm() / lr2.norm()) < 4e-2


def test_indexer_selects_topk_causal():
    from pocketllm_b200.models import glm_dsa as glm
    torch.manual_seed(0)
    T, S, Hi, D = 5, 12, 3, 16
    qi, ki, wh = torch.randn(T, Hi, D), torch.randn(S, D), torch.rand(T, Hi)
    pos = torch.arange(S - T, S)
    m = glm.indexer_select(qi, ki, wh, pos, 4)
    assert m.shape == (T, S) and (m.sum(-1) == 4).all()
    assert not m[0, int(pos[0]) + 1:].any()                     # causal
    score = (torch.relu(torch.einsum("thd,sd->ths", qi, ki)) * wh[:, :, None]).sum(1)
    t = 2
    allowed = score[t, : int(pos[t]) + 1]
    assert set(m[t].nonzero().flatten().tolist()) == set(torch.topk(allowed, 4).indices.tolist())


@pytest.mark.parametrize("mode", ["routed_tp", "expert_parallel"])
def test_two_rank_expert_sharding_adds_up_to_one_rank(tmp_path, mode):
    """Routed TP (every rank holds all experts but a block-aligned slice of the intermediate dimension) and expert
    parallelism (whole experts per rank): the ranks' partial MoE outputs add up to the one-rank output. The two ranks are
    two runtime objects in one process; the cross-rank sum is done here."""
    import dataclasses
    from pocketllm_b200.models import glm_dsa as glm
    cfg = dataclasses.replace(glm.GLMDSAConfig.tiny(), expert_inter=512)
    path = tmp_path / "glm.gguf"
    glm.write_random_gguf(path, cfg, seed=3)
    one = glm.GLMDSAModel(path, max_context=64)
    ranks = [glm.GLMDSAModel(path, max_context=64, rank=r, world=2, routed_tp=mode == "routed_tp") for r in range(2)]
    for m in ranks:
        m._combine = lambda y: y                                     # the sum over ranks happens below
        assert m.routed_tp == (mode == "routed_tp")
        assert m.inter_local == (256 if mode == "routed_tp" else 512) and m.e_local == (cfg.n_experts if mode == "routed_tp" else cfg.n_experts // 2)
    torch.manual_seed(0)
    layer = cfg.leading_dense_layers
    for T in (3, 70):                                                # per-route kernels and the grouped tensor-core path
        x = torch.randn(T, cfg.dim, device="cuda")
        want = one.moe(layer, x)
        got = ranks[0].moe(layer, x) + ranks[1].moe(layer, x)
        assert ((got - want).norm() / want.norm()).item() < (2e-5 if T == 3 else 6e-3)


def test_experts_staged_from_host_match_resident_experts(tiny_gguf):
    """`expert_slots`: routed experts in pinned host memory, a few device slots per layer, staged per step (and in waves
    when a chunk needs more distinct experts than there are slots): same logits as the resident model."""
    from pocketllm_b200.models import glm_dsa as glm
    full = glm.GLMDSAModel(tiny_gguf, max_context=128, dsa_topk=8)
    slots = full.cfg.top_k + 1
    staged = glm.GLMDSAModel(tiny_gguf, max_context=128, dsa_topk=8, expert_slots=slots)
    assert staged.expert_slots == slots and len(staged.staging) == full.cfg.n_layers - full.cfg.leading_dense_layers
    prompt = [3, 77, 140, 9, 255, 31, 8, 500, 64, 2, 19, 33, 21, 400]
    a, b = full.forward(prompt), staged.forward(prompt)
    assert ((a - b).norm() / a.norm()).item() < 1e-2
    nxt = int(a.argmax())
    a2, b2 = full.forward([nxt]), staged.forward([nxt])
    assert ((a2 - b2).norm() / a2.norm()).item() < 1e-2
    cache = next(iter(staged.staging.values()))
    assert cache.bytes_staged > 0 and cache.lru.stats["evictions"] > 0
    # a budget that holds everything plans no staging at all
    roomy = glm.GLMDSAModel(tiny_gguf, max_context=128, dsa_topk=8, gpu_memory_gib=64.0)
    assert roomy.expert_slots is None and not roomy.staging
