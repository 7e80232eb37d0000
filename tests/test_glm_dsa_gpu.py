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
