"""MiniMax-M2 on a tiny synthetic GGUF: raw-block GPU runtime vs the fp32 oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny_gguf(tmp_path_factory):
    from pocketllm_b200.models import minimax_m2 as mm
    p = tmp_path_factory.mktemp("mm") / "tiny.gguf"
    mm.write_random_gguf(p, mm.MiniMaxM2Config.tiny(), seed=0, sigma=0.05)
    return p


def test_forward_matches_oracle(tiny_gguf):
    from pocketllm_b200.models import minimax_m2 as mm
    ref = mm.ReferenceModel(tiny_gguf)
    model = mm.MiniMaxM2Model(tiny_gguf, max_context=128)
    prompt = [3, 77, 140, 9, 255, 31, 8, 500, 64, 2, 19]
    lr = ref.forward(prompt)[-1]
    lg = model.forward(torch.tensor(prompt, dtype=torch.int32, device="cuda")).cpu()
    assert ((lg - lr).norm() / lr.norm()) < 3e-2
    # one decode step after the prefill
    nxt = int(lr.argmax())
    lr2 = ref.forward([nxt])[-1]
    lg2 = model.forward(torch.tensor([nxt], dtype=torch.int32, device="cuda")).cpu()
    assert ((lg2 - lr2).norm() / lr2.norm()) < 3e-2


def test_generate_cli_runtime(tiny_gguf):
    from pocketllm_b200.models import registry
    from pocketllm_b200.runtime import generation as gen
    rt = registry.build_runtime(tiny_gguf, max_context=64)
    res = gen.greedy_generate(rt, [1, 2, 3, 4], 6)
    assert len(res.tokens) == 6 and res.prefill_seconds > 0 and res.decode_tps > 0
    assert res.result_line().startswith("RESULT prefill_seconds=")


def test_synthetic_full_shape_constructor_runs_small():
    """Random block payloads made on the device (constant block scales): the model runs and produces finite logits."""
    from pocketllm_b200.models import minimax_m2 as mm
    cfg = mm.MiniMaxM2Config(vocab_size=1024, dim=512, n_layers=2, n_heads=8, n_kv_heads=2, n_experts=16, n_experts_used=4, expert_inter=256)
    m = mm.MiniMaxM2Model.synthetic(cfg, max_context=96)
    logits = m.forward(torch.arange(40, dtype=torch.int32, device="cuda"))      # 40 rows: tensor-core linears
    assert logits.shape == (cfg.vocab_size,) and torch.isfinite(logits).all()
    tok = m.decode_one(int(logits.argmax()))
    assert 0 <= tok < cfg.vocab_size and m.pos == 41


def test_experts_staged_from_host_match_resident_experts(tiny_gguf):
    """Experts in pinned host memory with a few device slots per layer: same logits as the resident model, with real evictions."""
    from pocketllm_b200.models import minimax_m2 as mm
    full = mm.MiniMaxM2Model(tiny_gguf, max_context=128)
    slots = full.cfg.n_experts_used + 1
    staged = mm.MiniMaxM2Model(tiny_gguf, max_context=128, expert_slots=slots)
    assert all("cache" in L and "w13" not in L for L in staged.layers) and not staged.use_graph
    prompt = torch.tensor([3, 77, 140, 9, 255, 31, 8, 500, 64, 2, 19], dtype=torch.int32, device="cuda")
    a, b = full.forward(prompt), staged.forward(prompt)
    assert ((a - b).norm() / a.norm()).item() < 1e-2
    nxt = torch.tensor([int(a.argmax())], dtype=torch.int32, device="cuda")
    a2, b2 = full.forward(nxt), staged.forward(nxt)
    assert ((a2 - b2).norm() / a2.norm()).item() < 1e-2
    cache = staged.layers[0]["cache"]
    assert cache.slab["w13"].shape[0] == slots and cache.bytes_staged > 0 and cache.lru.stats["evictions"] > 0
