"""External DSpark drafter of the Qwen hybrid model on the GPU: runtime against the fp32 definition, the engine's target
taps against the oracle's per-layer residual stream, and the speculative loop against plain greedy decode."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _drafter_cfg(vocab=1024, target_layers=4):
    from pocketllm_b200.models.qwen_dspark import QwenDSparkConfig
    return QwenDSparkConfig(hidden_size=256, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1, head_dim=128,
                            vocab_size=vocab, block_size=4, markov_rank=64, mask_token_id=vocab - 1, target_layer_ids=(1, target_layers - 1),
                            rope_theta=10000.0, rope_factor=4.0, rope_original_max_positions=64)


def test_runtime_matches_the_fp32_definition():
    from pocketllm_b200.models import qwen_dspark as qd
    from pocketllm_b200.models.qwen_dspark_runtime import QwenDSparkRuntime
    cfg = _drafter_cfg()
    W = qd.random_checkpoint(cfg, seed=1)
    g = torch.Generator().manual_seed(2)
    embed = (torch.randn(cfg.vocab_size, cfg.hidden_size, generator=g) * 0.5).to(torch.bfloat16)
    lm_head = (torch.randn(cfg.vocab_size, cfg.hidden_size, generator=g) * 0.05).to(torch.bfloat16)
    oracle = qd.QwenDSparkOracle(cfg, W, embed, lm_head)
    rt = QwenDSparkRuntime(cfg, W, embed, lm_head, max_context=256)
    taps = (torch.randn(23, 2 * cfg.hidden_size, generator=g) * 0.5).to(torch.bfloat16)
    oracle.append_target_taps(taps[:20], 0)
    rt.append_target_taps(taps[:20].cuda(), 0)
    for anchor in (5, 700):
        want_tok, want_conf, want_logits = oracle.propose(anchor)
        tok, conf, logits = rt.propose(anchor)
        rel = ((logits.cpu() - want_logits).norm() / want_logits.norm()).item()
        assert rel < 3e-2, rel
        assert (conf.cpu() - want_conf).abs().max().item() < 3e-2
        # a row's pick feeds the next row's bias: compare until the first near-tie
        for r, (a, b) in enumerate(zip(tok.tolist(), want_tok)):
            top2 = want_logits[r].topk(2).values
            if (top2[0] - top2[1]).item() < 0.05 * want_logits[r].abs().max().item():
                break
            assert a == b, (r, tok.tolist(), want_tok)
        # rejected suffix: crop three rows, append other rows in their place
        oracle.crop_context(17)
        rt.crop_context(17)
        oracle.append_target_taps(taps[20:23], 17)
        rt.append_target_taps(taps[20:23].cuda(), 17)
    with pytest.raises(ValueError, match="position order"):
        rt.append_target_taps(taps[:2].cuda(), 3)


def _target(tmp_path):
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg = qh.QwenHybridConfig.tiny(layers=4, hidden=256, inter=512, vocab=1024)
    tensors = qh.random_checkpoint(cfg, seed=1, sigma=0.05)
    qh.save_checkpoint(tmp_path, cfg, tensors)
    return cfg, tensors


def test_engine_taps_are_the_residual_stream_after_the_tap_layers(tmp_path):
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg, tensors = _target(tmp_path)
    ref = qh.ReferenceModel(cfg, tensors)
    prompt = [5, 17, 300, 44, 9, 1000, 2, 77, 12, 640, 3, 8, 100, 200, 301, 55, 6, 90]
    want = []
    for t in prompt:
        ref.step(t)
        want.append(torch.cat([ref.layer_hidden[1], ref.layer_hidden[3]]))
    want = torch.stack(want)
    eng = qh.QwenEngine(cfg, max_context=256, prefill_chunk=64).load(tmp_path)
    eng.set_tap_layers([1, 3])
    first = eng.prefill(prompt)                        # 18 rows: tensor-core chunk path
    taps = eng.taps().float().cpu()
    assert taps.shape == (18, 512) and ((taps - want).norm() / want.norm()).item() < 2e-2
    ref.step(first)
    eng.decode(1)                                      # one launch per projection while taps are on
    assert not eng.persistent_decode
    row = eng.taps().float().cpu()[0]
    w1 = torch.cat([ref.layer_hidden[1], ref.layer_hidden[3]])
    assert ((row - w1).norm() / w1.norm()).item() < 3e-2
    eng.reset()
    eng.prefill(prompt[:6])                            # 6 rows: streaming path
    t6 = eng.taps().float().cpu()
    assert ((t6 - want[:6]).norm() / want[:6].norm()).item() < 2e-2
    eng.close()


def test_speculative_generation_with_the_block_drafter_equals_greedy(tmp_path):
    from pocketllm_b200.models import qwen_dspark as qd
    from pocketllm_b200.models import qwen_hybrid as qh
    from pocketllm_b200.models.qwen_dspark_runtime import QwenDSparkRuntime, QwenDSparkSpeculator
    cfg, tensors = _target(tmp_path)
    dcfg = _drafter_cfg()
    dcfg.validate_for_target(cfg.hidden_size, cfg.vocab_size, cfg.num_hidden_layers)
    W = qd.random_checkpoint(dcfg, seed=4)
    pre = "model.language_model."
    embed, lm_head = tensors[pre + "embed_tokens.weight"], tensors.get("lm_head.weight", tensors[pre + "embed_tokens.weight"])
    torch.manual_seed(5)
    prompt = torch.randint(0, cfg.vocab_size - 1, (70,)).tolist()
    eng = qh.QwenEngine(cfg, max_context=512, prefill_chunk=32, persistent_decode=0).load(tmp_path)
    plain = eng.generate(prompt, 40)
    spec = QwenDSparkSpeculator(eng, QwenDSparkRuntime(dcfg, W, embed, lm_head, max_context=512))
    got = spec.generate(prompt, 40)
    assert got == plain
    assert spec.stats["rounds"] > 0 and spec.stats["proposed"] >= spec.stats["accepted"] >= 0
    eng.close()


def test_server_backend_with_drafter_streams_the_greedy_tokens(tmp_path):
    """`--qwen-dspark DIR` of the Python server: the Qwen backend runs greedy requests as block-drafted speculative rounds
    and yields exactly the plain backend's tokens."""
    from pocketllm_b200.models import qwen_dspark as qd
    from pocketllm_b200.models import qwen_hybrid as qh
    from pocketllm_b200.models.qwen_dspark_runtime import QwenDSparkRuntime, QwenDSparkSpeculator
    from pocketllm_b200.server.backends import QwenBackend
    from pocketllm_b200.server.engine import SamplingParams
    cfg, tensors = _target(tmp_path)
    dcfg = _drafter_cfg()
    ddir = tmp_path / "drafter"
    qd.save_checkpoint(ddir, dcfg, qd.random_checkpoint(dcfg, seed=9))
    dcfg2, dw = qd.load_checkpoint(ddir)
    pre = "model.language_model."
    embed, lm_head = tensors[pre + "embed_tokens.weight"], tensors["lm_head.weight"]
    torch.manual_seed(6)
    prompt = torch.randint(0, cfg.vocab_size - 1, (45,)).tolist()
    eng = qh.QwenEngine(cfg, max_context=512, prefill_chunk=32, persistent_decode=0).load(tmp_path)
    params = SamplingParams(max_tokens=30, temperature=0.0)
    plain = list(QwenBackend(eng).generate(prompt, params))
    spec = QwenDSparkSpeculator(eng, QwenDSparkRuntime(dcfg2, dw, embed, lm_head, max_context=512))
    drafted = list(QwenBackend(eng, speculator=spec).generate(prompt, params))
    assert drafted == plain and len(plain) == 30
    eng.close()
