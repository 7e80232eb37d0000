"""Qwen DSpark drafter: checkpoint layout and the fp32 definition (the native engine does not run this drafter yet)."""
import pytest
import torch

from pocketllm_b200.models import qwen_dspark as qd


def _setup(seed=0):
    cfg = qd.QwenDSparkConfig.tiny()
    W = qd.random_checkpoint(cfg, seed=seed)
    g = torch.Generator().manual_seed(seed + 1)
    embed = torch.randn(cfg.vocab_size, cfg.hidden_size, generator=g) * 0.05
    head = torch.randn(cfg.vocab_size, cfg.hidden_size, generator=g) * 0.05
    return cfg, W, qd.QwenDSparkOracle(cfg, W, embed, head), g


def test_checkpoint_layout():
    full = qd.QwenDSparkConfig()
    names = qd.tensor_names(full)
    assert len(names) == 62 and dict(names)["fc.weight"] == (5120, 5 * 5120)
    assert dict(names)["layers.4.self_attn.q_proj.weight"] == (40 * 128, 5120) and dict(names)["confidence_head.proj.weight"] == (1, 5120 + 256)
    full.validate_for_target(5120, 151936, 64)
    with pytest.raises(ValueError):
        full.validate_for_target(4096, 151936, 64)
    with pytest.raises(ValueError):
        full.validate_for_target(5120, 151936, 48)           # tap layer 52 does not exist
    cfg = qd.QwenDSparkConfig.tiny()
    W = qd.random_checkpoint(cfg)
    assert set(W) == {n for n, _ in qd.tensor_names(cfg)} and all(W[n].shape == s for n, s in qd.tensor_names(cfg))


def test_yarn_frequencies():
    cfg = qd.QwenDSparkConfig.tiny()
    plain = qd.yarn_inv_freq(cfg)
    assert plain.shape == (cfg.head_dim // 2,) and plain[0] == 1.0 and cfg.attention_factor() == 1.0
    cfg.rope_factor, cfg.rope_original_max_positions = 4.0, 64
    scaled = qd.yarn_inv_freq(cfg)
    assert torch.all(scaled <= plain + 1e-12) and torch.all(scaled >= plain / 4 - 1e-12)
    assert scaled[0] == plain[0] and abs(scaled[-1] - plain[-1] / 4) < 1e-12      # fast dims keep, slow dims are interpolated
    assert abs(cfg.attention_factor() - (0.1 * torch.log(torch.tensor(4.0)).item() + 1.0)) < 1e-9


def test_proposal_semantics():
    cfg, W, orc, g = _setup()
    taps = torch.randn(9, cfg.hidden_size * len(cfg.target_layer_ids), generator=g)
    orc.append_target_taps(taps[:5], 0)
    orc.append_target_taps(taps[5:], 5)
    with pytest.raises(ValueError):
        orc.append_target_taps(taps[:1], 4)                  # gaps and rewrites are refused
    toks, conf, logits = orc.propose(17)
    assert len(toks) == cfg.block_size and conf.shape == (cfg.block_size,) and ((conf > 0) & (conf < 1)).all()
    assert toks == [int(l.argmax()) for l in logits]
    assert orc.propose(17)[0] == toks and orc.committed == 9          # a proposal does not commit anything
    # chunked and one-shot context appends agree
    other = _setup()[2]
    other.append_target_taps(taps, 0)
    assert torch.allclose(other.propose(17)[2], logits, atol=1e-5)
    # no causal mask inside the block: the anchor row depends on nothing but the context and the block inputs, and the
    # block inputs after the anchor are mask tokens, so changing the mask embedding changes even the first row
    orc2 = _setup()[2]
    orc2.append_target_taps(taps, 0)
    orc2.embed[cfg.mask_token_id] += 1.0
    assert not torch.allclose(orc2.propose(17)[2][0], logits[0], atol=1e-4)
    # cropping the context rewinds the drafter
    orc.crop_context(5)
    assert orc.committed == 5
    orc.append_target_taps(taps[5:], 5)
    assert torch.allclose(orc.propose(17)[2], logits, atol=1e-5)
    # the Markov bias is applied row by row with the previous pick
    w1, w2 = W["markov_head.markov_w1.weight"].float(), W["markov_head.markov_w2.weight"].float()
    orc.W["markov_head.markov_w2.weight"] = torch.zeros_like(w2)
    base = orc.propose(17)[2]
    prev = 17
    for r in range(cfg.block_size):
        assert torch.allclose(logits[r], base[r] + w2 @ w1[prev], atol=1e-4)
        prev = toks[r]
