"""Drafter checkpoint directories of the external DSpark block drafter (config.json + Safetensors)."""
import torch


def test_drafter_checkpoint_directory_round_trip(tmp_path):
    import pytest
    from pocketllm_b200.models import qwen_dspark as qd
    cfg = qd.QwenDSparkConfig.tiny()
    W = qd.random_checkpoint(cfg, seed=3)
    qd.save_checkpoint(tmp_path, cfg, W)
    cfg2, W2 = qd.load_checkpoint(tmp_path)
    assert cfg2 == cfg and set(W2) == set(W)
    assert all(torch.equal(W2[k], W[k]) for k in W)
    # a missing tensor is reported by name
    W.pop("norm.weight")
    other = tmp_path / "broken"
    qd.save_checkpoint(other, cfg, W)
    with pytest.raises(ValueError, match="norm.weight"):
        qd.load_checkpoint(other)
