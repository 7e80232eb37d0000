"""Checkpoint tools of the native CLI that need no GPU: `--qwen-audit` (every tensor the engine reads, with dtype,
shape and shard-cut checks) and `--inspect-tensor`, on a tiny hybrid checkpoint written by the Python side."""
import subprocess
from pathlib import Path

import pytest
import torch

from pocketllm_b200.models import qwen_hybrid as qh

ROOT = Path(__file__).resolve().parent.parent
ENGINE = ROOT / "pocketllm_b200" / "_C" / "pocket_engine"


def _run(*args):
    r = subprocess.run([str(ENGINE), *map(str, args)], capture_output=True, text=True, timeout=120)
    return r.returncode, r.stdout + r.stderr


def _fields(text, key):
    line = [l for l in text.splitlines() if l.startswith(key + "=")][-1]
    return dict(part.partition("=")[::2] for part in line.split())


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    if not ENGINE.exists():
        pytest.skip("native engine binary not built")
    cfg = qh.QwenHybridConfig.tiny()
    W = qh.random_checkpoint(cfg, seed=3, mtp=True)
    d = tmp_path_factory.mktemp("qwen_tools")
    qh.save_checkpoint(d / "good", cfg, W)
    return cfg, W, d


def test_audit_accepts_a_complete_checkpoint_and_counts_its_tensors(ckpt):
    cfg, W, d = ckpt
    rc, out = _run("--ckpt", d / "good", "--qwen-audit", "--qwen-mtp")
    f = _fields(out, "qwen_audit")
    assert rc == 0 and f["ok"] == "1" and f["problems"] == "0" and f["unused_tensors"] == "0", out
    assert int(f["expected_tensors"]) == len(W) and int(f["layers"]) == cfg.num_hidden_layers
    # without the predictor its tensors are simply unused
    rc, out = _run("--ckpt", d / "good", "--qwen-audit")
    f = _fields(out, "qwen_audit")
    assert rc == 0 and int(f["unused_tensors"]) == sum(1 for n in W if n.startswith("mtp."))
    # two ranks cut every FP8 linear on its 128-wide scale blocks at this size
    rc, out = _run("--ckpt", d / "good", "--qwen-audit", "--tp-world", "2")
    assert rc == 0, out


def test_audit_names_what_is_wrong(ckpt):
    cfg, W, d = ckpt
    bad = dict(W)
    gone = next(n for n in bad if n.endswith("layers.1.mlp.down_proj.weight_scale_inv"))
    del bad[gone]
    wrong = next(n for n in bad if n.endswith("layers.0.input_layernorm.weight"))
    bad[wrong] = torch.zeros(cfg.hidden_size + 1, dtype=torch.bfloat16)
    bad["model.language_model.extra.weight"] = torch.zeros(4, dtype=torch.bfloat16)
    qh.save_checkpoint(d / "bad", cfg, bad)
    rc, out = _run("--ckpt", d / "bad", "--qwen-audit")
    assert rc == 1
    assert f"qwen_audit_problem=missing {gone}" in out
    assert f"qwen_audit_problem=shape {wrong}" in out
    assert "qwen_audit_unused=model.language_model.extra.weight" in out
    assert _fields(out, "qwen_audit")["ok"] == "0"
    # four ranks: 64-row shares do not fall on the scale blocks (or the config refuses the split outright)
    rc, out = _run("--ckpt", d / "good", "--qwen-audit", "--tp-world", "4")
    assert rc == 1 and "qwen_audit_problem=" in out


def test_inspect_tensor_prints_dtype_shape_and_values(ckpt):
    cfg, W, d = ckpt
    name = next(n for n in W if n.endswith("layers.0.input_layernorm.weight"))
    rc, out = _run("--ckpt", d / "good", "--inspect-tensor", name)
    f = _fields(out, "tensor")
    assert rc == 0 and f["found"] == "1" and f["dtype"].upper() == "BF16" and f["shape"] == f"[{cfg.hidden_size}]"
    first = [float(v) for v in f["first"].strip("[]").split(",")]
    assert first == pytest.approx(W[name].float()[:8].tolist())
    assert float(f["sum"]) == pytest.approx(W[name].float().sum().item(), rel=1e-5, abs=1e-5)
    fp8 = next(n for n in W if n.endswith("layers.0.mlp.gate_proj.weight"))
    rc, out = _run("--ckpt", d / "good", "--inspect-tensor", fp8)
    f = _fields(out, "tensor")
    first = [float(v) for v in f["first"].strip("[]").split(",")]
    assert rc == 0 and first == pytest.approx(W[fp8].float().flatten()[:8].tolist())
    rc, out = _run("--ckpt", d / "good", "--inspect-tensor", "no.such.tensor")
    assert rc == 1 and "found=0" in out


def test_flags_of_other_engines_answer_with_a_pointer(ckpt):
    _, _, d = ckpt
    rc, out = _run("--ckpt", d / "good", "--qwen-dspark", "/nowhere")
    assert rc == 1 and "pocketllm_b200.server.openai" in out
    rc, out = _run("--ckpt", d / "good", "--forward-token", "5")
    assert rc == 1 and "--token-ids" in out
