"""The bundled model configuration files parse through the Python config classes and the native parsers."""
import json
import subprocess
from pathlib import Path

import pytest

from pocketllm_b200 import configs

BINARY = Path(__file__).resolve().parent.parent / "pocketllm_b200" / "_C" / "pocket_engine"


def test_python_config_classes_read_the_files():
    q = configs.load("qwen3_8_27b_fp8")
    assert (q.num_hidden_layers, q.hidden_size, q.intermediate_size, q.vocab_size) == (64, 5120, 17408, 151936)
    assert q.layer_types.count("full_attention") == 16
    d = configs.load("deepseek_v4_flash")
    assert (d.n_layers, d.dim, d.n_routed_experts, d.n_activated_experts, len(d.compress_ratios)) == (43, 4096, 256, 6, 44)
    m = configs.load("minimax_m2")
    assert (m.n_layers, m.dim, m.n_experts, m.n_experts_used, m.expert_inter) == (62, 3072, 256, 8, 1536)
    g = configs.load("glm_5_dsa")
    assert (g.n_layers, g.dim, g.n_experts, g.top_k, g.dsa_topk) == (78, 6144, 256, 8, 2048)
    with pytest.raises(FileNotFoundError):
        configs.load("nope")


@pytest.mark.skipif(not BINARY.exists(), reason="pocket_engine is not built")
def test_native_parsers_read_the_files(tmp_path):
    out = subprocess.run([str(BINARY), "--dsv4-config", str(configs.path("deepseek_v4_flash")), "--tp-world", "8"], capture_output=True,
                         text=True, timeout=60)
    assert out.returncode == 0, out.stderr
    d = json.loads(out.stdout)
    assert d["n_layers"] == 43 and d["dim"] == 4096 and d["n_routed_experts"] == 256
    # the Qwen parser wants a checkpoint directory: config.json alone is enough for --dump-config
    ck = tmp_path / "ck"
    ck.mkdir()
    (ck / "config.json").write_text(configs.path("qwen3_8_27b_fp8").read_text())
    out = subprocess.run([str(BINARY), "--ckpt", str(ck), "--dump-config", "--tp-world", "8"], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stderr
    assert "64" in out.stdout and "5120" in out.stdout
