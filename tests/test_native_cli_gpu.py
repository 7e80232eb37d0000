"""Run modes of the native CLI that need a GPU: `--smoke-forward`, `--generate-token`, `--resident-bench`."""
import subprocess
from pathlib import Path

import pytest
import torch

from pocketllm_b200.models import qwen_hybrid as qh

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
ENGINE = ROOT / "pocketllm_b200" / "_C" / "pocket_engine"


def _run(*args):
    r = subprocess.run([str(ENGINE), *map(str, args)], capture_output=True, text=True, timeout=300)
    return r.returncode, r.stdout + r.stderr


def _fields(line):
    return dict(part.partition("=")[::2] for part in line.split())


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    if not ENGINE.exists():
        pytest.skip("native engine binary not built")
    cfg = qh.QwenHybridConfig.tiny()
    d = tmp_path_factory.mktemp("qwen_cli") / "ck"
    qh.save_checkpoint(d, cfg, qh.random_checkpoint(cfg, seed=5))
    return d


def test_smoke_forward_runs_the_first_layers_with_random_weights(ckpt):
    rc, out = _run("--ckpt", ckpt, "--smoke-forward", "--smoke-layers", "2", "--max-context", "256")
    line = [l for l in out.splitlines() if l.startswith("smoke_forward=")][-1]
    f = _fields(line)
    assert rc == 0 and f["ok"] == "1" and f["layers"] == "2" and len(f["generated_token_ids"].split(",")) == 3, out


def test_generate_token_and_resident_bench(ckpt):
    rc, out = _run("--ckpt", ckpt, "--token-ids", "1,2,3,4,5", "--generate-token", "--max-context", "256")
    one = _fields([l for l in out.splitlines() if l.startswith("qwen_runtime=")][-1])
    assert rc == 0 and one["generated_tokens"] == "1", out
    rc, out = _run("--ckpt", ckpt, "--token-ids", "1,2,3,4,5", "--max-new-tokens", "6", "--resident-bench", "3", "--max-context", "256")
    runs = [_fields(l) for l in out.splitlines() if l.startswith("qwen_resident_run=")]
    summary = _fields([l for l in out.splitlines() if l.startswith("qwen_resident_bench=")][-1])
    assert rc == 0 and len(runs) == 3 and summary["runs"] == "3" and summary["comm_status"] == "0", out
    assert len({r["generated_token_ids"] for r in runs}) == 1                 # a resident engine repeats itself
    assert runs[0]["generated_token_ids"].split(",")[0] == one["generated_token_ids"]
    assert float(summary["decode_tokens_per_s_mean"]) > 0
