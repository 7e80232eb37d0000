"""TP1 and TP2 must produce the same greedy tokens on a toy checkpoint (needs 2 GPUs)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


PROMPT_SHORT = "5,17,300,44,9,1000,2,77,12"
PROMPT_LONG = ",".join(str((i * 37 + 11) % 1024) for i in range(100))   # 64 + 36 rows: tensor-core prefill


def _run(world: int, ckpt: Path, port: int, prompt: str = PROMPT_SHORT, extra: tuple = (), new: int = 10) -> dict:
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), "-m", "pocketllm_b200.parallel.tp_check", "--ckpt", str(ckpt), "--prompt",
           prompt, "--new", str(new), *extra]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
    return json.loads(line)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_matches_tp1(tmp_path):
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg = qh.QwenHybridConfig.tiny(layers=4, hidden=256, inter=512, vocab=1024)
    qh.save_checkpoint(tmp_path, cfg, qh.random_checkpoint(cfg, seed=2, sigma=0.05))
    one = _run(1, tmp_path, 29531)
    two = _run(2, tmp_path, 29532)
    assert two["ranks_agree"] and two["comm_status"] == [0, 0]
    assert one["tokens"] == two["tokens"]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_tensor_core_prefill_matches_tp1(tmp_path):
    """The GEMM epilogue pushes partial tiles to the peer; the next norm sums them."""
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg = qh.QwenHybridConfig.tiny(layers=4, hidden=256, inter=512, vocab=1024)
    qh.save_checkpoint(tmp_path, cfg, qh.random_checkpoint(cfg, seed=4, sigma=0.05))
    one = _run(1, tmp_path, 29533, PROMPT_LONG)
    two = _run(2, tmp_path, 29534, PROMPT_LONG)
    assert two["ranks_agree"] and two["comm_status"] == [0, 0]
    # partial sums are added in a different order: allow a late divergence, not an early one
    same = sum(1 for a, b in zip(one["tokens"], two["tokens"]) if a == b)
    assert one["tokens"][:3] == two["tokens"][:3] and same >= 6, (one["tokens"], two["tokens"])


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_mtp_speculative_decode_equals_plain(tmp_path):
    """The predictor's layer is sharded like the backbone's; drafts come out of the merged candidates, so every rank takes
    the same accept / rewind decisions and the speculative tokens equal the plain ones."""
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg = qh.QwenHybridConfig.tiny(layers=4, hidden=256, inter=512, vocab=1024)
    qh.save_checkpoint(tmp_path, cfg, qh.random_checkpoint(cfg, seed=6, sigma=0.05, mtp=True))
    two = _run(2, tmp_path, 29535, PROMPT_LONG, extra=("--mtp", "4"), new=24)
    assert two["ranks_agree"] and two["comm_status"] == [0, 0]
    assert two["spec_tokens"] == two["tokens"] and two["replay_tokens"] == two["tokens"]
    assert two["replay_stats"]["accepted"] == two["replay_stats"]["proposed"] > 0 and two["replay_stats"]["rollbacks"] == 0


def _wide_cfg():
    """Heads and widths that divide by eight, every per-rank K a multiple of 128 (so the native FP8 GEMM runs at every world)."""
    from pocketllm_b200.models import qwen_hybrid as qh
    return qh.QwenHybridConfig(vocab_size=2048, hidden_size=256, intermediate_size=1024, num_hidden_layers=4, num_attention_heads=8,
                               num_key_value_heads=8, linear_num_key_heads=8, linear_num_value_heads=8, max_position_embeddings=4096)


@pytest.mark.parametrize("world", [4, 8])
@pytest.mark.parametrize("prompt", ["short", "long"])
def test_tp4_tp8_tokens_and_prefill_logits_match_tp1(tmp_path, world, prompt):
    """The first 16 greedy tokens and the prefill logits of TP4 / TP8 against one rank: streaming prefill (short prompt)
    and the tensor-core prefill with reduce-scatter + all-gather (long prompt), both followed by the persistent decode."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg = _wide_cfg()
    qh.save_checkpoint(tmp_path, cfg, qh.random_checkpoint(cfg, seed=8, sigma=0.05))
    text = PROMPT_SHORT if prompt == "short" else PROMPT_LONG
    one = _run(1, tmp_path, 29541, text, new=16)
    many = _run(world, tmp_path, 29542 + world, text, new=16)
    assert many["ranks_agree"] and many["comm_status"] == [0] * world
    a, b = torch.tensor(one["prefill_logits_head"]), torch.tensor(many["prefill_logits_head"])
    assert ((a - b).norm() / a.norm()).item() < 3e-2
    assert abs(one["prefill_logits_norm"] - many["prefill_logits_norm"]) < 3e-2 * one["prefill_logits_norm"]
    assert one["prefill_logits_top"][0][0] in [i for i, _ in many["prefill_logits_top"][:3]]
    # partial sums are added in a different order: the picks may part ways on a near-tie, not early and not often
    same = sum(1 for x, y in zip(one["tokens"], many["tokens"]) if x == y)
    assert one["tokens"][:3] == many["tokens"][:3] and same >= 6, (one["tokens"], many["tokens"])


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_peer_wait_timeout_switches_the_engine_to_nccl(tmp_path):
    """Rank 0 runs a step that rank 1 never joins: bounded waits run out, the step raises, rank 0 moves to NCCL by itself,
    rank 1 follows on the host's word, and the next request comes out of the NCCL path with the same tokens."""
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg = qh.QwenHybridConfig.tiny(layers=4, hidden=256, inter=512, vocab=1024)
    qh.save_checkpoint(tmp_path, cfg, qh.random_checkpoint(cfg, seed=2, sigma=0.05))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29561",
           "-m", "pocketllm_b200.parallel.nccl_fallback_check", "--ckpt", str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr[-3000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    r0, r1 = res["ranks"]
    assert r0["peer_status"] == 0 and "bounded device wait ran out" in r0["error"] and "NCCL" in r0["error"]
    assert r0["switched_by_itself"] and not r1["switched_by_itself"] and r0["nccl_mode"] and r1["nccl_mode"]
    assert r0["status_after"] == 0 and r1["status_after"] == 0
    assert r0["nccl_tokens"] == r1["nccl_tokens"] and r0["peer_tokens"] == r1["peer_tokens"]
    same = sum(1 for a, b in zip(r0["peer_tokens"], r0["nccl_tokens"]) if a == b)
    assert r0["peer_tokens"][:3] == r0["nccl_tokens"][:3] and same >= 6, (r0["peer_tokens"], r0["nccl_tokens"])


def _nccl_smoke(world: int, tmp_path) -> list[str]:
    exe = ROOT / "pocketllm_b200" / "_C" / "pocket_engine"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([str(exe), "--nccl-smoke", "--tp-world", str(world), "--tp-rank", str(r), "--nccl-id-path", str(tmp_path / "id")],
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env) for r in range(world)]
    outs = []
    for p in procs:
        out, err = p.communicate(timeout=300)
        assert p.returncode == 0, out + err
        outs.append([l for l in out.splitlines() if l.startswith("nccl_smoke=1")][-1])
    return outs


def test_native_nccl_baseline_single_rank(tmp_path):
    """The NCCL path of the native side (library opened at run time): sum, broadcast, gather, global top-1."""
    (line,) = _nccl_smoke(1, tmp_path)
    assert "available=1" in line and "ok=1" in line and "sum=1.0" in line and "top1=1000" in line


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_native_nccl_baseline_two_ranks(tmp_path):
    lines = _nccl_smoke(2, tmp_path)
    assert all("ok=1" in l and "sum=3.0" in l and "broadcast=4242" in l and "top1=1001" in l for l in lines), lines
