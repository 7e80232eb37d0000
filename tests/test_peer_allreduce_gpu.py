"""Peer-memory all-reduce: bounded wait on one GPU, agreement with NCCL on two."""
import json
import os
import subprocess
import sys
import time
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_wait_runs_out_and_context_stays_usable():
    """A context whose 'peers' never publish: the wait gives up after its budget, the status word says so,
    and the same context works again for a world of one."""
    from pocketllm_b200.parallel.peer_allreduce import PeerAllReduce
    par = PeerAllReduce(1024, timeout_us=200_000, _solo_world=2)      # rank 0 of 2; nobody plays rank 1
    x = torch.ones(1024, device="cuda")
    t0 = time.perf_counter()
    par.all_reduce(x.clone())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert 0.15 < dt < 5.0
    assert par.status() == 1
    with pytest.raises(TimeoutError):
        par.check()
    assert par.status() == 0
    par.close()
    solo = PeerAllReduce(1024, _solo_world=1)
    y = solo.all_reduce(torch.arange(1000, device="cuda", dtype=torch.float32))
    assert torch.equal(y, torch.arange(1000, device="cuda", dtype=torch.float32)) and solo.status() == 0
    z = solo.all_reduce(torch.full((7,), 2.5, device="cuda"))          # odd length: scalar tail
    assert torch.equal(z, torch.full((7,), 2.5, device="cuda"))
    solo.close()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_matches_nccl_on_two_gpus():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29551",
           "-m", "pocketllm_b200.parallel.par_check", "--sizes", "1001,4096,262144", "--iters", "20"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr[-3000:]
    out = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert out["status"] == 0 and max(out["max_abs_err"]) < 1e-5


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_multimem_all_reduce_matches_nccl_on_two_gpus():
    """The in-switch all-reduce (multimem.ld_reduce, and multimem.st for the two-shot form) against NCCL; skipped where
    the machine offers no multicast mapping. No rank leaves early here: every rank runs to the final barrier."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29553",
           "-m", "pocketllm_b200.parallel.par_check", "--sizes", "1001,4096,262144", "--iters", "20", "--multimem"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr[-3000:]
    out = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    if out["multimem"] != "ok":
        pytest.skip(out["multimem"])
    assert out["status"] == 0 and max(out["mm_max_abs_err"]) < 1e-5


def _ep(world: int, ckpt, port: int, extra=()):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", str(port),
           "-m", "pocketllm_b200.parallel.dsv4_ep_check", "--ckpt", str(ckpt), "--prompt", ",".join(str((i * 29 + 3) % 500) for i in range(37)), "--new", "8", *extra]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr[-3000:]
    return json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_dsv4_expert_parallel_matches_single_gpu(tmp_path):
    from pocketllm_b200.models import deepseek_v4 as d4
    from pocketllm_b200.models import deepseek_v4_loader as ld
    cfg = d4.DSV4Config.tiny()
    ld.save_checkpoint(tmp_path, cfg, d4.random_checkpoint(cfg, seed=0))
    one = _ep(1, tmp_path, 29581)
    two = _ep(2, tmp_path, 29582)
    nccl = _ep(2, tmp_path, 29583, ["--nccl"])
    assert two["ranks_agree"] and two["status"] == 0 and two["combine_calls"]["peer"] > 0 and two["combine_calls"]["nccl"] == 0
    assert nccl["combine_calls"]["peer"] == 0
    assert one["tokens"] == two["tokens"] == nccl["tokens"]
    assert abs(one["logit_checksum"] - two["logit_checksum"]) < 1e-3
    # two pipeline stages of two layers each: same tokens, same logits
    pp = _ep(2, tmp_path, 29585, ["--pp"])
    assert pp["ranks_agree"] and pp["tokens"] == one["tokens"] and abs(one["logit_checksum"] - pp["logit_checksum"]) < 1e-5
    # the same run with every combine through the in-switch all-reduce (where the machine offers multicast)
    mm = _ep(2, tmp_path, 29584, ["--multimem"])
    if mm["combine_calls"]["multimem"] > 0:
        assert mm["ranks_agree"] and mm["status"] == 0 and mm["combine_calls"]["peer"] == 0
        assert mm["tokens"] == one["tokens"] and abs(one["logit_checksum"] - mm["logit_checksum"]) < 1e-3


@pytest.mark.parametrize("world", [1, 2])
def test_moe_combine_as_peer_stores_from_the_reduce(world):
    """Expert-parallel grouped experts ending in the combine kernel (reduce -> peer stores -> signal -> wait -> sum): every
    rank gets the one-rank result; world 1 exercises the kernel through a single arena."""
    import json, os, subprocess, sys
    from pathlib import Path
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=str(root))
    if world == 1:
        cmd = [sys.executable, "-m", "pocketllm_b200.parallel.moe_combine_check"]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
               "--master-port", "29571", "-m", "pocketllm_b200.parallel.moe_combine_check"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=str(root))
    assert r.returncode == 0, r.stderr[-3000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert res["world"] == world and len(res["ranks"]) == world
    for rk in res["ranks"]:
        assert rk["combined"] and rk["status"] == 0 and rk["rel_err"] < 1e-5
