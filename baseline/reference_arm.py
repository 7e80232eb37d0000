"""`bench.py --impl reference`: the unmodified reference engine on the same metric.

What runs: the reference's own `dsv4_cpp_engine` (built from its sources for sm_100 into
`baseline/_ref/cpp_build/`, NCCL tensor parallel, its stock Qwen path) in its
`--qwen-persistent-stdin` mode, one process per GPU, on a random-init checkpoint of the
benchmark shape written in its own Safetensors layout. None of this repository's kernels,
models or engine are on that path; only the checkpoint writer is shared.

Requests are fed as `<max_new_tokens> tok0 tok1 ...` lines; the engine answers with a
`qwen_persistent_result=1 ... decode_tokens_per_s=... prefill_tokens_per_s=...` line per
request (reference timing: host wall clock around its own device work).
"""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
BINARY = ROOT / "baseline" / "_ref" / "cpp_build" / "dsv4_cpp_engine"
PUBLISHED_DECODE_TOK_S = 35.87


def _unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why}


def _ckpt_dir() -> Path:
    env = os.environ.get("POCKET_REF_CKPT")
    if env:
        return Path(env)
    shm = Path("/dev/shm")
    try:
        if shm.exists() and shutil.disk_usage(shm).free > 60 * (1 << 30):
            return shm / "pocket_ref_qwen27b"
    except OSError:
        pass
    return Path("/tmp/pocket_ref_qwen27b")


def _field(line: str, key: str) -> float:
    for tok in line.split():
        if tok.startswith(key + "="):
            return float(tok.split("=", 1)[1])
    raise KeyError(key)


def run(args) -> dict:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if getattr(args, "model", "qwen27b") == "minimax-m2":
        # the reference's GGUF runtime loads a checkpoint file; a 60 GB MiniMax-M2 GGUF cannot be produced offline within the run
        return _unavailable("MiniMax-M2: the reference's loader needs a full GGUF checkpoint file (about 60 GB), which cannot be made offline here") if rank == 0 else {}
    if not BINARY.exists():
        return _unavailable("baseline/_ref/cpp_build/dsv4_cpp_engine is not built (offline cmake build of the reference missing)") if rank == 0 else {}
    import torch
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("gloo")
    ckpt = _ckpt_dir()
    err = ""
    if rank == 0 and not (ckpt / ".complete").exists():
        try:
            from baseline import make_qwen_checkpoint as mk
            from pocketllm_b200.models.qwen_hybrid import QwenHybridConfig
            cfg = QwenHybridConfig.benchmark_27b() if args.model == "qwen27b" else QwenHybridConfig.tiny()
            mk.write_checkpoint(ckpt, cfg)
        except Exception as e:  # disk full, ...
            err = f"could not write the reference checkpoint: {e}"
    if world > 1:
        box = [err]
        dist.broadcast_object_list(box, src=0)
        err = box[0]
    if err:
        return _unavailable(err) if rank == 0 else {}

    g = torch.Generator().manual_seed(1234)
    vocab = 151936 if args.model == "qwen27b" else 1024
    prompts = [torch.randint(0, vocab, (args.prompt_len,), generator=g).tolist() for _ in range(args.warmup + args.steps)]
    max_new = args.decode_len + 1
    id_path = f"/tmp/pocket_ref_nccl_{os.environ.get('MASTER_PORT', '0')}.id"
    if rank == 0:
        for p in (id_path, id_path + ".cmdsock"):
            try:
                os.unlink(p)
            except OSError:
                pass
    if world > 1:
        dist.barrier()
    cmd = [str(BINARY), "--ckpt", str(ckpt), "--tp-world", str(world), "--tp-rank", str(rank), "--device", str(local),
           "--nccl-id-path", id_path, "--smoke-layers", "0", "--qwen-persistent-stdin", "--qwen-no-prefix-cache",
           "--max-context", str(args.prompt_len + max_new + 8), "--prefill-chunk-tokens", "512", "--max-new-tokens", str(max_new)]
    env = dict(os.environ)
    env.pop("CUDA_VISIBLE_DEVICES", None)
    t_start = time.perf_counter()
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE if rank == 0 else subprocess.DEVNULL, stdout=subprocess.PIPE if rank == 0 else subprocess.DEVNULL,
                            stderr=subprocess.STDOUT, text=True, env=env)
    results: list[str] = []
    log: list[str] = []
    fail = ""
    try:
        if rank == 0:
            for pr in prompts:
                proc.stdin.write(f"{max_new} " + " ".join(str(t) for t in pr) + "\n")
                proc.stdin.flush()
                while True:
                    line = proc.stdout.readline()
                    if not line:
                        fail = "reference engine exited early: " + " | ".join(log[-3:])
                        break
                    log.append(line.strip()[:300])
                    if line.startswith("qwen_persistent_result=1"):
                        results.append(line)
                        break
                if fail:
                    break
            if proc.stdin:
                proc.stdin.close()
        proc.wait(timeout=3600)
    except Exception as e:
        fail = f"reference run failed: {e}"
        proc.kill()
    wall = time.perf_counter() - t_start
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return {}
    if fail or len(results) < args.warmup + args.steps:
        return _unavailable(fail or "reference engine produced too few result lines")
    timed = results[args.warmup:]
    dec_s = sum(_field(l, "decode_seconds") for l in timed)
    pre_s = sum(_field(l, "prefill_seconds") for l in timed)
    dec = args.steps * args.decode_len / dec_s
    pre = args.steps * args.prompt_len / pre_s
    return {"impl": "reference", "metric": "single-request decode tok/s (Qwen3.8-27B-FP8 shape, 512-token prompt, 256 greedy steps)",
            "value": round(dec, 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round((dec_s + pre_s) / args.steps * 1e3, 3), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(dec / PUBLISHED_DECODE_TOK_S, 3), "dtype": "fp16 activations, fp8 e4m3 weights (reference default path)",
            "data": "synthetic: uniform-random token prompts, random-init FP8 checkpoint in the reference's Safetensors layout",
            "prefill_tok_s": round(pre, 1), "timing": "reference's own host wall clock per request",
            # the same keys as the other arm's config
            "config": {"model": "Qwen3.8-27B-FP8-shaped hybrid (64L, hidden 5120, inter 17408, vocab 151936)" if args.model == "qwen27b" else "tiny",
                       "global_batch": 1, "seq_len": args.prompt_len, "decode_len": args.decode_len, "parallelism": f"tp{world}",
                       "l2": "inputs larger than L2 (27 GB of weights streamed per token)", "prefill_chunk": 512},
            "engine": "dsv4_cpp_engine --qwen-persistent-stdin (NCCL)",
            # the prompt's token ids go in as text on stdin and the generated ids come back as text on stdout; counted as
            # 4-byte ids like the other arm's pinned-memory copies
            "e2e": {"value": round(dec, 2), "unit": "tok/s", "h2d_bytes_per_step": args.prompt_len * 4, "d2h_bytes_per_step": (args.decode_len + 1) * 4,
                    "note": "the reference's CLI is its public API; tokens enter and leave through the host"},
            "first_tokens": [int(t) for t in timed[-1].split("generated_token_ids=")[-1].split()[0].split(",")[:16]] if "generated_token_ids=" in timed[-1] else [],
            "total_wall_s": round(wall, 1)}
