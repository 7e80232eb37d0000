"""Tensor-parallel consistency run (launch with torchrun): every rank loads its shard of a
checkpoint directory, the ranks generate greedily through the peer-memory collectives, and
rank 0 prints one JSON line with the tokens, the comm status word and timings. The same
check as the reference's TP1-vs-TP4 output diff (cpp_engine/tests/test_dspark_tp_consistency.cpp),
as a library entry point.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29511 \
        -m pocketllm_b200.parallel.tp_check --ckpt DIR --prompt 1,2,3 --new 8
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch
import torch.distributed as dist

from ..models import qwen_hybrid as qh
from . import tp


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--prompt", default="1,2,3,4,5,6,7,8,9,10")
    ap.add_argument("--new", type=int, default=8)
    ap.add_argument("--prefill-chunk", type=int, default=64)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--mtp", type=int, default=0, help="draft length limit; > 0 also runs the speculative decode of the multi-token predictor")
    args = ap.parse_args()
    rank, world, local = tp.env_rank_world()
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = qh.QwenHybridConfig.from_json((Path(args.ckpt) / "config.json").read_text())
    eng = qh.QwenEngine(cfg, tp_rank=rank, tp_world=world, device=local, max_context=512,
                        prefill_chunk=args.prefill_chunk, use_cuda_graph=not args.no_graph, mtp=args.mtp > 0).load(args.ckpt)
    tp.connect_engine(eng)
    prompt = [int(t) for t in args.prompt.split(",")]
    first = eng.prefill(prompt)
    # the prefill logits of the whole vocabulary (every rank holds one shard), as a digest that runs of different world
    # sizes can be compared by: the eight largest entries and the norm
    shard = eng.logits(0).float().cuda().contiguous()
    if world > 1:
        parts = [torch.empty_like(shard) for _ in range(world)]
        dist.all_gather(parts, shard)
        full = torch.cat(parts)
    else:
        full = shard
    full = full.cpu()
    top = full.topk(8)
    tokens = [first] + eng.decode(args.new - 1) if args.new > 1 else [first]
    logits = eng.logits(0)
    out = {"world": world, "tokens": tokens, "comm_status": eng.comm_status(), "timings": eng.timings(),
           "logit_shard_sum": float(logits.double().sum()), "prefill_logits_top": [[int(i), float(v)] for v, i in zip(top.values, top.indices)],
           "prefill_logits_norm": float(full.double().norm()), "prefill_logits_head": [float(v) for v in full[:64]]}
    if args.mtp > 0:
        eng.reset()
        out["spec_tokens"], out["spec_stats"] = eng.generate_mtp(prompt, args.new, args.mtp)
        eng.reset()
        eng.set_draft_replay(tokens[1:])
        out["replay_tokens"], out["replay_stats"] = eng.generate_mtp(prompt, args.new, args.mtp)
        out["comm_status"] |= eng.comm_status()
    gathered = [None] * world
    if world > 1:
        dist.all_gather_object(gathered, out)
    else:
        gathered = [out]
    if rank == 0:
        same = all(g["tokens"] == gathered[0]["tokens"] for g in gathered)
        extra = {k: gathered[0][k] for k in ("spec_tokens", "spec_stats", "replay_tokens", "replay_stats") if k in gathered[0]}
        if extra:
            same = same and all(g["spec_tokens"] == gathered[0]["spec_tokens"] and g["replay_tokens"] == gathered[0]["replay_tokens"] for g in gathered)
        print(json.dumps({"world": world, "tokens": gathered[0]["tokens"], "ranks_agree": same,
                          "comm_status": [g["comm_status"] for g in gathered], "timings": gathered[0]["timings"],
                          "prefill_logits_top": gathered[0]["prefill_logits_top"], "prefill_logits_norm": gathered[0]["prefill_logits_norm"],
                          "prefill_logits_head": gathered[0]["prefill_logits_head"], **extra}), flush=True)
    eng.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
