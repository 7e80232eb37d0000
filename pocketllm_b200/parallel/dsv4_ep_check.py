"""Expert-parallel consistency run for the DeepSeek-V4 runtime (launch with torchrun): every rank holds a slice of
the routed experts, the combine runs over peer memory (or NCCL with --nccl, or the in-switch all-reduce with --multimem);
with --pp every rank holds a contiguous layer range instead and the hidden state travels stage to stage. Rank 0 prints
one JSON line.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29571 \
        -m pocketllm_b200.parallel.dsv4_ep_check --ckpt DIR --prompt 1,2,3 --new 8
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist

from ..models import deepseek_v4_loader as ld
from ..models.deepseek_v4_runtime import DSV4Runtime
from . import tp


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--prompt", default="1,2,3,4,5,6,7,8,9,10")
    ap.add_argument("--new", type=int, default=8)
    ap.add_argument("--nccl", action="store_true")
    ap.add_argument("--multimem", action="store_true", help="combine through the in-switch all-reduce (every payload size)")
    ap.add_argument("--pp", action="store_true", help="layer pipeline instead of expert parallelism: each rank holds a contiguous layer range")
    args = ap.parse_args()
    rank, world, local = tp.env_rank_world()
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg, W = ld.load_checkpoint(args.ckpt)
    if args.pp and world > 1:
        from .pipeline import PipelineStage
        rt = DSV4Runtime(cfg, W, max_context=256, max_rows=16, pipeline=PipelineStage(cfg.n_layers))
    else:
        rt = DSV4Runtime(cfg, W, max_context=256, max_rows=16, rank=rank, world=world, use_peer_allreduce=not args.nccl)
    if args.multimem and world > 1:
        from .combine import ExpertCombine
        rt.combine = ExpertCombine(world, None, capacity=16 * cfg.dim, multimem=True, multimem_min_floats=1)
    prompt = [int(t) for t in args.prompt.split(",")]
    logits = rt.forward_logits(prompt)
    rt.last_token = int(logits[-1].argmax())
    tokens = [rt.last_token] + rt.decode(args.new - 1)
    status = max(rt.combine.peer.status() if rt.combine.peer is not None else 0, rt.combine.mm.status() if rt.combine.mm is not None else 0)
    agree = True
    if world > 1:
        t = torch.tensor(tokens, device="cuda")
        ref = t.clone()
        dist.broadcast(ref, 0)
        ok = torch.tensor([int(torch.equal(t, ref)), status], device="cuda")
        dist.all_reduce(ok, op=dist.ReduceOp.MAX if False else dist.ReduceOp.MIN)
        agree = bool(ok[0])
    if rank == 0:
        print(json.dumps({"world": world, "tokens": tokens, "ranks_agree": agree, "status": status, "combine_calls": rt.combine.calls,
                          "logit_checksum": round(float(logits.float().abs().mean()), 6)}))
    if world > 1:
        # every rank lets go of a multicast-bound buffer together
        torch.cuda.synchronize()
        dist.barrier()
        rt.combine.mm = None
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
