"""Peer-memory all-reduce check and timing (launch with torchrun): compares `PeerAllReduce` with NCCL on random
fp32 tensors of several sizes and prints one JSON line on rank 0.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29541 \
        -m pocketllm_b200.parallel.par_check --sizes 4096,65536,2097152
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist

from . import tp
from .peer_allreduce import PeerAllReduce


def _time(fn, iters: int) -> float:
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters * 1e3], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="4096,65536,2097152")
    ap.add_argument("--iters", type=int, default=50)
    args = ap.parse_args()
    rank, world, local = tp.env_rank_world()
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    sizes = [int(s) for s in args.sizes.split(",")]
    par = PeerAllReduce(max(sizes))
    out = {"world": world, "sizes": sizes, "max_abs_err": [], "peer_us": [], "nccl_us": [], "status": None}
    for n in sizes:
        torch.manual_seed(1234 + rank)
        x = torch.randn(n, device="cuda")
        want = x.clone()
        dist.all_reduce(want)
        got = par.all_reduce(x.clone())
        # a second call right away uses the other slot set; a third reuses the first
        again = par.all_reduce(x.clone())
        third = par.all_reduce(x.clone())
        torch.cuda.synchronize()
        err = max((got - want).abs().max().item(), (again - want).abs().max().item(), (third - want).abs().max().item())
        out["max_abs_err"].append(err)
        buf, buf2 = x.clone(), x.clone()
        out["peer_us"].append(round(_time(lambda: par.all_reduce(buf), args.iters), 2))
        out["nccl_us"].append(round(_time(lambda: dist.all_reduce(buf2), args.iters), 2))
    st = torch.tensor([par.status()], device="cuda")
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    out["status"] = int(st)
    par.close()
    if rank == 0:
        print(json.dumps(out))
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
