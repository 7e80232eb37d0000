"""Peer-memory all-reduce check and timing (launch with torchrun): compares `PeerAllReduce` with NCCL on random
fp32 tensors of several sizes and prints one JSON line on rank 0; `--multimem` adds the in-switch all-reduce
(`MultimemAllReduce`, one shot and two shot) where the machine offers multicast.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29541 \
        -m pocketllm_b200.parallel.par_check --sizes 4096,65536,2097152
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist

from . import tp
from .multimem_allreduce import MulticastUnavailable, MultimemAllReduce
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
    ap.add_argument("--multimem", action="store_true", help="also run the in-switch (multimem) all-reduce, one shot and two shot")
    args = ap.parse_args()
    rank, world, local = tp.env_rank_world()
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    sizes = [int(s) for s in args.sizes.split(",")]
    par = PeerAllReduce(max(sizes))
    out = {"world": world, "sizes": sizes, "max_abs_err": [], "peer_us": [], "nccl_us": [], "status": None}
    mm = None
    if args.multimem:
        try:
            mm = MultimemAllReduce(max(sizes))
            out.update({"multimem": "ok", "mm_max_abs_err": [], "mm_one_shot_us": [], "mm_two_shot_us": []})
        except (MulticastUnavailable, RuntimeError) as e:      # every rank takes the same branch: the probe is collective
            out["multimem"] = f"unavailable: {str(e)[:200]}"
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
        if mm is not None:
            errs = []
            for two in (False, True, False, True, True):          # both data sets under both schemes, and a reuse
                r = mm.all_reduce(x.clone(), two_shot=two)
                torch.cuda.synchronize()
                errs.append((r - want).abs().max().item())
            out["mm_max_abs_err"].append(max(errs))
            b3, b4 = x.clone(), x.clone()
            out["mm_one_shot_us"].append(round(_time(lambda: mm.all_reduce(b3, two_shot=False), args.iters), 2))
            out["mm_two_shot_us"].append(round(_time(lambda: mm.all_reduce(b4, two_shot=True), args.iters), 2))
    st = torch.tensor([max(par.status(), mm.status() if mm is not None else 0)], device="cuda")
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    out["status"] = int(st)
    par.close()
    # every rank lets go of the multicast-bound buffer together
    torch.cuda.synchronize()
    dist.barrier()
    del mm
    if rank == 0:
        print(json.dumps(out))
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
