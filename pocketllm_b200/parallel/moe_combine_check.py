"""Expert-parallel MoE with the combine fused into the per-token reduce, on two or more ranks:

    torchrun --nproc-per-node 2 -m pocketllm_b200.parallel.moe_combine_check

Every rank builds the same random quantised experts and routes, runs the grouped tensor-core path on ITS experts and ends
with the combine kernel (weighted per-token reduce -> stores into every rank's arena -> signal -> bounded wait -> sum); the
result on every rank must equal the one-rank result over all experts. Rank 0 prints one JSON line.
"""
from __future__ import annotations

import json

import numpy as np
import torch
import torch.distributed as dist

from ..formats import gguf_quants as gq
from ..ops import gguf_ops as go
from . import tp
from .peer_allreduce import PeerAllReduce


def main() -> int:
    rank, world, local = tp.env_rank_world()
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    E, H, I, T, topk = 8, 512, 256, 200, 2
    rng = np.random.default_rng(0)
    w13 = torch.from_numpy(gq.quantize((rng.standard_normal((E * 2 * I, H)) * 0.05).astype(np.float32), "q4_k")).cuda().view(-1)
    w2 = torch.from_numpy(gq.quantize((rng.standard_normal((E * H, I)) * 0.05).astype(np.float32), "q4_k")).cuda().view(-1)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, H, generator=g).cuda().to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(T)]).int().cuda()
    wts = torch.rand(T, topk, generator=g).cuda()
    routes = go.group_routes(ids, wts, E)
    want = go.gguf_moe_forward_grouped(x, w13, w2, "q4_k", "q4_k", E, I, routes)
    per = E // world
    lo13, lo2 = rank * per * 2 * I * go.row_bytes("q4_k", H), rank * per * H * go.row_bytes("q4_k", I)
    n13, n2 = per * 2 * I * go.row_bytes("q4_k", H), per * H * go.row_bytes("q4_k", I)
    peer = PeerAllReduce(T * H, group=dist.group.WORLD if world > 1 else None, _solo_world=1 if world == 1 else None)
    errs = []
    for _ in range(3):                      # both slot sets and a reuse
        got = go.gguf_moe_forward_grouped(x, w13[lo13:lo13 + n13], w2[lo2:lo2 + n2], "q4_k", "q4_k", E, I, routes, expert_offset=rank * per,
                                          local_experts=per, peer=peer)
        torch.cuda.synchronize()
        errs.append(((got - want).norm() / want.norm()).item())
    out = {"rank": rank, "combined": bool(routes.combined), "rel_err": max(errs), "status": peer.status()}
    gathered = [None] * world
    if world > 1:
        dist.all_gather_object(gathered, out)
    else:
        gathered = [out]
    if rank == 0:
        print(json.dumps({"world": world, "ranks": gathered}), flush=True)
    peer.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
