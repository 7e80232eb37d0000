"""Peer-path failure -> NCCL fallback, on two or more ranks:

    torchrun --nproc-per-node 2 -m pocketllm_b200.parallel.nccl_fallback_check --ckpt DIR

Every rank generates through the peer-store path, then rank 0 runs one decode step that the other ranks never join: its
bounded waits run out (nothing faults or hangs; the budget is lowered to a fraction of a second first), the step raises and
rank 0 moves to NCCL collectives by itself. The other ranks learn of it on the host (a barrier) and switch too. The same
prompt is then generated again through NCCL; rank 0 prints one JSON line with both token lists.
"""
from __future__ import annotations

import argparse
import json
import tempfile
from pathlib import Path

import torch
import torch.distributed as dist

from ..models import qwen_hybrid as qh
from . import tp


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--prompt", default="5,17,300,44,9,1000,2,77,12")
    ap.add_argument("--new", type=int, default=10)
    ap.add_argument("--prefill-chunk", type=int, default=64)
    args = ap.parse_args()
    rank, world, local = tp.env_rank_world()
    if world < 2:
        raise SystemExit("needs at least two ranks")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = qh.QwenHybridConfig.from_json((Path(args.ckpt) / "config.json").read_text())
    eng = qh.QwenEngine(cfg, tp_rank=rank, tp_world=world, device=local, max_context=512, prefill_chunk=args.prefill_chunk).load(args.ckpt)
    tp.connect_engine(eng)
    # rendezvous directory shared by the ranks
    box = [tempfile.mkdtemp(prefix="pk_nccl_id_") if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    eng.enable_nccl_fallback(str(Path(box[0]) / "id"))
    prompt = [int(t) for t in args.prompt.split(",")]
    peer_tokens = eng.generate(prompt, args.new)
    peer_status = eng.comm_status()
    # the step only rank 0 runs
    eng.reset()
    eng.prefill(prompt)
    eng.set_comm_timeout_us(200_000)
    torch.cuda.synchronize()
    dist.barrier()
    error = ""
    if rank == 0:
        try:
            eng.decode(1)
        except qh.EngineError as e:
            error = str(e)
    torch.cuda.synchronize()
    dist.barrier()
    switched_by_itself = eng.nccl_mode
    if not eng.nccl_mode:
        eng.switch_to_nccl()
    eng.set_comm_timeout_us(2_000_000)
    dist.barrier()
    eng.reset()
    nccl_tokens = eng.generate(prompt, args.new)
    out = {"rank": rank, "peer_tokens": peer_tokens, "nccl_tokens": nccl_tokens, "error": error, "switched_by_itself": switched_by_itself,
           "nccl_mode": eng.nccl_mode, "peer_status": peer_status, "status_after": eng.comm_status(), "persistent": eng.persistent_decode}
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    if rank == 0:
        print(json.dumps({"world": world, "ranks": gathered}), flush=True)
    eng.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
