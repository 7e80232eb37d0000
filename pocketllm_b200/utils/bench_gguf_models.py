"""Single-request prefill and decode rates of the raw-GGUF-block model families at their published shapes, on random
block payloads made on the device (no checkpoint file is needed):

    python -m pocketllm_b200.utils.bench_gguf_models --model minimax-m2 --prompt-len 256 --decode-len 128
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29590 \
        -m pocketllm_b200.utils.bench_gguf_models --model minimax-m2          # experts split over the ranks

Times are CUDA-event times on the launching stream, maximum over ranks; rank 0 prints one JSON line. The decode loop
reads every token back to the host (greedy pick), as a serving loop does.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="minimax-m2", choices=["minimax-m2"])
    ap.add_argument("--layers", type=int, default=0, help="run only the first N layers (0 = all)")
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--decode-len", type=int, default=128)
    ap.add_argument("--routing", default="balanced", choices=["balanced", "model"],
                    help="balanced: token t goes to experts (t * k + j + 37 * layer) mod E, as a trained load-balanced router spreads them; "
                         "model: the random router's own picks (with random weights the hidden states collapse and all tokens share 8 experts)")
    ap.add_argument("--kernel-table", type=int, default=0,
                    help="after the timed runs, decode 4 more tokens without the captured graph under torch.profiler and print the N kernels "
                         "with the largest share of device time (shares only: times under a profiler are not benchmark numbers)")
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=1)
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        group = dist.group.WORLD
    from ..models import minimax_m2 as mm
    cfg = mm.MiniMaxM2Config()
    if args.layers:
        cfg.n_layers = args.layers
    model = mm.MiniMaxM2Model.synthetic(cfg, device=f"cuda:{local}", rank=rank, world=world, max_context=args.prompt_len + args.decode_len + 8,
                                        group=group)
    model.balanced_routes = args.routing == "balanced"
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab_size, (args.prompt_len,), generator=g).tolist()
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    pre_ms, dec_ms, last = [], [], []
    for it in range(args.warmup + args.steps):
        model.reset()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        tok = model.prefill(prompt)
        e1.record()
        out = [tok]
        for _ in range(args.decode_len):
            out.append(model.decode_one(out[-1]))
        e2.record()
        torch.cuda.synchronize()
        if it >= args.warmup:
            pre_ms.append(e0.elapsed_time(e1))
            dec_ms.append(e1.elapsed_time(e2))
        last = out[-4:]
    t = torch.tensor([sum(pre_ms) / len(pre_ms), sum(dec_ms) / len(dec_ms)], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    pre, dec = t.tolist()
    if rank == 0:
        print(json.dumps({"model": args.model, "n_gpus": world, "layers": cfg.n_layers, "prompt_len": args.prompt_len, "decode_len": args.decode_len,
                          "prefill_ms": round(pre, 2), "prefill_tok_s": round(args.prompt_len / pre * 1e3, 1),
                          "decode_ms_per_token": round(dec / args.decode_len, 3), "decode_tok_s": round(args.decode_len / dec * 1e3, 2),
                          "weight_bytes_per_rank": model.weight_bytes(), "routing": args.routing, "expert_type": cfg.expert_type, "attn_type": cfg.attn_type,
                          "data": "synthetic: uniform-random prompt, random block payloads with constant block scales", "last_tokens": last}), flush=True)
    if args.kernel_table > 0 and rank == 0 and world == 1:
        from torch.profiler import ProfilerActivity, profile
        model.use_graph = False
        tok = last[-1]
        tok = model.decode_one(tok)
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(4):
                tok = model.decode_one(tok)
            torch.cuda.synchronize()
        rows = sorted(prof.key_averages(), key=lambda e: -e.self_device_time_total)
        total = sum(e.self_device_time_total for e in rows) or 1.0
        for e in rows[: args.kernel_table]:
            print(f"kernel_share={100.0 * e.self_device_time_total / total:5.1f}% calls={e.count:4d} avg_us={e.self_device_time_total / max(e.count, 1):8.1f} name={e.key[:90]}")
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
