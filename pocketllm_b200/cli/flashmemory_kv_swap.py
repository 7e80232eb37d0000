"""Long-context retrieval attention end to end: FlashMemory chunk scoring (three scorer layers, max ensemble) -> top-k
chunks -> KV swap (compressed rows live in pinned host memory, `--gpu-chunks` device slots, LRU) -> DSV4 sparse attention
over the window rows and the swapped-in slots. Synthetic weights and keys of the DeepSeek-V4 indexer shape; prints one JSON
line with the step time and the tier's hit / miss / transfer counters, and (with `--check`) the agreement with attention
over a fully resident cache.

    python -m pocketllm_b200.cli.flashmemory_kv_swap --context 65536 --gpu-chunks 2560 --keep 2048 --steps 32 --check

Role of the reference's scripts/flashmemory_kv_swap_demo.sh (FlashMemory + KV_SWAP run of its GGUF engine) and of the
counters it logs (cpp_engine/src/dsv4_engine.cpp:5260-5434).
"""
from __future__ import annotations

import argparse
import json
import time

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--context", type=int, default=65536, help="tokens already in the context")
    ap.add_argument("--ratio", type=int, default=4, help="tokens per compressed KV row")
    ap.add_argument("--gpu-chunks", type=int, default=2560, help="device slots of the KV swap tier")
    ap.add_argument("--keep", type=int, default=2048, help="chunks selected per step")
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--heads", type=int, default=64, help="attention and scorer heads")
    ap.add_argument("--scorer-layers", type=int, default=3)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--q-lora-rank", type=int, default=1024)
    ap.add_argument("--check", action="store_true", help="compare every step with attention over a fully resident cache")
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    from ..ops import dsv4_ops as dk
    from ..ops import flashmemory as fm
    from ..runtime.kv_swap import KvSwapTier

    dev = "cuda"
    torch.manual_seed(args.seed)
    hd, rd, win = 128, 64, 128
    n_chunks = args.context // args.ratio
    if args.keep > args.gpu_chunks or args.keep > n_chunks:
        raise SystemExit("--keep must not exceed --gpu-chunks or the number of chunks")
    g = torch.Generator().manual_seed(args.seed)
    mk = lambda *s, sd: (torch.randn(*s, generator=g) * sd).to(dev)
    scorers = [fm.ScorerWeights(wq_a=mk(args.q_lora_rank, args.hidden, sd=args.hidden ** -0.5), wq_b=mk(args.heads * 128, args.q_lora_rank, sd=args.q_lora_rank ** -0.5),
                                q_norm=torch.ones(args.q_lora_rank, device=dev), weights_proj=mk(args.heads, args.hidden, sd=args.hidden ** -0.5),
                                inv_freqs=fm.yarn_inv_freqs(rd, 160000.0, 16.0, 65536, 32.0, 1.0).to(dev)) for _ in range(args.scorer_layers)]
    # per scorer layer: compressed keys (E4M3 + scale); one attention layer's compressed KV rows (bf16, K == V)
    keys = [fm.quantize_keys(torch.randn(n_chunks, hd, device=dev)) for _ in range(args.scorer_layers)]
    kv_rows = (torch.randn(n_chunks, hd, device=dev) * 0.5).to(torch.bfloat16)
    window_rows = (torch.randn(win, hd, device=dev) * 0.5).to(torch.bfloat16)
    small = torch.zeros(win + args.gpu_chunks, hd, device=dev, dtype=torch.bfloat16)
    small[:win] = window_rows
    tier = KvSwapTier(capacity=n_chunks, device_slots=args.gpu_chunks, row_bytes=hd * 2, window=0, pool=small[win:])
    for lo in range(0, n_chunks, 1 << 16):
        tier.store(lo, kv_rows[lo:lo + (1 << 16)])
    full = torch.cat([window_rows, kv_rows]) if args.check else None
    ang = torch.outer(torch.arange(args.context + args.steps + 8).double(), 1.0 / (10000.0 ** (torch.arange(0, rd, 2).double() / rd)))
    cos_t, sin_t = torch.cos(ang).float().to(dev), torch.sin(ang).float().to(dev)
    sink = torch.zeros(args.heads, device=dev)
    layer_scores = torch.empty(args.scorer_layers, n_chunks, device=dev)
    worst = 0.0
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall = time.perf_counter()
    e0.record()
    for step in range(args.steps):
        position = args.context + step
        hidden = torch.randn(args.hidden, device=dev)
        for l, (w, (codes, scale)) in enumerate(zip(scorers, keys)):
            qcodes, head_w = fm.build_query(w, hidden, position)
            fm.score_chunks(codes, scale, qcodes, head_w, sigmoid=True, out=layer_scores[l])
        ens = fm.ensemble(layer_scores, n_chunks, use_max=True)
        idx, _ = fm.topk(ens, args.keep)
        phys = tier.swap_in(idx.view(1, -1))
        q = torch.randn(1, args.heads, hd, device=dev).to(torch.bfloat16)
        pos = torch.tensor([position], device=dev, dtype=torch.int32)
        out = dk.sparse_attn(q, small, pos, sink, cos_t, sin_t, win=win, ring=win, ratio=args.ratio, rd=rd, sel=phys)
        if args.check:
            want = dk.sparse_attn(q, full, pos, sink, cos_t, sin_t, win=win, ring=win, ratio=args.ratio, rd=rd, sel=idx.view(1, -1).contiguous())
            worst = max(worst, (out.float() - want.float()).abs().max().item())
    e1.record()
    torch.cuda.synchronize()
    s = tier.stats
    res = {"context_tokens": args.context, "chunks": n_chunks, "gpu_chunks": args.gpu_chunks, "keep": args.keep, "steps": args.steps,
           "scorer_layers": args.scorer_layers, "ms_per_step": round(e0.elapsed_time(e1) / args.steps, 3),
           "wall_ms_per_step": round((time.perf_counter() - t_wall) * 1e3 / args.steps, 3),
           "kv_swap": {"hits": s["hits"], "misses": s["misses"], "evictions": s["evictions"], "h2d_mib": round(s["h2d_bytes"] / 2 ** 20, 2),
                       "d2h_mib": round(s["d2h_bytes"] / 2 ** 20, 2), "host_mib": round(s["host_bytes"] / 2 ** 20, 1),
                       "device_mib": round(args.gpu_chunks * hd * 2 / 2 ** 20, 2)},
           "resident_cache_mib": round(n_chunks * hd * 2 / 2 ** 20, 1)}
    if args.check:
        res["max_abs_diff_vs_resident"] = worst
    print(json.dumps(res), flush=True)
    tier.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
