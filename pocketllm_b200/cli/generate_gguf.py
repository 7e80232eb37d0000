"""Raw-block GGUF generation CLI (MiniMax-M2, GLM-DSA):

    torchrun --nproc-per-node N -m pocketllm_b200.cli.generate_gguf --gguf-path P \
        (--seed-file F | --tokens 1,2,3) --max-new-tokens M [--architecture A] [--layers L]
        [--gpu-memory-gib G | --expert-slots N] [--dtype bf16] [--prewarm]

Prints `RESULT prefill_seconds=... prefill_tps=... decode_seconds=... decode_tps=...` and
`generated_token_ids=...` on rank 0 (same surface as the reference's
src/cli/generate_gguf.py and src/runtime/generation.py:174-276).
"""
from __future__ import annotations

import argparse

from ..models import registry
from ..runtime import generation as gen


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gguf-path", required=True)
    ap.add_argument("--architecture", default=None)
    ap.add_argument("--seed-file", default=None)
    ap.add_argument("--tokens", default=None)
    ap.add_argument("--max-new-tokens", type=int, default=16)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--max-context", type=int, default=4096)
    ap.add_argument("--prewarm", action="store_true", help="read the file once to warm the page cache")
    ap.add_argument("--gpu-memory-gib", type=float, default=None,
                    help="HBM this rank may use: experts that do not fit stay in pinned host memory and are staged per step (glm-dsa)")
    ap.add_argument("--expert-slots", type=int, default=None, help="resident experts per layer (the rest are staged from pinned host memory)")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "auto"], help="activation dtype (weights stay in their GGUF block types)")
    args = ap.parse_args(argv)
    rank, world, local = gen.setup_dist()
    if args.prewarm:
        from ..formats import prewarm
        prewarm.prewarm(args.gguf_path)
    prompt = gen.read_seed_tokens(args.seed_file) if args.seed_file else [int(t) for t in (args.tokens or "1").split(",")]
    extra = {}
    if args.expert_slots is not None:
        extra["expert_slots"] = args.expert_slots
    if args.gpu_memory_gib is not None:
        extra["gpu_memory_gib"] = args.gpu_memory_gib
    rt = registry.build_runtime(args.gguf_path, args.architecture, rank=rank, world=world, device=f"cuda:{local}",
                                max_context=args.max_context, layers=args.layers, **extra)
    res = gen.greedy_generate(rt, prompt, args.max_new_tokens)
    if rank == 0:
        print(res.result_line(), flush=True)
        print("generated_token_ids=" + ",".join(str(t) for t in res.tokens), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
