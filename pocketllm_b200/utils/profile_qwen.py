"""One prefill and a few eager (non-graph) decode steps of the hybrid decoder, for `ncu`.

    python -m pocketllm_b200.utils.profile_qwen --model qwen27b --prompt-len 512 --decode 2

prints the number of kernels launched by the weight initialisation (skip them with
`ncu -s`) and by each phase, so that a capture can be sized before it is run.
"""
from __future__ import annotations

import argparse

import torch

from ..models import qwen_hybrid as qh


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen27b", choices=["qwen27b", "tiny"])
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (keeps the 3:1 pattern)")
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--prefill-chunk", type=int, default=512)
    ap.add_argument("--decode", type=int, default=2)
    ap.add_argument("--graph", action="store_true")
    args = ap.parse_args()
    cfg = qh.QwenHybridConfig.benchmark_27b() if args.model == "qwen27b" else qh.QwenHybridConfig.tiny()
    if args.layers:
        cfg.num_hidden_layers = args.layers
        cfg.layer_types = []
        cfg.__post_init__()
    eng = qh.QwenEngine(cfg, max_context=args.prompt_len + args.decode + 16, prefill_chunk=args.prefill_chunk,
                        use_cuda_graph=args.graph)
    eng.init_random(0, 0.02)
    torch.cuda.synchronize()
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab_size, (args.prompt_len,), generator=g).tolist()
    l0 = eng.timings()["kernel_launches"]
    eng.prefill(prompt)
    t = eng.timings()
    print(f"prefill: {t['prefill_ms']:.3f} ms, {int(t['kernel_launches'] - l0)} launches")
    l1 = t["kernel_launches"]
    if args.decode:
        eng.decode(args.decode)
        t = eng.timings()
        print(f"decode: {t['decode_ms'] / args.decode:.3f} ms/token, {int(t['kernel_launches'] - l1)} launches")
    eng.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
