"""Re-encode a DeepSeek-V4 Safetensors checkpoint (reference: src/cli/convert_checkpoint.py, which turns the
FP8 / FP4 original into INT8 for cards without those formats). On B200 both formats are native, so the useful
directions are: keep as is (re-shard), dequantise to bf16 (debugging, oracles), or quantise a bf16 / fp32
checkpoint into the serving layout (FP8 E8M0-block dense linears, FP4 routed experts).

    python -m pocketllm_b200.cli.convert_checkpoint --hf-ckpt-path IN --save-path OUT [--dense fp8|bf16|keep] [--experts mxfp4|bf16|keep]
"""
from __future__ import annotations

import argparse
import re

import torch

from ..formats import fp4
from ..models import deepseek_v4_loader as ld

_EXPERT = re.compile(r"\.experts\.\d+\.w[123]\.weight$")


def convert(W: dict[str, torch.Tensor], dense: str, experts: str) -> dict[str, torch.Tensor]:
    out: dict[str, torch.Tensor] = {}
    for k, t in W.items():
        if k.endswith(".scale"):
            continue
        base = k[:-len("weight")] if k.endswith("weight") else None
        if _EXPERT.search(k):
            packed = t.dtype in (torch.uint8, torch.int8)
            if experts == "keep" or (experts == "mxfp4" and packed):
                out[k] = t
                if packed:
                    out[base + "scale"] = W[base + "scale"]
            elif experts == "bf16":
                out[k] = (fp4.dequantize_e2m1(t.view(torch.uint8), W[base + "scale"].view(torch.uint8)) if packed else t.float()).to(torch.bfloat16)
            else:                                              # mxfp4 from a dense tensor
                out[k], out[base + "scale"] = fp4.quantize_e2m1(t.float())
        elif t.dtype == torch.float8_e4m3fn:
            if dense == "bf16":
                out[k] = ld.dequantize_fp8_e8m0(t, W[base + "scale"]).to(torch.bfloat16)
            else:
                out[k], out[base + "scale"] = t, W[base + "scale"]
        else:
            out[k] = t
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--hf-ckpt-path", required=True)
    ap.add_argument("--save-path", required=True)
    ap.add_argument("--dense", choices=["fp8", "bf16", "keep"], default="keep")
    ap.add_argument("--experts", choices=["mxfp4", "bf16", "keep"], default="keep")
    args = ap.parse_args(argv)
    cfg, W = ld.load_checkpoint(args.hf_ckpt_path)
    out = convert(W, args.dense, args.experts)
    # save_checkpoint quantises dense fp32/bf16 linears when asked to; tensors that are already FP8 pass through
    ld.save_checkpoint(args.save_path, cfg, {k: (v.float() if v.dtype == torch.bfloat16 and args.dense == "fp8" else v) for k, v in out.items()},
                       fp8_dense=args.dense == "fp8")
    n_q = sum(1 for v in out.values() if v.dtype == torch.float8_e4m3fn)
    print(f"converted {len(W)} tensors -> {args.save_path} (dense={args.dense}, experts={args.experts}, fp8 tensors kept: {n_q})")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
