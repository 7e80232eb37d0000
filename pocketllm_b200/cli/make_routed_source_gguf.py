"""Build a GGUF whose routed-expert tensors come from an FP4 Safetensors checkpoint, keeping everything else
(tokenizer, metadata, dense tensors) from a template GGUF (reference: src/cli/make_routed_source_gguf.py:538-551).
The experts are dequantised from E2M1 + E8M0 and re-encoded as `--target-type` (f16 by default: a lossless
"source" file for later requantisation; any type with a quantiser here works too).

    python -m pocketllm_b200.cli.make_routed_source_gguf --template-gguf T.gguf --hf-ckpt-path DIR --output OUT.gguf
        [--layers 0,3-5] [--target-type f16|bf16|q8_0|q4_k|...] [--max-routed-tensors N] [--dry-run]
"""
from __future__ import annotations

import argparse
import re
import sys
from pathlib import Path

import numpy as np
import torch

from ..formats import fp4, gguf, gguf_quants
from ..formats import safetensors_io as st

_ROUTED = re.compile(r"^blk\.(\d+)\.ffn_(gate|up|down)_exps\.weight$")
_PART = {"gate": "w1", "up": "w3", "down": "w2"}


def parse_layers(text: str | None) -> set[int] | None:
    if not text:
        return None
    out: set[int] = set()
    for part in text.split(","):
        lo, _, hi = part.partition("-")
        out.update(range(int(lo), int(hi or lo) + 1))
    return out


def expert_matrix(model: st.SafetensorsModel, layer: int, part: str, e: int) -> torch.Tensor:
    name = f"layers.{layer}.ffn.experts.{e}.{_PART[part]}"
    return fp4.dequantize_e2m1(model.get(name + ".weight").view(torch.uint8), model.get(name + ".scale").view(torch.uint8))


def encode(mat: np.ndarray, type_name: str) -> np.ndarray:
    if type_name == "f16":
        return mat.astype(np.float16)
    if type_name == "f32":
        return mat.astype(np.float32)
    if type_name == "bf16":
        return torch.from_numpy(mat).to(torch.bfloat16).view(torch.int16).numpy()
    return gguf_quants.quantize(mat, type_name)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--template-gguf", required=True)
    ap.add_argument("--hf-ckpt-path", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--layers", default=None)
    ap.add_argument("--target-type", default="f16")
    ap.add_argument("--max-routed-tensors", type=int, default=None)
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args(argv)
    if Path(args.output).exists():
        print(f"refusing to overwrite {args.output}", file=sys.stderr)
        return 2
    src = gguf.GGUFFile(args.template_gguf)
    model = st.SafetensorsModel(args.hf_ckpt_path)
    layers = parse_layers(args.layers)
    plan, budget = [], args.max_routed_tensors
    for name in src.tensors:
        m = _ROUTED.match(name)
        take = bool(m) and (layers is None or int(m.group(1)) in layers) and (budget is None or budget > 0)
        if take and budget is not None:
            budget -= 1
        plan.append((name, "rewrite" if take else "copy"))
    n_rw = sum(1 for _, a in plan if a == "rewrite")
    print(f"plan: {n_rw} routed tensors rewritten as {args.target_type}, {len(plan) - n_rw} tensors copied")
    if args.dry_run:
        for name, action in plan:
            if action == "rewrite":
                print(f"  rewrite {name} {tuple(src.tensors[name].shape)} {src.tensors[name].type_name} -> {args.target_type}")
        return 0
    w = gguf.GGUFWriter()
    for k, v in src.metadata.items():
        if k != "general.alignment":
            w.add_meta(k, v, src.metadata_types[k])
    for name, action in plan:
        t = src.tensors[name]
        if action == "copy":
            w.add_tensor(name, src.raw(name), t.type_name, t.shape)
            continue
        m = _ROUTED.match(name)
        layer, part = int(m.group(1)), m.group(2)
        E = t.shape[0]
        mats = [encode(expert_matrix(model, layer, part, e).numpy(), args.target_type) for e in range(E)]
        blob = np.stack(mats, 0)
        if tuple(expert_matrix(model, layer, part, 0).shape) != tuple(t.shape[1:]):
            raise SystemExit(f"{name}: checkpoint expert shape does not match the template {tuple(t.shape)}")
        w.add_tensor(name, blob, args.target_type, t.shape)
    w.write(args.output)
    print(f"wrote {args.output}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
