"""GGUF inspection: `--summary`, `--architecture`, `--spec-summary`, `--validate-spec`, `--validate-ds4-q2`,
`--capability-report`, `--placement-report` (flags of the reference's src/cli/inspect_gguf.py)."""
from __future__ import annotations

import argparse
import json
from collections import Counter

from ..formats import gguf
from ..moe import spec


# Block types of the published 2-bit DeepSeek-V4 files and of everything this package decodes on the device.
DS4_Q2_EXPERT_TYPES = (("ffn_gate_exps.weight", "iq2_xxs"), ("ffn_up_exps.weight", "iq2_xxs"), ("ffn_down_exps.weight", "q2_k"),
                       ("ffn_gate_shexp.weight", "q8_0"), ("ffn_up_shexp.weight", "q8_0"), ("ffn_down_shexp.weight", "q8_0"))
DS4_Q2_METADATA = ("deepseek4.block_count", "deepseek4.embedding_length", "deepseek4.expert_count", "deepseek4.expert_used_count",
                   "deepseek4.expert_feed_forward_length")
DECODABLE_TYPES = {"f32", "f16", "bf16", "i32", "iq2_xxs", "q2_k", "iq1_m", "q4_k", "q5_k", "iq2_xs", "iq3_xxs", "iq4_xs", "q6_k", "q8_0", "mxfp4"}


def validate_ds4_q2(b: gguf.GGUFBundle) -> list[str]:
    """Problems of a 2-bit DeepSeek-V4 GGUF (empty list = fine): architecture and container version, the metadata the
    config reader needs, the block type of every layer's routed and shared expert tensors (gate / up IQ2_XXS, down Q2_K,
    shared experts Q8_0), and no tensor of a type that has no device decoder. Reference: `--validate-ds4-q2` of
    src/cli/inspect_gguf.py:183-240."""
    problems: list[str] = []
    if b.architecture() != "deepseek4":
        problems.append(f"general.architecture is {b.architecture()!r}, expected 'deepseek4'")
    version = getattr(b.files[0], "version", 3)
    if version != 3:
        problems.append(f"GGUF version is {version}, expected 3")
    for key in DS4_Q2_METADATA:
        if key not in b.metadata:
            problems.append(f"missing metadata {key}")
    try:
        n_layers = int(b.metadata.get("deepseek4.block_count", 43))
    except (TypeError, ValueError):
        n_layers = 43
    for layer in range(n_layers):
        for suffix, want in DS4_Q2_EXPERT_TYPES:
            t = b.tensors.get(f"blk.{layer}.{suffix}")
            if t is None:
                problems.append(f"missing tensor blk.{layer}.{suffix}")
            elif t.type_name != want:
                problems.append(f"blk.{layer}.{suffix} is {t.type_name}, expected {want}")
    odd = sorted({t.type_name for t in b.tensors.values()} - DECODABLE_TYPES)
    if odd:
        problems.append("tensor types without a decoder: " + ", ".join(odd))
    return problems


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("path")
    ap.add_argument("--summary", action="store_true")
    ap.add_argument("--architecture", action="store_true")
    ap.add_argument("--spec-summary", action="store_true")
    ap.add_argument("--validate-spec", action="store_true")
    ap.add_argument("--validate-ds4-q2", action="store_true", help="check a 2-bit DeepSeek-V4 file: metadata, expert block types, decodable types")
    ap.add_argument("--capability-report", action="store_true")
    ap.add_argument("--placement-report", action="store_true")
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--hbm-gib", type=float, default=180.0)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    b = gguf.GGUFBundle(args.path)
    out: dict = {}
    if args.architecture or not any([args.summary, args.spec_summary, args.validate_spec, args.validate_ds4_q2, args.capability_report,
                                     args.placement_report]):
        out["architecture"] = b.architecture()
    if args.summary:
        types = Counter(t.type_name for t in b.tensors.values())
        out["summary"] = {"files": len(b.files), "tensors": len(b.tensors), "bytes": b.total_bytes(), "types": dict(types),
                          "metadata_keys": len(b.metadata)}
    if args.spec_summary:
        out["spec"] = spec.parse_params(b).__dict__
    rc = 0
    if args.validate_spec:
        v = spec.validate(b)
        out["validation"] = {"ok": v.ok, "missing": v.missing[:20], "wrong_shape": v.wrong_shape[:20], "unexpected_types": v.unexpected_types[:20]}
        rc = 0 if v.ok else 2
    if args.validate_ds4_q2:
        problems = validate_ds4_q2(b)
        out["ds4_q2_validation"] = {"ok": not problems, "problems": problems[:50], "more": max(0, len(problems) - 50)}
        rc = max(rc, 1 if problems else 0)
    if args.capability_report:
        c = spec.capability(b)
        out["capability"] = {"supported": c.supported, "unsupported": c.unsupported, "per_type_bytes": c.per_type_bytes}
    if args.placement_report:
        p = spec.placement(b, spec.HardwareProfile(n_gpus=args.gpus, hbm_gib=args.hbm_gib))
        out["placement"] = p.__dict__
    if args.json:
        print(json.dumps(out))
    else:
        for k, v in out.items():
            print(f"{k}: {json.dumps(v) if not isinstance(v, str) else v}")
    return rc


if __name__ == "__main__":
    raise SystemExit(main())
