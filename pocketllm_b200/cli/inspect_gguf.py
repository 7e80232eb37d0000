"""GGUF inspection: `--summary`, `--architecture`, `--spec-summary`, `--validate-spec`,
`--capability-report`, `--placement-report` (flags of the reference's src/cli/inspect_gguf.py)."""
from __future__ import annotations

import argparse
import json
from collections import Counter

from ..formats import gguf
from ..moe import spec


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("path")
    ap.add_argument("--summary", action="store_true")
    ap.add_argument("--architecture", action="store_true")
    ap.add_argument("--spec-summary", action="store_true")
    ap.add_argument("--validate-spec", action="store_true")
    ap.add_argument("--capability-report", action="store_true")
    ap.add_argument("--placement-report", action="store_true")
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--hbm-gib", type=float, default=180.0)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    b = gguf.GGUFBundle(args.path)
    out: dict = {}
    if args.architecture or not any([args.summary, args.spec_summary, args.validate_spec, args.capability_report, args.placement_report]):
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
