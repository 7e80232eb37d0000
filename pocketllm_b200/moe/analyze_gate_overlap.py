"""How well do a model's routed experts repeat from one decode token to the next? Reads a dump of router choices and
prints, per layer, the mean overlap of consecutive tokens' expert sets and the hit rate an LRU cache of N device slots
would have had: the figures that decide how many experts per layer to keep resident (`expert_slots`) and whether a
prefetch from the previous token's set pays.

    python -m pocketllm_b200.moe.analyze_gate_overlap DUMP.jsonl [--slots 16,32,64] [--skip-prefill] [--json]

The dump has one JSON object per router call: {"layer": L, "ids": [[expert ids of token 0], [token 1], ...]} (calls in the
order they ran; a call with several tokens is a prefill chunk). `dump_capture()` writes one from the `capture` dict of
`DSV4Runtime` (keys `layers.L.ffn.route_idx`). Role of the reference's scripts/analyze_gate_overlap.py.
"""
from __future__ import annotations

import argparse
import json
from collections import defaultdict
from pathlib import Path

from .expert_cache import LRUSlots


def dump_capture(capture: dict, path: str | Path) -> int:
    """Write the router choices recorded by a runtime (`capture[f"layers.{L}.ffn.route_idx"]` = list of [T, k] tensors, one
    per call) as a dump file; returns the number of lines."""
    calls: dict[int, list] = {}
    for key, tensors in capture.items():
        parts = key.split(".")
        if len(parts) >= 4 and parts[0] == "layers" and parts[-1] == "route_idx":
            calls[int(parts[1])] = [t.tolist() if hasattr(t, "tolist") else list(t) for t in tensors]
    n_calls = max((len(v) for v in calls.values()), default=0)
    lines = 0
    with open(path, "w") as f:
        for c in range(n_calls):                       # call-major, the order the routers ran in
            for layer in sorted(calls):
                if c < len(calls[layer]):
                    f.write(json.dumps({"layer": layer, "ids": calls[layer][c]}) + "\n")
                    lines += 1
    return lines


def analyze(lines, slots: list[int], skip_prefill: bool = False) -> dict:
    """Per layer: tokens seen, mean |S_t & S_{t-1}| / |S_t| over consecutive tokens, and for every slot count the share of
    expert uses that an LRU cache of that size would have served without a copy."""
    per_layer: dict[int, list[list[int]]] = defaultdict(list)
    for ln in lines:
        ln = ln.strip()
        if not ln:
            continue
        rec = json.loads(ln)
        rows = rec["ids"]
        if skip_prefill and len(rows) > 1:
            rows = rows[-1:]                            # a prefill chunk only sets the starting point
        per_layer[int(rec["layer"])].extend([int(e) for e in row] for row in rows)
    out = {}
    for layer in sorted(per_layer):
        toks = per_layer[layer]
        overlaps = [len(set(a) & set(b)) / max(len(set(b)), 1) for a, b in zip(toks, toks[1:])]
        rates = {}
        for n in slots:
            if any(len(set(t)) > n for t in toks):
                rates[str(n)] = None                   # one token needs more experts than there are slots
                continue
            lru = LRUSlots(n)
            for t in toks:
                lru.assign(t)
            uses = lru.stats["hits"] + lru.stats["misses"]
            rates[str(n)] = lru.stats["hits"] / uses if uses else None
        out[str(layer)] = {"tokens": len(toks), "distinct_experts": len({e for t in toks for e in t}),
                           "mean_consecutive_overlap": sum(overlaps) / len(overlaps) if overlaps else None, "lru_hit_rate": rates}
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("path")
    ap.add_argument("--slots", default="8,16,32,64")
    ap.add_argument("--skip-prefill", action="store_true", help="count only the last token of calls with several tokens")
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    slots = [int(s) for s in args.slots.split(",") if s]
    with open(args.path) as f:
        res = analyze(f, slots, args.skip_prefill)
    if args.json:
        print(json.dumps(res))
        return 0
    print("layer tokens distinct overlap " + " ".join(f"lru{n}" for n in slots))
    for layer, r in res.items():
        fmt = lambda v: "   -  " if v is None else f"{v:6.3f}"
        print(f"{int(layer):5d} {r['tokens']:6d} {r['distinct_experts']:8d} {fmt(r['mean_consecutive_overlap'])} " +
              " ".join(fmt(r["lru_hit_rate"][str(n)]) for n in slots))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
