"""Requests per second and tokens per second of a resident OpenAI-compatible server (the Python server of
`pocketllm_b200.server.openai` or the native one started by `serve_native`): sends chat requests one after the other
(the engines serve one request at a time), reads `usage` from the answers, and prints one JSON object.
Role of the reference's scripts/bench_openai_resident.py.

    python -m pocketllm_b200.cli.bench_openai_resident --url http://127.0.0.1:8000 --requests 8 --max-tokens 128
"""
from __future__ import annotations

import argparse
import json
import statistics
import time
import urllib.request


def one_request(url: str, body: dict, timeout: float) -> tuple[dict, float]:
    req = urllib.request.Request(url.rstrip("/") + "/v1/chat/completions", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    t0 = time.perf_counter()
    with urllib.request.urlopen(req, timeout=timeout) as r:
        out = json.loads(r.read().decode())
    return out, time.perf_counter() - t0


def run(url: str, prompts: list[str], max_tokens: int, model: str, timeout: float = 600.0, warmup: int = 1) -> dict:
    rows = []
    for i, text in enumerate(prompts):
        body = {"model": model, "messages": [{"role": "user", "content": text}], "max_tokens": max_tokens, "temperature": 0}
        out, wall = one_request(url, body, timeout)
        u = out.get("usage", {})
        rows.append({"wall_s": wall, "prompt_tokens": u.get("prompt_tokens", 0), "completion_tokens": u.get("completion_tokens", 0),
                     "finish_reason": out["choices"][0].get("finish_reason")})
    timed = rows[warmup:] or rows
    total = sum(r["wall_s"] for r in timed)
    return {"bench": "openai_resident", "requests": len(timed), "warmup": min(warmup, len(rows) - 1 if len(rows) > 1 else 0),
            "completion_tok_s": round(sum(r["completion_tokens"] for r in timed) / total, 2),
            "total_tok_s": round(sum(r["completion_tokens"] + r["prompt_tokens"] for r in timed) / total, 2),
            "requests_per_s": round(len(timed) / total, 3), "median_request_s": round(statistics.median(r["wall_s"] for r in timed), 4),
            "rows": rows}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="pocketllm-b200")
    ap.add_argument("--requests", type=int, default=8)
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--prompt-words", type=int, default=200, help="length of the synthetic user message")
    ap.add_argument("--shared-prefix", action="store_true", help="every request starts with the same long message (prefix reuse)")
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)
    base = " ".join(f"word{i % 97}" for i in range(args.prompt_words))
    prompts = [(base + f" question {i}?") if args.shared_prefix else (f"request {i}: " + base) for i in range(args.requests + 1)]
    res = run(args.url, prompts, args.max_tokens, args.model)
    text = json.dumps(res)
    print(text)
    if args.out:
        with open(args.out, "w") as f:
            f.write(text + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
