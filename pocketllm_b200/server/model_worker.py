"""Model worker of the native server: one of the Python model backends (DeepSeek-V4 runtime, GGUF runtimes, the Qwen
engine's Python binding) behind a JSON-lines protocol on stdin / stdout, so that `pocket_engine --serve --model-worker KIND`
can serve every model family from the C++ HTTP / SSE front end while generation runs here on the GPU.

    {"op": "hello"}                                              -> {"ok": true, "max_context": N, "model": KIND}
    {"op": "prefill", "tokens": [...], "sampler": {...}, "seed": S} -> {"token": T [, "logprob": L, "top": [[id, lp], ...]]}
    {"op": "next"}                                               -> the same; {"token": 0, "done": true} after the backend's last token
    {"op": "end"}                                                -> {"ok": true}   (the request is over; the generator is closed)
    {"op": "quit"}
    any failure                                                  -> {"error": "...", "lost": b}   (lost: the step must be discarded)

`sampler` carries temperature, top_p, top_k, min_p, the three penalties and `logprobs` (-1 or k); `max_tokens` and
`stop_token_ids` of the request travel with the prefill, so that the backend stops by itself and, under several ranks,
every rank leaves the request at the same step (a request that ends earlier on a stop string is still run to that
point on the other ranks). Started by torchrun the worker runs on several ranks: rank 0 owns stdin / stdout and announces
every request to the others over a gloo control group (`server/distributed.py`). Role in the reference: the DSV4 path of cpp_engine/src/openai_server.cpp, whose model
lives in the same process; here the family's runtime is the Python one.
"""
from __future__ import annotations

import argparse
import json
import sys

from .engine import SamplingParams, TokenInfo


class ScriptedBackend:
    """Stand-in model for tests: replays the code points of `script`, then token 0; with log-probabilities asked for it
    reports ln(0.5) for every token and the following code points as alternatives."""

    def __init__(self, script: str):
        self.script = script

    def generate(self, prompt_ids, p: SamplingParams):
        for ch in self.script + "\0":
            t = ord(ch)
            if ch == "☠":
                raise TimeoutError("scripted step failure")
            yield TokenInfo(t, -0.6931472, [(t + i, -0.6931472 * (i + 1)) for i in range(p.logprobs)]) if p.logprobs >= 0 else t


def _reply(tok) -> dict:
    if isinstance(tok, TokenInfo):
        return {"token": int(tok.token), "logprob": float(tok.logprob), "top": [[int(i), float(lp)] for i, lp in tok.top]}
    return {"token": int(tok)}


def serve(backend, kind: str, max_context: int, stdin=sys.stdin, stdout=sys.stdout) -> int:
    gen = None
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        req = json.loads(line)
        op = req.get("op")
        if op == "quit":
            break
        try:
            if op == "hello":
                out = {"ok": True, "max_context": max_context, "model": kind}
            elif op == "prefill":
                s = req.get("sampler") or {}
                limit = int(req.get("max_tokens") or 0)
                params = SamplingParams(max_tokens=limit if limit > 0 else max_context, temperature=float(s.get("temperature", 0.0)), top_p=float(s.get("top_p", 1.0)),
                                        top_k=int(s.get("top_k", 0)), min_p=float(s.get("min_p", 0.0)),
                                        frequency_penalty=float(s.get("frequency_penalty", 0.0)), presence_penalty=float(s.get("presence_penalty", 0.0)),
                                        repetition_penalty=float(s.get("repetition_penalty", 1.0)), seed=req.get("seed"),
                                        stop_token_ids=tuple(int(t) for t in req.get("stop_token_ids", ())), logprobs=int(s.get("logprobs", -1)))
                if gen is not None:
                    gen.close()
                gen = iter(backend.generate([int(t) for t in req["tokens"]], params))
                out = _reply(next(gen))
            elif op == "end":
                # the request is over: under several ranks the others run it to the step where its limits end it, so does rank 0
                if gen is not None:
                    gen.close()
                    gen = None
                out = {"ok": True}
            elif op == "next":
                if gen is None:
                    raise RuntimeError("next before prefill")
                try:
                    out = _reply(next(gen))
                except StopIteration:
                    out = {"token": 0, "done": True}
            else:
                out = {"error": f"unknown op {op!r}", "lost": False}
        except Exception as e:                                     # the worker survives a failed request
            gen = None
            out = {"error": f"{type(e).__name__}: {e}", "lost": isinstance(e, TimeoutError)}
        stdout.write(json.dumps(out) + "\n")
        stdout.flush()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True, choices=["qwen", "gguf", "dsv4", "scripted"])
    ap.add_argument("--ckpt", default="")
    ap.add_argument("--max-context", type=int, default=4096)
    ap.add_argument("--tokenizer-path", default=None)
    ap.add_argument("--script", default="Hello", help="scripted: the text the stand-in model generates")
    ap.add_argument("--qwen-dspark", default="", help="qwen: directory of an external DSpark block drafter (greedy requests run as speculative rounds)")
    args = ap.parse_args(argv)
    import os
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    # stdout is the protocol channel of rank 0: whatever libraries (or other ranks) print goes to stderr
    real_stdout, sys.stdout = sys.stdout, sys.stderr
    group = None
    if world > 1:
        import torch.distributed as dist
        from . import distributed
        if args.model == "scripted":
            dist.init_process_group("gloo")
        else:
            import torch
            torch.cuda.set_device(local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        group = distributed.control_group()
    if args.model == "scripted":
        backend = ScriptedBackend(args.script)
    else:
        from . import backends
        backend, _ = backends.build(args.model, args.ckpt, args.max_context, tokenizer_path=args.tokenizer_path,
                                    qwen_dspark=args.qwen_dspark or None)
    if world > 1:
        from . import distributed
        if rank != 0:
            served = distributed.worker_loop(backend, group)
            print(f"model worker rank {rank}: followed {served} requests", file=sys.stderr, flush=True)
            return 0
        backend = distributed.DistributedBackend(backend, group)
    rc = serve(backend, args.model, args.max_context, stdout=real_stdout)
    if world > 1:
        backend.shutdown()
    return rc


if __name__ == "__main__":
    raise SystemExit(main())
