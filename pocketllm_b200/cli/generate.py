"""Text generation from a checkpoint (reference: src/cli/generate.py:8-19 and src/cli/generate_glm.py:28-43).

    python -m pocketllm_b200.cli.generate --ckpt-path DIR_OR_GGUF [--ckpt-format auto|safetensors|gguf] [--tokenizer-path P]
        [--prompt TEXT | --input-file F | --interactive] [--chat] [--thinking] [--system-prompt S]
        [--max-new-tokens N] [--temperature T] [--top-p P] [--seed S] [--mtp] [--skip-special]

`safetensors` directories hold a DeepSeek-V4 checkpoint (run by the DSV4 runtime, optionally with MTP speculative
decoding); `gguf` files go through the architecture registry (MiniMax-M2, GLM-DSA). Tokenizer: a directory with
`tokenizer.json`, the GGUF's own metadata, or `chars` (one token per character, for tiny test models).
"""
from __future__ import annotations

import argparse
import sys
import time
from pathlib import Path

import torch

from ..encoding import chat, dsv4


def _load(args):
    fmt = args.ckpt_format
    if fmt == "auto":
        fmt = "gguf" if str(args.ckpt_path).endswith(".gguf") else "safetensors"
    if fmt == "gguf":
        from ..encoding import gguf_tokenizer
        from ..models import registry
        md = gguf_tokenizer.read_metadata(args.ckpt_path)
        rt = registry.build_runtime(args.ckpt_path, max_context=args.max_context)
        tok = None if args.tokenizer_path == "chars" else gguf_tokenizer.build_tokenizer(md)
        sp = gguf_tokenizer.special_ids(md)
        arch = md.get("general.architecture")
        render = (lambda m, thinking: chat.render_glm(m, thinking=thinking)) if arch == "glm-dsa" else (lambda m, thinking: chat.render_minimax(m, thinking=thinking))
        step = lambda t: rt.decode_one(t)
        return rt.prefill, step, None, tok, [i for i in (sp["eos"], sp["eot"]) if i is not None], render
    from ..models import deepseek_v4_loader as ld
    from ..models.deepseek_v4_runtime import DSV4Runtime
    cfg, W = ld.load_checkpoint(args.ckpt_path)
    rt = DSV4Runtime(cfg, W, max_context=args.max_context)
    tok = None
    if args.tokenizer_path and args.tokenizer_path != "chars":
        from tokenizers import Tokenizer
        tok = Tokenizer.from_file(str(Path(args.tokenizer_path) / "tokenizer.json"))
    eos = [tok.token_to_id(dsv4.EOS)] if tok is not None and tok.token_to_id(dsv4.EOS) is not None else [0]
    render = lambda m, thinking: dsv4.encode_messages(m, thinking_mode="thinking" if thinking else "chat")

    def step(t):
        rt.last_token = t
        return rt.forward_rows([t])[0]
    return rt.prefill, step, rt, tok, eos, render


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ckpt-path", required=True)
    ap.add_argument("--ckpt-format", choices=["auto", "safetensors", "gguf"], default="auto")
    ap.add_argument("--tokenizer-path", default=None)
    ap.add_argument("--prompt", default=None)
    ap.add_argument("--input-file", default="")
    ap.add_argument("--interactive", action="store_true")
    ap.add_argument("--chat", action="store_true")
    ap.add_argument("--thinking", action="store_true")
    ap.add_argument("--system-prompt", default=None)
    ap.add_argument("--max-new-tokens", type=int, default=64)
    ap.add_argument("--max-context", type=int, default=4096)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--mtp", action="store_true", help="DSV4: draft with the MTP block and verify two rows per pass")
    ap.add_argument("--skip-special", action="store_true")
    args = ap.parse_args(argv)
    prefill, step, dsv4_rt, tok, eos, render = _load(args)
    enc = (lambda s: tok.encode(s, add_special_tokens=False).ids) if tok is not None else (lambda s: [ord(c) for c in s])
    dec = (lambda ids: tok.decode(ids, skip_special_tokens=args.skip_special)) if tok is not None else (lambda ids: "".join(chr(i) for i in ids))
    prompts = []
    if args.prompt is not None:
        prompts.append(args.prompt)
    if args.input_file:
        prompts += [l.rstrip("\n") for l in Path(args.input_file).read_text().splitlines() if l.strip()]
    gen = torch.Generator().manual_seed(args.seed)

    def run(text: str) -> str:
        if args.chat:
            msgs = ([{"role": "system", "content": args.system_prompt}] if args.system_prompt else []) + [{"role": "user", "content": text}]
            text = render(msgs, args.thinking)
        ids = enc(text)
        t0 = time.perf_counter()
        if args.mtp and dsv4_rt is not None and args.temperature <= 0:
            out, stats = dsv4_rt.generate_mtp(ids, args.max_new_tokens)
            if any(t in eos for t in out):
                out = out[:min(out.index(t) for t in eos if t in out)]
            print(f"[mtp rounds={stats['rounds']} accepted={stats['accepted']}]", file=sys.stderr)
        else:
            out, t = [], prefill(ids)
            while len(out) < args.max_new_tokens and t not in eos:
                out.append(t)
                if args.temperature > 0 and dsv4_rt is not None:
                    from ..server.engine import SamplingParams, sample_token
                    lg = dsv4_rt.forward_logits([t])[0]
                    t = sample_token(lg.float().cpu(), SamplingParams(max_tokens=1, temperature=args.temperature, top_p=args.top_p), gen)
                else:
                    t = step(t)
        dt = time.perf_counter() - t0
        print(f"[{len(ids)} prompt tokens, {len(out)} generated, {len(out) / dt:.2f} tok/s]", file=sys.stderr)
        return dec(out)

    for p in prompts:
        print(run(p))
    if args.interactive:
        while True:
            try:
                line = input(">>> ")
            except EOFError:
                break
            if line.strip() in ("/exit", "/quit"):
                break
            print(run(line))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
