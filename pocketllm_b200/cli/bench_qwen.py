"""Benchmark drivers of the hybrid decoder beyond the headline run of `bench.py`: long contexts, the multi-token
predictor, and prefix reuse across requests. Roles of the reference's scripts/bench_qwen_long_context.py,
bench_qwen_mtp.py, bench_qwen_dspark.py and bench_qwen_prefix_cache.py. One JSON object is printed (and written with --out).

    python -m pocketllm_b200.cli.bench_qwen long-context --gpus 1 --prompt-lens 4096,8192,32768 --decode-len 64
    python -m pocketllm_b200.cli.bench_qwen mtp --gpus 1 --prompt-len 512 --decode-len 256 --max-draft 4
    python -m pocketllm_b200.cli.bench_qwen prefix-cache --gpus 1 --prompt-len 4096 --turns 4
    python -m pocketllm_b200.cli.bench_qwen dspark --gpus 1 --prompt-len 512 --decode-len 64 --max-draft 7

With --gpus N > 1 the driver starts itself under `torch.distributed.run` (one rank per GPU, 127.0.0.1 rendezvous);
every rank generates the same tokens or the run fails. Weights are random (N(0, 0.02) quantised to FP8) in the
27B shape unless --ckpt names a checkpoint directory; timings are device times (CUDA events inside the engine), the
maximum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys


def _engine(args, **kw):
    import torch
    import torch.distributed as dist
    from ..models import qwen_hybrid as qh
    from ..parallel import tp
    rank, world, local = tp.env_rank_world()
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if args.ckpt:
        from pathlib import Path
        cfg = qh.QwenHybridConfig.from_json((Path(args.ckpt) / "config.json").read_text())
    else:
        cfg = qh.QwenHybridConfig.benchmark_27b() if args.model == "qwen27b" else qh.QwenHybridConfig.tiny()
    eng = qh.QwenEngine(cfg, tp_rank=rank, tp_world=world, device=local, max_context=kw.pop("max_context"),
                        prefill_chunk=args.prefill_chunk, kv_cache_dtype=args.kv_cache_dtype, **kw)
    if args.ckpt:
        eng.load(args.ckpt)
    else:
        eng.init_random(seed=0, sigma=0.02)
    if world > 1:
        tp.connect_engine(eng)
    return cfg, eng, rank, world


def _max_over_ranks(vals: list[float]) -> list[float]:
    import torch
    import torch.distributed as dist
    if not dist.is_initialized():
        return vals
    t = torch.tensor(vals, dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def _same_on_all_ranks(tokens: list[int]) -> bool:
    import torch.distributed as dist
    if not dist.is_initialized():
        return True
    box = [None] * dist.get_world_size()
    dist.all_gather_object(box, tokens)
    return all(b == box[0] for b in box)


def _prompt(cfg, n: int, seed: int) -> list[int]:
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()


def run_long_context(args) -> dict:
    lens = [int(x) for x in args.prompt_lens.split(",")]
    cfg, eng, rank, world = _engine(args, max_context=max(lens) + args.decode_len + 16)
    rows = []
    for n in lens:
        best = None
        for rep in range(args.repeats):
            eng.reset()
            first = eng.prefill(_prompt(cfg, n, 100 + n))
            toks = [first] + eng.decode(args.decode_len)
            t = eng.timings()
            pre, dec = _max_over_ranks([t["prefill_ms"], t["decode_ms"]])
            row = {"prompt_tokens": n, "decode_tokens": args.decode_len, "prefill_tok_s": round(n / (pre / 1e3), 1),
                   "decode_tok_s": round(args.decode_len / (dec / 1e3), 2), "prefill_ms": round(pre, 2),
                   "decode_ms_per_token": round(dec / args.decode_len, 4), "ranks_agree": _same_on_all_ranks(toks)}
            if best is None or row["decode_tok_s"] > best["decode_tok_s"]:
                best = row
        rows.append(best)
    out = {"bench": "qwen_long_context", "n_gpus": world, "kv_cache_dtype": args.kv_cache_dtype, "kv_cache_bytes_per_rank": eng.kv_cache_bytes,
           "decode_kernel": "persistent" if eng.persistent_decode else "per-projection", "comm_status": eng.comm_status(), "rows": rows}
    eng.close()
    return out if rank == 0 else {}


def _row_count_independent_kernels() -> None:
    """Speculative loops compare picks of passes over different numbers of rows (plain step, verify, replay). One and two rows
    normally stream through the shared-memory rings and three to eight through registers, which add in different orders;
    with random weights the logits are nearly flat and such a difference flips picks. POCKET_MATVEC_RING=0 keeps every row
    count on the register-streaming kernel, whose arithmetic per row does not depend on the row count."""
    os.environ.setdefault("POCKET_MATVEC_RING", "0")


def run_mtp(args) -> dict:
    _row_count_independent_kernels()
    cfg, eng, rank, world = _engine(args, max_context=args.prompt_len + args.decode_len + 32, mtp=True)
    prompt = _prompt(cfg, args.prompt_len, 7)
    eng.reset()
    first = eng.prefill(prompt)
    plain = [first] + eng.decode(args.decode_len)
    plain_ms, = _max_over_ranks([eng.timings()["decode_ms"]])
    res = {"bench": "qwen_mtp", "n_gpus": world, "prompt_tokens": args.prompt_len, "decode_tokens": args.decode_len,
           "plain_decode_tok_s": round(args.decode_len / (plain_ms / 1e3), 2), "rows": []}
    # the predictor's own drafts (random weights: low acceptance) and the known continuation as drafts (acceptance 1: the
    # ceiling of what a perfect drafter buys with this verify path)
    for label, replay in (("predictor_drafts", None), ("perfect_drafts", plain[1:])):
        eng.reset()
        eng.set_draft_replay(replay or [])
        toks, st = eng.generate_mtp(prompt, args.decode_len + 1, args.max_draft)
        ms, = _max_over_ranks([eng.timings()["decode_ms"]])
        res["rows"].append({"drafts": label, "decode_tok_s": round(args.decode_len / (ms / 1e3), 2),
                            "speedup_vs_plain": round(plain_ms / ms, 3), "acceptance": round(st["accepted"] / max(st["proposed"], 1), 3),
                            "rounds": st["rounds"], "rollbacks": st["rollbacks"], "tokens_equal_plain": toks == plain,
                            "ranks_agree": _same_on_all_ranks(toks)})
    eng.set_draft_replay([])
    res["comm_status"] = eng.comm_status()
    eng.close()
    return res if rank == 0 else {}


def _continue(spec, first: int, n: int) -> list[int]:
    """n more tokens after a prefill that produced `first`, through the speculator's rounds (decode time only)."""
    return spec.decode(first, n)


def run_dspark(args) -> dict:
    """Block drafter on one GPU: the published drafter shape (5 layers, block 7) with random weights next to the target. Random
    drafts are almost never right, so the row of interest is the cost model: drafting time, verify time for k + 1 rows and the
    plain step time give the acceptance at which drafting breaks even; `perfect_drafts` replays the known continuation."""
    import time
    import torch
    from ..models import qwen_dspark as qd
    from ..models.qwen_dspark_runtime import QwenDSparkRuntime, QwenDSparkSpeculator
    if args.gpus != 1:
        raise SystemExit("the block drafter's taps are captured on one rank")
    _row_count_independent_kernels()
    cfg, eng, rank, world = _engine(args, max_context=args.prompt_len + args.decode_len + 64, persistent_decode=0)
    tiny = args.model == "tiny"
    dcfg = qd.QwenDSparkConfig(hidden_size=cfg.hidden_size, intermediate_size=256 if tiny else 17408, num_hidden_layers=2 if tiny else 5,
                               num_attention_heads=2 if tiny else 40, num_key_value_heads=1 if tiny else 8, head_dim=128, vocab_size=cfg.vocab_size,
                               block_size=7, markov_rank=64 if tiny else 256, mask_token_id=cfg.vocab_size - 1,
                               target_layer_ids=tuple(sorted({min(i, cfg.num_hidden_layers - 1) for i in ((1, 3) if tiny else (4, 16, 28, 40, 52))})))
    W = {}
    g = torch.Generator(device="cuda").manual_seed(3)
    for name, shape in qd.tensor_names(dcfg):                       # made on the device: the 5-layer drafter is 3.6 G parameters
        if name.endswith("norm.weight"):
            W[name] = torch.ones(*shape, device="cuda", dtype=torch.bfloat16)
        else:
            W[name] = (torch.randn(*shape, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    embed = (torch.randn(cfg.vocab_size, cfg.hidden_size, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    drafter = QwenDSparkRuntime(dcfg, W, embed, embed, max_context=args.prompt_len + args.decode_len + 64)
    prompt = _prompt(cfg, args.prompt_len, 7)
    eng.reset()
    first = eng.prefill(prompt)
    plain = [first] + eng.decode(args.decode_len)
    plain_ms = eng.timings()["decode_ms"]
    spec = QwenDSparkSpeculator(eng, drafter, max_draft=args.max_draft)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    got = spec.generate(prompt, args.decode_len + 1, chunk=args.prefill_chunk)
    torch.cuda.synchronize()
    spec_s = time.perf_counter() - t0
    # cost of the parts, timed on the device
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        drafter.propose(plain[-1])
    e1.record()
    torch.cuda.synchronize()
    propose_ms = e0.elapsed_time(e1) / 5
    eng.reset()
    eng.prefill(prompt)
    t0 = time.perf_counter()
    eng.forward_rows(plain[: args.max_draft + 1])
    verify_ms = (time.perf_counter() - t0) * 1e3
    step_ms = plain_ms / args.decode_len
    # the known continuation as drafts (acceptance 1): what a perfect drafter buys with this verify path
    class _Replay:
        cfg = dcfg
        def __init__(self, seq): self.seq, self.at = seq, 0
        def reset(self): self.at = 0
        def append_target_taps(self, taps, position): pass
        def propose(self, anchor):
            self.at = self.seq.index(anchor, self.at) + 1 if anchor in self.seq[self.at:] else len(self.seq)
            nxt = self.seq[self.at:self.at + dcfg.block_size]
            nxt = nxt + [0] * (dcfg.block_size - len(nxt))
            return torch.tensor(nxt, dtype=torch.int32), torch.ones(dcfg.block_size), None
    perfect = QwenDSparkSpeculator(eng, _Replay(plain), max_draft=args.max_draft)
    eng.reset()
    first2 = perfect.prefill(prompt, chunk=args.prefill_chunk)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    got2 = [first2] + _continue(perfect, first2, args.decode_len)
    torch.cuda.synchronize()
    perfect_s = time.perf_counter() - t0
    res = {"bench": "qwen_dspark", "n_gpus": 1, "prompt_tokens": args.prompt_len, "decode_tokens": args.decode_len, "block_size": dcfg.block_size,
           "max_draft": args.max_draft, "drafter_layers": dcfg.num_hidden_layers, "plain_decode_tok_s": round(1e3 / step_ms, 2),
           "plain_step_ms": round(step_ms, 3), "propose_ms": round(propose_ms, 3), f"verify_{args.max_draft + 1}_rows_ms": round(verify_ms, 3),
           "break_even_tokens_per_round": round((propose_ms + verify_ms) / step_ms, 2),
           "perfect_drafts": {"tokens_equal_plain": got2 == plain, "decode_tok_s": round(args.decode_len / perfect_s, 2),
                              "speedup_vs_plain": round((args.decode_len / perfect_s) / (1e3 / step_ms), 3), "rounds": perfect.stats["rounds"],
                              "accepted": perfect.stats["accepted"], "proposed": perfect.stats["proposed"], "rollbacks": perfect.stats["rollbacks"]},
           "random_drafter": {"tokens_equal_plain": got == plain, "rounds": spec.stats["rounds"], "proposed": spec.stats["proposed"],
                              "accepted": spec.stats["accepted"], "rollbacks": spec.stats["rollbacks"],
                              "wall_tok_s_incl_prefill": round(args.decode_len / spec_s, 2)}}
    eng.close()
    return res


def run_prefix_cache(args) -> dict:
    ctx = args.prompt_len + args.turns * (args.turn_tokens + args.decode_len) + 64
    cfg, eng, rank, world = _engine(args, max_context=ctx)
    eng.configure_prefix_cache(True, snapshot_interval=args.snapshot_interval, max_snapshots=args.max_snapshots)
    convo = _prompt(cfg, args.prompt_len, 3)
    rows = []
    for turn in range(args.turns):
        first, st = eng.prefill_reusing(convo)
        pre_ms, = _max_over_ranks([eng.timings()["prefill_ms"]])
        reply = [first] + eng.decode(args.decode_len - 1)
        rows.append({"request": turn + 1, "prompt_tokens": len(convo), "reused_tokens": st["reused_tokens"], "computed_tokens": st["computed_tokens"],
                     "resume": st["source"], "request_prefill_tok_s": round(len(convo) / (pre_ms / 1e3), 1), "prefill_ms": round(pre_ms, 2),
                     "snapshots": st["snapshots"], "ranks_agree": _same_on_all_ranks(reply)})
        convo = convo + reply + _prompt(cfg, args.turn_tokens, 50 + turn)      # the chat grows: old prompt + reply + new turn
    # a request that shares only the first half of the original prompt: resumes from a stored recurrent state
    fork = convo[: args.prompt_len // 2] + _prompt(cfg, 64, 999)
    first, st = eng.prefill_reusing(fork)
    pre_ms, = _max_over_ranks([eng.timings()["prefill_ms"]])
    rows.append({"request": "fork", "prompt_tokens": len(fork), "reused_tokens": st["reused_tokens"], "resume": st["source"],
                 "request_prefill_tok_s": round(len(fork) / (pre_ms / 1e3), 1), "prefill_ms": round(pre_ms, 2)})
    out = {"bench": "qwen_prefix_cache", "n_gpus": world, "snapshot_interval": args.snapshot_interval, "rows": rows,
           "comm_status": eng.comm_status()}
    eng.close()
    return out if rank == 0 else {}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("bench", choices=["long-context", "mtp", "prefix-cache", "dspark"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--model", default="qwen27b", choices=["qwen27b", "tiny"])
    ap.add_argument("--ckpt", default="")
    ap.add_argument("--kv-cache-dtype", default="bf16", choices=["bf16", "fp8"])
    ap.add_argument("--prefill-chunk", type=int, default=512)
    ap.add_argument("--prompt-lens", default="4096,8192,32768")
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--decode-len", type=int, default=64)
    ap.add_argument("--repeats", type=int, default=1)
    ap.add_argument("--max-draft", type=int, default=4)
    ap.add_argument("--turns", type=int, default=4)
    ap.add_argument("--turn-tokens", type=int, default=32)
    ap.add_argument("--snapshot-interval", type=int, default=1024)
    ap.add_argument("--max-snapshots", type=int, default=16)
    ap.add_argument("--master-port", type=int, default=29733)
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 and world == 1:
        # re-enter under torchrun, one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1",
               "--master-port", str(args.master_port), "-m", "pocketllm_b200.cli.bench_qwen", *(argv if argv is not None else sys.argv[1:])]
        return subprocess.run(cmd, env=dict(os.environ, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "0"))).returncode
    if args.gpus != world:
        ap.error(f"--gpus {args.gpus} but WORLD_SIZE is {world}")
    res = {"long-context": run_long_context, "mtp": run_mtp, "prefix-cache": run_prefix_cache, "dspark": run_dspark}[args.bench](args)
    if res:
        text = json.dumps(res)
        print(text, flush=True)
        if args.out:
            with open(args.out, "w") as f:
                f.write(text + "\n")
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
