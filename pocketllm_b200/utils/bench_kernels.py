"""Micro-benchmarks of the hot kernels at the benchmark model's shapes, timed with CUDA
events (warm-up, synchronise on both sides, weight copies larger than L2 cycled through) and reported
as a fraction of the measured peaks (`MEASURED_PEAKS.json` at the repository root, else
6.65 TB/s / 1.59 PFLOP/s as the stated fallback).

    python -m pocketllm_b200.utils.bench_kernels --op gemm --M 512 --N 34816 --K 5120 --epi 1
    python -m pocketllm_b200.utils.bench_kernels --op matvec --N 34816 --K 5120 --epi 1
    python -m pocketllm_b200.utils.bench_kernels --suite
    python -m pocketllm_b200.utils.bench_kernels --op dsv4 --M 64 --ctx 32768      # indexer scores, top-k, sparse attention
    python -m pocketllm_b200.utils.bench_kernels --op deltanet --M 512 --heads 16,32  # one chunked DeltaNet layer
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from .. import ops


def peaks() -> tuple[float, float, str]:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def _time(fns, reps: int = 20, warmup: int = 3) -> float:
    """Mean time of one launch in microseconds. `fns` is a list of equivalent launches over
    different weight copies (together larger than L2) that are cycled through, so that every
    launch streams its weights from HBM; `reps` launches are queued back to back between one
    pair of events so that host launch overhead stays off the device timeline."""
    for i in range(warmup):
        fns[i % len(fns)]()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        fns[i % len(fns)]()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e3


def _copies(nbytes: int) -> int:
    return max(2, -(-(300 << 20) // nbytes))


def _fp8(n: int, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    w = torch.randint(0, 119, (n, k), device="cuda", dtype=torch.uint8)   # finite positive codes
    w |= torch.randint(0, 2, (n, k), device="cuda", dtype=torch.uint8) << 7
    s = torch.full(((n + 127) // 128, (k + 127) // 128), 1e-4, device="cuda", dtype=torch.float32)
    return w.view(torch.float8_e4m3fn), s


def bench_gemm(M: int, N: int, K: int, epi: int, iters: int, wfmt: str = "fp8") -> dict:
    hbm, tf, src = peaks()
    if wfmt in ("bf16", "bf16p"):
        ws = [((torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16), None) for _ in range(_copies(N * K * 2))]
    elif wfmt == "cublas":
        ws = [((torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16), None) for _ in range(_copies(N * K * 2))]
    else:
        ws = [_fp8(N, K) for _ in range(_copies(N * K))]
    a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    resid = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16) if epi == ops.EPI_RESID else None
    if wfmt == "cublas":
        fns = [(lambda w=w: torch.matmul(a, w.t())) for w, _ in ws]
    elif wfmt == "bf16p":
        fns = [(lambda w=w: ops.gemm_bf16(a, w, epi=epi, resid=resid)) for w, _ in ws]
    elif wfmt in ("fp8n1", "fp8n2"):
        # the native FP8 GEMM on the stored codes; the activation quantiser runs once, outside the timed calls
        aq, asc = ops.quant_act_fp8(a, 1 if wfmt == "fp8n1" else 2)
        fns = [(lambda w=w, s=s: ops.gemm_fp8(aq, asc, M, w.view(torch.uint8), s, epi=epi, resid=resid)) for w, s in ws]
    else:
        fns = [(lambda w=w, s=s: ops.gemm_umma(a, w, s, epi=epi, resid=resid)) for w, s in ws]
    us = _time(fns, iters)
    flops = 2.0 * M * N * K
    return {"op": "torch.matmul" if wfmt == "cublas" else "gemm_bf16" if wfmt == "bf16p" else "gemm_fp8" if wfmt.startswith("fp8n") else "gemm_umma", "wfmt": wfmt, "M": M, "N": N, "K": K, "epi": epi, "us": round(us, 2),
            "tflops": round(flops / us / 1e6, 1), "frac_of_peak": round(flops / us / 1e6 / tf, 3), "peak": f"{tf} TFLOP/s bf16 ({src})",
            "weight_gbs": round(N * K / us / 1e3, 1)}


def bench_attention(M: int, ctx: int, Hq: int, Hkv: int, iters: int, simt: bool = False) -> dict:
    """A prefill chunk of M rows ending at position ctx - 1: tcgen05 flash attention (or the split-context SIMT kernel)."""
    hbm, tf, src = peaks()
    D = 128
    kc = torch.randn(Hkv, ctx + 128, D, device="cuda").to(torch.bfloat16)
    vc = torch.randn(Hkv, ctx + 128, D, device="cuda").to(torch.bfloat16)
    q = torch.randn(M, Hq, D, device="cuda").to(torch.bfloat16)
    pos = torch.arange(ctx - M, ctx, device="cuda", dtype=torch.int32)
    fn = (lambda: ops.gqa_decode(q, kc, vc, pos, nsplit=1)) if simt else (lambda: ops.gqa_prefill(q, kc, vc, pos))
    us = _time([fn], iters)
    flops = 4.0 * D * Hq * sum(min(ctx - M + m + 1, ctx) for m in range(M))          # QK^T and PV over the causal extent
    return {"op": "gqa_decode(nsplit=1)" if simt else "gqa_prefill_umma", "M": M, "ctx": ctx, "Hq": Hq, "Hkv": Hkv, "us": round(us, 2),
            "tflops": round(flops / us / 1e6, 1), "frac_of_peak": round(flops / us / 1e6 / tf, 3), "peak": f"{tf} TFLOP/s bf16 ({src})"}


def bench_dsv4_select_attend(M: int, ctx: int, iters: int) -> list[dict]:
    """The sparse-attention step of a DeepSeek-V4-Flash-shaped ratio-4 layer for M rows ending at position ctx - 1:
    lightning-indexer scores over ctx / 4 compressed keys (64 index heads of 128), radix-select top-512, and sink-softmax
    attention of 64 heads of 512 over 128 window rows + the 512 selected rows (K == V)."""
    from ..ops import dsv4_ops as dk
    hbm, tf, src = peaks()
    H, hd, rd, win, ratio, ih, idim, topk = 64, 512, 64, 128, 4, 64, 128, 512
    n_ent, ring = ctx // ratio, win + M
    pos = torch.arange(ctx - M, ctx, device="cuda", dtype=torch.int32)
    ang = torch.rand(ctx + M, rd // 2, device="cuda") * 6.28
    cos_t, sin_t = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
    iq = torch.randn(M, ih, idim, device="cuda").to(torch.bfloat16)
    ik = torch.randn(n_ent, idim, device="cuda").to(torch.bfloat16)
    iw = torch.rand(M, ih, device="cuda")
    q = torch.randn(M, H, hd, device="cuda").to(torch.bfloat16)
    kv = torch.randn(ring + n_ent, hd, device="cuda").to(torch.bfloat16)
    sink = torch.zeros(H, device="cuda")
    score = dk.index_score(iq, ik, iw, pos, ratio, n_ent, 1.0 / (idim ** 0.5 * ih ** 0.5))
    sel = dk.topk_select(score, topk)
    out = []
    us = _time([lambda: dk.index_score(iq, ik, iw, pos, ratio, n_ent, 1.0)], iters)
    flops = 2.0 * M * ih * n_ent * idim
    out.append({"op": "dsv4 index_score", "M": M, "entries": n_ent, "us": round(us, 2), "tflops_fp32_simt": round(flops / us / 1e6, 1),
                "key_bytes_over_time_gbs": round(n_ent * idim * 2 / us / 1e3, 1)})
    us = _time([lambda: dk.topk_select(score, topk)], iters)
    nbytes = 5.0 * M * n_ent * 4                                           # five streaming passes over the scores
    out.append({"op": "topk_select", "M": M, "n": n_ent, "k": topk, "us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1),
                "frac_of_peak": round(nbytes / us / 1e3 / hbm, 3), "peak": f"{hbm} GB/s copy ({src}); the scores ({M * n_ent * 4 >> 10} KiB) stay in L2"})
    fn = lambda: dk.sparse_attn(q, kv, pos, sink, cos_t, sin_t, win=win, ring=ring, ratio=ratio, rd=rd, sel=sel)
    us = _time([fn], iters)
    flops = 4.0 * M * H * (win + topk) * hd
    nbytes = M * (win + topk) * hd * 2.0 + 2.0 * M * H * hd * 2
    out.append({"op": "dsv4 sparse_attn", "M": M, "H": H, "hd": hd, "rows_per_query": win + topk, "us": round(us, 2),
                "tflops_fp32_simt": round(flops / us / 1e6, 1), "unique_kv_gbs": round(nbytes / us / 1e3, 1),
                "note": "every head's warp re-reads the query row's KV rows (L1 / L2 hits): 64 x the unique bytes"})
    return out


def bench_deltanet(T: int, Hk: int, Hv: int, iters: int) -> dict:
    """The whole chunked Gated DeltaNet layer op (prep, chunk products, state pass, gated norm) for T tokens."""
    ld = (2 * Hk + 2 * Hv) * 128 + 2 * Hv
    ld = (ld + 7) // 8 * 8
    torch.manual_seed(0)
    proj = (torch.randn(T, ld, device="cuda") * 0.5).to(torch.bfloat16)
    C = (2 * Hk + Hv) * 128
    conv_w, conv_state = torch.randn(C, 4, device="cuda") * 0.3, torch.zeros(C, 3, device="cuda")
    A_log, dt_bias, norm_w = torch.zeros(Hv, device="cuda"), torch.zeros(Hv, device="cuda"), torch.ones(128, device="cuda")
    state = torch.zeros(Hv, 128, 128, device="cuda")
    us = _time([lambda: ops.deltanet_chunked(proj, Hk, Hv, conv_w, conv_state, A_log, dt_bias, norm_w, 1e-6, state)], iters, warmup=5)
    return {"op": "deltanet_chunked (prep + chunk + state + out)", "T": T, "key_heads": Hk, "value_heads": Hv, "us": round(us, 1)}


def bench_matvec(M: int, N: int, K: int, epi: int, iters: int) -> dict:
    hbm, tf, src = peaks()
    ws = [_fp8(N, K) for _ in range(_copies(N * K))]
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    gamma = torch.zeros(K, device="cuda")
    fns = [(lambda w=w, s=s: ops.matvec(x, w, s, gamma=gamma, epi=epi)) for w, s in ws]
    us = _time(fns, iters)
    nbytes = N * K + ws[0][1].numel() * 4
    return {"op": "matvec", "M": M, "N": N, "K": K, "epi": epi, "us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1),
            "frac_of_peak": round(nbytes / us / 1e3 / hbm, 3), "peak": f"{hbm} GB/s copy ({src})"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="gemm", choices=["gemm", "matvec", "attention", "attention-simt", "dsv4", "deltanet"])
    ap.add_argument("--ctx", type=int, default=8192, help="attention: position after the chunk's last row")
    ap.add_argument("--heads", default="24,4", help="attention: query heads, KV heads")
    ap.add_argument("--M", type=int, default=512)
    ap.add_argument("--N", type=int, default=34816)
    ap.add_argument("--K", type=int, default=5120)
    ap.add_argument("--epi", type=int, default=0)
    ap.add_argument("--iters", type=int, default=40)
    ap.add_argument("--wfmt", default="fp8", choices=["fp8", "bf16", "bf16p", "fp8n1", "fp8n2", "cublas"],
                    help="gemm: fp8 = codes decoded in shared memory, bf16p = persistent bf16 kernel, fp8n1 / fp8n2 = native FP8 math with one / two "
                         "activation terms, cublas = torch.matmul on bf16 (the library baseline)")
    ap.add_argument("--suite", action="store_true", help="all projections of the 27B-shaped model")
    args = ap.parse_args()
    if args.suite:
        for name, n, k, epi in [("in_proj", 12288, 5120, 0), ("out_proj", 5120, 4096, 0), ("qkv", 12288, 5120, 0),
                                ("o_proj", 5120, 5120, 0), ("gate_up", 34816, 5120, 1), ("down", 5120, 17408, 0)]:
            r = bench_gemm(512, n, k, epi, args.iters)
            r["name"] = name
            print(json.dumps(r))
            r = bench_matvec(1, n, k, epi, args.iters)
            r["name"] = name
            print(json.dumps(r))
        return 0
    if args.op == "deltanet":
        hk, hv = (int(v) for v in args.heads.split(",")) if args.heads != "24,4" else (16, 32)
        print(json.dumps(bench_deltanet(args.M, hk, hv, args.iters)))
        return 0
    if args.op == "dsv4":
        for r in bench_dsv4_select_attend(min(args.M, 64), args.ctx, args.iters):
            print(json.dumps(r))
        return 0
    if args.op.startswith("attention"):
        hq, hkv = (int(v) for v in args.heads.split(","))
        print(json.dumps(bench_attention(args.M, args.ctx, hq, hkv, args.iters, simt=args.op == "attention-simt")))
        return 0
    r = bench_gemm(args.M, args.N, args.K, args.epi, args.iters, args.wfmt) if args.op == "gemm" else bench_matvec(args.M if args.op != "matvec" or args.M <= 8 else 1, args.N, args.K, args.epi, args.iters)
    print(json.dumps(r))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
