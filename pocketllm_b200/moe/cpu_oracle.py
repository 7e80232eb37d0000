"""CPU oracle of a routed FP4 MoE block (native C++ in `csrc/cpu/moe_cpu.cpp`) and the
plain PyTorch fp32 restatement it is checked against.

This is the benchmark's CPU configuration: hidden 1024, 8 routed experts top-2 with softmax
gating, one shared expert, SwiGLU intermediate 512, FP4 E2M1 weights with E8M0 scales per
32 values, 16 tokens. Reference path: `deepseek_cpu_moe_ext.routed_fp4_moe_forward(_raw)`
(src/csrc/deepseek_cpu_moe_ext.cpp:1778-1999) checked the same way by
tests/test_cpu_fp4_raw_moe.py.
"""
from __future__ import annotations

import ctypes
import time
from dataclasses import dataclass

import numpy as np
import torch

from ..formats import fp4
from ..ops import lib as _lib

SCORE_FUNCS = {"softmax": 0, "sigmoid": 1, "sqrtsoftplus": 2}


@dataclass
class Fp4MoEWeights:
    router: torch.Tensor                 # [E, H] fp32
    w13: torch.Tensor                    # uint8 [E, 2I, H/2]  gate rows then up rows
    s13: torch.Tensor                    # uint8 [E, 2I, H/32]
    w2: torch.Tensor                     # uint8 [E, H, I/2]
    s2: torch.Tensor                     # uint8 [E, H, I/32]
    shared_w13: torch.Tensor | None = None
    shared_s13: torch.Tensor | None = None
    shared_w2: torch.Tensor | None = None
    shared_s2: torch.Tensor | None = None
    bias: torch.Tensor | None = None

    @property
    def dims(self) -> tuple[int, int, int]:
        E, two_i, half_h = self.w13.shape
        return E, two_i // 2, half_h * 2


def random_fp4_moe(hidden: int = 1024, inter: int = 512, experts: int = 8, shared: bool = True, seed: int = 0,
                   sigma: float = 0.02) -> Fp4MoEWeights:
    g = torch.Generator().manual_seed(seed)
    w13, s13 = fp4.quantize_e2m1(torch.randn(experts, 2 * inter, hidden, generator=g) * sigma)
    w2, s2 = fp4.quantize_e2m1(torch.randn(experts, hidden, inter, generator=g) * sigma)
    out = Fp4MoEWeights(torch.randn(experts, hidden, generator=g) * sigma, w13, s13, w2, s2)
    if shared:
        a, b = fp4.quantize_e2m1(torch.randn(1, 2 * inter, hidden, generator=g) * sigma)
        c, d = fp4.quantize_e2m1(torch.randn(1, hidden, inter, generator=g) * sigma)
        out.shared_w13, out.shared_s13, out.shared_w2, out.shared_s2 = a, b, c, d
    return out


def route_torch(x: torch.Tensor, w: Fp4MoEWeights, topk: int, score_func: str = "softmax", norm_topk: bool = True,
                route_scale: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
    logits = x.float() @ w.router.t()
    if score_func == "softmax":
        sc = torch.softmax(logits, -1)
    elif score_func == "sigmoid":
        sc = torch.sigmoid(logits)
    else:
        sc = torch.sqrt(torch.nn.functional.softplus(logits))
    sel = sc + (w.bias if w.bias is not None else 0.0)
    ids = torch.topk(sel, topk, dim=-1).indices
    wt = torch.gather(sc, 1, ids)
    if norm_topk:
        wt = wt / wt.sum(-1, keepdim=True)
    return ids.int(), wt * route_scale


def forward_torch(x: torch.Tensor, w: Fp4MoEWeights, topk: int = 2, **route_kw) -> tuple[torch.Tensor, torch.Tensor]:
    """Dequantised fp32 MoE; returns (y [T, H], tokens per expert [E])."""
    E, I, H = w.dims
    ids, wt = route_torch(x, w, topk, **route_kw)
    d13 = fp4.dequantize_e2m1(w.w13, w.s13)
    d2 = fp4.dequantize_e2m1(w.w2, w.s2)
    xf = x.float()
    y = torch.zeros(x.shape[0], H)
    for t in range(x.shape[0]):
        for j in range(topk):
            e = int(ids[t, j])
            gu = d13[e] @ xf[t]
            y[t] += wt[t, j] * (d2[e] @ (torch.nn.functional.silu(gu[:I]) * gu[I:]))
    if w.shared_w13 is not None:
        s13, s2 = fp4.dequantize_e2m1(w.shared_w13, w.shared_s13)[0], fp4.dequantize_e2m1(w.shared_w2, w.shared_s2)[0]
        gu = xf @ s13.t()
        si = s13.shape[0] // 2
        y += (torch.nn.functional.silu(gu[:, :si]) * gu[:, si:]) @ s2.t()
    return y, torch.bincount(ids.reshape(-1).long(), minlength=E)


def _p(t: torch.Tensor | None, ctype):
    if t is None:
        return None
    return ctypes.cast(t.data_ptr(), ctypes.POINTER(ctype))


@dataclass
class Int8MoEWeights:
    """Routed experts as int8 codes with one fp32 scale per weight row (no shared expert in this format)."""
    router: torch.Tensor                 # [E, H] fp32
    w13: torch.Tensor                    # int8 [E, 2I, H]  gate rows then up rows
    s13: torch.Tensor                    # fp32 [E, 2I]
    w2: torch.Tensor                     # int8 [E, H, I]
    s2: torch.Tensor                     # fp32 [E, H]
    bias: torch.Tensor | None = None

    @property
    def dims(self) -> tuple[int, int, int]:
        E, two_i, H = self.w13.shape
        return E, two_i // 2, H

    @classmethod
    def quantize(cls, router: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, bias: torch.Tensor | None = None) -> "Int8MoEWeights":
        """fp32 w13 [E, 2I, H], w2 [E, H, I] -> int8 rows through the native row quantiser (absmax / 127)."""
        L = _lib.cpu()
        out = []
        for w in (w13, w2):
            wf = w.float().contiguous()
            q = torch.empty(wf.shape, dtype=torch.int8)
            sc = torch.empty(wf.shape[:-1], dtype=torch.float32)
            L.pk_cpu_quantize_int8_rows(_p(wf, ctypes.c_float), ctypes.c_long(wf.numel() // wf.shape[-1]), wf.shape[-1], _p(q, ctypes.c_int8),
                                        _p(sc, ctypes.c_float))
            out += [q, sc]
        return cls(router.float().contiguous(), out[0], out[1], out[2], out[3], bias)


def forward_native(x: torch.Tensor, w: "Fp4MoEWeights | Int8MoEWeights", topk: int = 2, score_func: str = "softmax", norm_topk: bool = True,
                   route_scale: float = 1.0, swiglu_limit: float = 0.0) -> tuple[torch.Tensor, torch.Tensor, float]:
    """Same block on the native CPU oracle; returns (y, counts, seconds of the expert pass)."""
    L = _lib.cpu()
    E, I, H = w.dims
    T = x.shape[0]
    xf = x.float().contiguous()
    ids = torch.empty(T, topk, dtype=torch.int32)
    wt = torch.empty(T, topk, dtype=torch.float32)
    router = w.router.float().contiguous()
    st = L.pk_cpu_route(_p(xf, ctypes.c_float), T, H, _p(router, ctypes.c_float), _p(w.bias, ctypes.c_float), E, topk,
                        SCORE_FUNCS[score_func], int(norm_topk), ctypes.c_float(route_scale), _p(ids, ctypes.c_int),
                        _p(wt, ctypes.c_float))
    if st != 0:
        raise RuntimeError(f"pk_cpu_route: status {st}")
    y = torch.empty(T, H, dtype=torch.float32)
    counts = torch.zeros(E, dtype=torch.int32)
    if isinstance(w, Int8MoEWeights):
        t0 = time.perf_counter()
        st = L.pk_cpu_moe_int8_forward(
            _p(xf, ctypes.c_float), T, H, I, E, topk, _p(ids, ctypes.c_int), _p(wt, ctypes.c_float), _p(w.w13.contiguous(), ctypes.c_int8),
            _p(w.s13.contiguous(), ctypes.c_float), _p(w.w2.contiguous(), ctypes.c_int8), _p(w.s2.contiguous(), ctypes.c_float),
            ctypes.c_float(swiglu_limit), _p(y, ctypes.c_float), _p(counts, ctypes.c_int))
        dt = time.perf_counter() - t0
        if st != 0:
            raise RuntimeError(f"pk_cpu_moe_int8_forward: status {st}")
        return y, counts, dt
    sh_i = 0 if w.shared_w13 is None else w.shared_w13.shape[1] // 2
    u8 = ctypes.c_uint8
    t0 = time.perf_counter()
    st = L.pk_cpu_moe_fp4_forward(
        _p(xf, ctypes.c_float), T, H, I, E, topk, _p(ids, ctypes.c_int), _p(wt, ctypes.c_float),
        _p(w.w13.contiguous(), u8), _p(w.s13.contiguous(), u8), _p(w.w2.contiguous(), u8), _p(w.s2.contiguous(), u8),
        _p(w.shared_w13, u8), _p(w.shared_s13, u8), _p(w.shared_w2, u8), _p(w.shared_s2, u8), sh_i,
        ctypes.c_float(swiglu_limit), _p(y, ctypes.c_float), _p(counts, ctypes.c_int))
    dt = time.perf_counter() - t0
    if st != 0:
        raise RuntimeError(f"pk_cpu_moe_fp4_forward: status {st}")
    return y, counts, dt
