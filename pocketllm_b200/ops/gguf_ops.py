"""Bindings of the raw-GGUF-block kernels: linear layers, router top-k, route grouping and
the routed-expert pass. Weights are uint8 tensors holding the file's blocks unchanged."""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import torch

from . import _check, _ptr, _sm_count, _stream
from . import lib as _lib

# device type ids (reference: src/loader/gguf/quant_types.py, plus q8_0 and bf16)
DEVICE_TYPE = {"iq2_xxs": 0, "q2_k": 1, "iq1_m": 2, "q4_k": 3, "q5_k": 4, "iq2_xs": 5, "iq3_xxs": 6, "iq4_xs": 7, "mxfp4": 11,
               "q6_k": 8, "q8_0": 9, "bf16": 10}
SCORE_FUNCS = {"softmax": 0, "sigmoid": 1, "sqrtsoftplus": 2}


def row_bytes(type_name: str, K: int) -> int:
    return K // 256 * _lib.kernels().pk_gguf_block_bytes(DEVICE_TYPE[type_name])


def gguf_linear(x: torch.Tensor, w_raw: torch.Tensor, type_name: str, N: int, *, gamma: torch.Tensor | None = None,
                eps: float = 1e-6, epi: int = 0) -> torch.Tensor:
    """y = rmsnorm?(x) @ dequant(W)^T for any number of rows.

    Up to `TENSOR_CORE_MIN_ROWS - 1` rows stream the quantised blocks and decode them in registers (groups of up to 8
    rows per launch). From there on the weight is decoded once into a bf16 scratch and the product runs on the
    tcgen05 GEMM: one decode instead of one per 8 rows (the reference switches to its prefill kernels for rows > 1,
    src/components/gguf/quantized_ops.py:9-76)."""
    M, K = x.shape
    ncols = N // 2 if epi == 1 else N
    if M >= TENSOR_CORE_MIN_ROWS and K % 64 == 0 and (epi != 1 or (N // 2) % 128 == 0):
        from . import gemm_bf16, rmsnorm, EPI_BF16, EPI_SWIGLU, EPI_F32
        w = _dequant_scratch(w_raw, type_name, N, K)
        xin = x.contiguous() if gamma is None else rmsnorm(x.contiguous(), gamma, mode=2, eps=eps)
        return gemm_bf16(xin, w, epi={0: EPI_BF16, 1: EPI_SWIGLU, 2: EPI_F32}[epi])
    y = torch.empty(M, ncols, device=x.device, dtype=torch.float32 if epi == 2 else torch.bfloat16)
    step = max(1, min(8, (184 * 1024) // (K * 4)))
    step = 8 if step >= 8 else 4 if step >= 4 else 2 if step >= 2 else 1
    for m0 in range(0, M, step):
        m = min(step, M - m0)
        st = _lib.kernels().pk_gguf_linear(_ptr(w_raw), c_int(DEVICE_TYPE[type_name]), c_int(N), c_int(K), c_int(m),
                                           _ptr(x[m0:]), _ptr(gamma), c_float(eps), c_int(epi), _ptr(y[m0:]), c_int(ncols),
                                           c_int(_sm_count()), _stream())
        _check(st, "pk_gguf_linear")
    return y


TENSOR_CORE_MIN_ROWS = 32
_scratch: dict = {}


def _dequant_scratch(w_raw: torch.Tensor, type_name: str, N: int, K: int) -> torch.Tensor:
    """bf16 [N, K] copy of a quantised weight in a per-device buffer that the next call reuses (stream ordered)."""
    key = (w_raw.device.index, torch.cuda.current_stream().cuda_stream)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < N * K:
        buf = torch.empty(N * K, device=w_raw.device, dtype=torch.bfloat16)
        _scratch[key] = buf
    out = buf[: N * K].view(N, K)
    rb = row_bytes(type_name, K)
    st = _lib.kernels().pk_gguf_dequant_rows(_ptr(w_raw), c_int(DEVICE_TYPE[type_name]), c_void_p(0), c_int(N), c_int(K), c_int(0),
                                             c_int(w_raw.numel() // rb), _ptr(out), _stream())
    _check(st, "pk_gguf_dequant_rows")
    return out


def router_topk(x: torch.Tensor, router_w: torch.Tensor, topk: int, *, bias: torch.Tensor | None = None,
                score_func: str = "sigmoid", norm_topk: bool = True, route_scale: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
    T, H = x.shape
    E = router_w.shape[0]
    ids = torch.empty(T, topk, device=x.device, dtype=torch.int32)
    w = torch.empty(T, topk, device=x.device, dtype=torch.float32)
    st = _lib.kernels().pk_router_topk(_ptr(x), _ptr(router_w), _ptr(bias), c_int(T), c_int(H), c_int(E), c_int(topk),
                                       c_int(SCORE_FUNCS[score_func]), c_int(int(norm_topk)), c_float(route_scale), _ptr(ids),
                                       _ptr(w), _stream())
    _check(st, "pk_router_topk")
    return ids, w


class Routes(tuple):
    """(seg_start [E+1], route_token [R], route_weight [R]) plus `.src` [R]: original route index t * topk + k of each
    sorted route, and `.topk`."""
    src: torch.Tensor
    topk: int


def group_routes(ids: torch.Tensor, weights: torch.Tensor, E: int) -> Routes:
    """Sort routes by expert (stable in route index)."""
    T, topk = ids.shape
    seg = torch.empty(E + 1, device=ids.device, dtype=torch.int32)
    tok = torch.empty(T * topk, device=ids.device, dtype=torch.int32)
    rw = torch.empty(T * topk, device=ids.device, dtype=torch.float32)
    src = torch.empty(T * topk, device=ids.device, dtype=torch.int32)
    st = _lib.kernels().pk_group_routes(_ptr(ids), _ptr(weights), c_int(T), c_int(topk), c_int(E), _ptr(seg), _ptr(tok),
                                        _ptr(rw), _ptr(src), _stream())
    _check(st, "pk_group_routes")
    r = Routes((seg, tok, rw))
    r.src, r.topk = src, topk
    return r


def gguf_moe_forward(x: torch.Tensor, w13_raw: torch.Tensor, w2_raw: torch.Tensor, type13: str, type2: str, E: int, inter: int,
                     seg: torch.Tensor, tok: torch.Tensor, rw: torch.Tensor, *, limit: float = 0.0, expert_offset: int = 0,
                     local_experts: int | None = None, out: torch.Tensor | None = None, routes: "Routes | None" = None) -> torch.Tensor:
    """Routed experts of this rank accumulated into fp32 `out` [T, H] (zeroed when not given). With `routes` (the object
    `group_routes` returned) the per-token sum runs in a fixed order and the result is bitwise reproducible; without it
    the routes are added with atomics."""
    T, H = x.shape
    R = tok.numel()
    local = E if local_experts is None else local_experts
    if out is None:
        out = torch.zeros(T, H, device=x.device, dtype=torch.float32)
    hbuf = torch.empty(R, inter, device=x.device, dtype=torch.float32)
    if routes is not None:
        ybuf = torch.empty(R, H, device=x.device, dtype=torch.float32)
        pos = torch.empty(R, device=x.device, dtype=torch.int32)
        st = _lib.kernels().pk_gguf_moe_forward_det(
            _ptr(w13_raw), _ptr(w2_raw), c_int(DEVICE_TYPE[type13]), c_int(DEVICE_TYPE[type2]), c_int(E), c_int(H), c_int(inter),
            _ptr(x), _ptr(seg), _ptr(tok), _ptr(rw), _ptr(routes.src), _ptr(hbuf), _ptr(ybuf), _ptr(pos), _ptr(out), c_int(T),
            c_int(routes.topk), c_float(limit), c_int(expert_offset), c_int(local), c_int(_sm_count()), _stream())
        _check(st, "pk_gguf_moe_forward_det")
        return out
    st = _lib.kernels().pk_gguf_moe_forward(
        _ptr(w13_raw), _ptr(w2_raw), c_int(DEVICE_TYPE[type13]), c_int(DEVICE_TYPE[type2]), c_int(E), c_int(H), c_int(inter),
        _ptr(x), _ptr(seg), _ptr(tok), _ptr(rw), _ptr(hbuf), _ptr(out), c_float(limit), c_int(expert_offset), c_int(local),
        c_int(_sm_count()), _stream())
    _check(st, "pk_gguf_moe_forward")
    return out


_GROUPED_SCRATCH: dict = {}


def gguf_moe_forward_grouped(x: torch.Tensor, w13_raw: torch.Tensor, w2_raw: torch.Tensor, type13: str, type2: str, E: int, inter: int,
                             routes: "Routes", *, expert_offset: int = 0, local_experts: int | None = None,
                             out: torch.Tensor | None = None, peer=None) -> torch.Tensor:
    """Routed experts of this rank on the tensor cores, for steps with many routes (prefill): the rank's experts are decoded
    to bf16 once per call into a scratch that is reused across layers, token rows are gathered in expert order, and two
    grouped tcgen05 GEMMs (gate|up with the SwiGLU epilogue, then down) run one persistent launch each over every
    (expert, row tile, column block) that has rows; the tile list comes from the route segments on the device. The
    per-token sum runs in route order (bitwise reproducible). Same result as `gguf_moe_forward` up to bf16 rounding of the
    hidden activations. With `peer` (a `PeerAllReduce` of the expert-parallel group) whose arena holds T * H floats the result
    is already summed over the ranks (`routes.combined` is set): the combine runs as peer stores out of the reduce."""
    from . import EPI_F32, EPI_SWIGLU
    seg, tok, rw = routes
    T, H = x.shape
    R = tok.numel()
    local = E if local_experts is None else local_experts
    dev = x.device
    if out is None:
        out = torch.zeros(T, H, device=dev, dtype=torch.float32)
    key = (dev.index, local, H, inter)
    sc = _GROUPED_SCRATCH.get(key)
    if sc is None:
        sc = (torch.empty(local * 2 * inter, H, device=dev, dtype=torch.bfloat16), torch.empty(local * H, inter, device=dev, dtype=torch.bfloat16))
        _GROUPED_SCRATCH.clear()          # one shape at a time: the scratch is as large as the layer's experts in bf16
        _GROUPED_SCRATCH[key] = sc
    w13, w2 = sc
    K = _lib.kernels()
    _check(K.pk_gguf_dequant_rows(_ptr(w13_raw), c_int(DEVICE_TYPE[type13]), c_void_p(0), c_int(local * 2 * inter), c_int(H), c_int(0),
                                  c_int(local * 2 * inter), _ptr(w13), _stream()), "pk_gguf_dequant_rows(w13)")
    _check(K.pk_gguf_dequant_rows(_ptr(w2_raw), c_int(DEVICE_TYPE[type2]), c_void_p(0), c_int(local * H), c_int(inter), c_int(0), c_int(local * H),
                                  _ptr(w2), _stream()), "pk_gguf_dequant_rows(w2)")
    xg = x.index_select(0, tok.long())                                   # [R, H] rows in expert order
    hbuf = torch.empty(R, inter, device=dev, dtype=torch.bfloat16)
    ybuf = torch.empty(R, H, device=dev, dtype=torch.float32)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    segl = seg[expert_offset:]
    _check(K.pk_gemm_bf16_grouped(_ptr(xg), c_int(H), _ptr(w13), _ptr(segl), c_int(local), c_int(R), c_int(2 * inter), c_int(H), c_int(EPI_SWIGLU),
                                  _ptr(hbuf), c_int(inter), _ptr(status), c_int(_sm_count()), _stream()), "pk_gemm_bf16_grouped(w13)")
    _check(K.pk_gemm_bf16_grouped(_ptr(hbuf), c_int(inter), _ptr(w2), _ptr(segl), c_int(local), c_int(R), c_int(H), c_int(inter), c_int(EPI_F32),
                                  _ptr(ybuf), c_int(H), _ptr(status), c_int(_sm_count()), _stream()), "pk_gemm_bf16_grouped(w2)")
    pos = torch.empty(R, device=dev, dtype=torch.int32)
    routes.combined = False
    if peer is not None and T * H <= peer.capacity:
        # several ranks: the per-token reduce is the producer of the combine kernel, which stores this rank's sums into every
        # rank's arena, signals, waits (bounded) and adds the ranks' slots: `out` is the sum over all ranks' experts
        _check(K.pk_invert_routes(_ptr(routes.src), c_int(R), _ptr(pos), _stream()), "pk_invert_routes")
        peer.moe_combine(ybuf, rw, pos, seg, expert_offset, local, T, routes.topk, out)
        routes.combined = True
        return out
    _check(K.pk_moe_reduce_routes(_ptr(ybuf), _ptr(rw), _ptr(routes.src), _ptr(seg), c_int(T), c_int(routes.topk), c_int(H), c_int(expert_offset),
                                  c_int(local), _ptr(pos), _ptr(out), _stream()), "pk_moe_reduce_routes")
    return out


GROUPED_MIN_ROUTES_PER_EXPERT = 4     # below this the decode of every local expert costs more than the route kernels' per-route decode


def moe_forward(x: torch.Tensor, w13_raw: torch.Tensor, w2_raw: torch.Tensor, type13: str, type2: str, E: int, inter: int, routes: "Routes", *,
                limit: float = 0.0, expert_offset: int = 0, local_experts: int | None = None, peer=None) -> torch.Tensor:
    """Routed experts of this rank, fp32 [T, H]: the grouped tensor-core path for steps with many routes per expert
    (prefill), the per-route streaming kernels otherwise (decode, clamped SwiGLU)."""
    seg, tok, rw = routes
    local = E if local_experts is None else local_experts
    H = x.shape[1]
    if (limit == 0.0 and tok.numel() >= GROUPED_MIN_ROUTES_PER_EXPERT * local and inter % 128 == 0 and H % 128 == 0 and local <= 512):
        return gguf_moe_forward_grouped(x, w13_raw, w2_raw, type13, type2, E, inter, routes, expert_offset=expert_offset, local_experts=local,
                                        peer=peer)
    routes.combined = False
    return gguf_moe_forward(x, w13_raw, w2_raw, type13, type2, E, inter, seg, tok, rw, limit=limit, expert_offset=expert_offset,
                            local_experts=local, routes=routes)


def gguf_dequant_rows(w_raw: torch.Tensor, type_name: str, K: int, rows: torch.Tensor | None = None, *, nrows: int | None = None,
                      row_offset: int = 0) -> torch.Tensor:
    """Decode rows of a quantised table to bf16 (quantised embedding gather, or a whole
    weight when `rows` is None)."""
    rb = row_bytes(type_name, K)
    table_rows = w_raw.numel() // rb
    n = rows.numel() if rows is not None else (nrows if nrows is not None else table_rows)
    out = torch.empty(n, K, device=w_raw.device, dtype=torch.bfloat16)
    st = _lib.kernels().pk_gguf_dequant_rows(_ptr(w_raw), c_int(DEVICE_TYPE[type_name]), _ptr(rows), c_int(n), c_int(K),
                                             c_int(row_offset), c_int(table_rows), _ptr(out), _stream())
    _check(st, "pk_gguf_dequant_rows")
    return out
