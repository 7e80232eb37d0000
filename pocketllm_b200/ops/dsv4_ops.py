"""Bindings of the DeepSeek-V4 kernels (`csrc/kernels/dsv4.cu`)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import torch

from . import _check, _ptr, _stream
from . import lib as _lib

PREP_NORM, PREP_ROPE, PREP_INV_ROPE, PREP_HADAMARD_FP4 = 1, 2, 4, 8


def hc_pre(h: torch.Tensor, fn: torch.Tensor, scale: torch.Tensor, base: torch.Tensor, gamma: torch.Tensor | None, *, iters: int = 20,
           hc_eps: float = 1e-6, norm_eps: float = 1e-6, head: bool = False, want_raw: bool = False):
    """h fp32 [M, hc, dim] -> (x bf16 [M, dim] = RMSNorm(mix(h)) * gamma, post [M, hc], comb [M, hc, hc]); with
    `head=True` only the mixed and normalised vector is produced. `want_raw` also returns the mix before the norm."""
    M, hc, dim = h.shape
    x = torch.empty(M, dim, device=h.device, dtype=torch.bfloat16)
    raw = torch.empty(M, dim, device=h.device, dtype=torch.float32) if want_raw else None
    post = comb = None
    if not head:
        post = torch.empty(M, hc, device=h.device, dtype=torch.float32)
        comb = torch.empty(M, hc, hc, device=h.device, dtype=torch.float32)
    st = _lib.kernels().pk_dsv4_hc_pre(_ptr(h), _ptr(fn), _ptr(scale), _ptr(base), _ptr(gamma), c_int(M), c_int(dim), c_int(hc),
                                       c_int(iters), c_int(int(head)), c_float(hc_eps), c_float(norm_eps), _ptr(x), _ptr(raw),
                                       _ptr(post), _ptr(comb), _stream())
    _check(st, "pk_dsv4_hc_pre")
    if head:
        return (x, raw) if want_raw else x
    return (x, post, comb, raw) if want_raw else (x, post, comb)


def hc_post(y: torch.Tensor, h: torch.Tensor, post: torch.Tensor, comb: torch.Tensor, y2: torch.Tensor | None = None,
            out: torch.Tensor | None = None) -> torch.Tensor:
    """h'[m, j] = post[m, j] * (y + y2)[m] + sum_i comb[m, i, j] * h[m, i]; y, y2 fp32 [M, dim]."""
    M, hc, dim = h.shape
    out = torch.empty_like(h) if out is None else out
    st = _lib.kernels().pk_dsv4_hc_post(_ptr(y), _ptr(y2), _ptr(h), _ptr(post), _ptr(comb), c_int(M), c_int(dim), c_int(hc),
                                        _ptr(out), _stream())
    _check(st, "pk_dsv4_hc_post")
    return out


def head_prep(x: torch.Tensor, pos: torch.Tensor, cos_t: torch.Tensor, sin_t: torch.Tensor, rd: int, flags: int, eps: float = 1e-6) -> torch.Tensor:
    """In place on bf16 [M, H, hd]: per-head RMS scaling / RoPE / inverse RoPE / Hadamard + FP4 fake quant."""
    M, H, hd = x.shape
    st = _lib.kernels().pk_dsv4_head_prep(_ptr(x), _ptr(pos), _ptr(cos_t), _ptr(sin_t), c_int(M), c_int(H), c_int(hd), c_int(rd),
                                          c_int(flags), c_float(eps), _stream())
    _check(st, "pk_dsv4_head_prep")
    return x


def kv_prep(kv: torch.Tensor, gamma: torch.Tensor, pos: torch.Tensor, cos_t: torch.Tensor, sin_t: torch.Tensor, rd: int, ring: int,
            dst: torch.Tensor, eps: float = 1e-6, dst_rows: torch.Tensor | None = None) -> None:
    """fp32 [M, hd] projections -> normalised, rotated (at `pos`), FP8-fake-quantised bf16 rows at `dst[pos % ring]`, or at
    `dst[dst_rows]` when given."""
    M, hd = kv.shape
    st = _lib.kernels().pk_dsv4_kv_prep_rows(_ptr(kv), _ptr(gamma), _ptr(pos), _ptr(dst_rows), _ptr(cos_t), _ptr(sin_t), c_int(M), c_int(hd),
                                             c_int(rd), c_int(ring), c_float(eps), _ptr(dst), _stream())
    _check(st, "pk_dsv4_kv_prep")


def compress(proj: torch.Tensor, ape: torch.Tensor, ring: torch.Tensor, gamma: torch.Tensor, cos_t: torch.Tensor, sin_t: torch.Tensor,
             pos0: int, ratio: int, cd: int, rd: int, rotate: bool, dst: torch.Tensor, eps: float = 1e-6) -> None:
    """Gated pooling over the rows of this call (positions pos0..) and the remembered earlier rows; completed
    entries go to `dst[c]`. `proj` fp32 [M, 2*C]: kv then score projections; `ring` fp32 [2, slots, C]."""
    M = proj.shape[0]
    st = _lib.kernels().pk_dsv4_compress(_ptr(proj), _ptr(ape), _ptr(ring), _ptr(gamma), _ptr(cos_t), _ptr(sin_t), c_int(pos0), c_int(M),
                                         c_int(ratio), c_int(cd), c_int(int(ratio == 4)), c_int(ring.shape[1]), c_int(rd), c_int(int(rotate)), c_float(eps),
                                         _ptr(dst), _stream())
    _check(st, "pk_dsv4_compress")


def index_score(q: torch.Tensor, k: torch.Tensor, w: torch.Tensor, pos: torch.Tensor, ratio: int, ld: int, wscale: float) -> torch.Tensor:
    M, ih, _ = q.shape
    score = torch.empty(M, ld, device=q.device, dtype=torch.float32)
    st = _lib.kernels().pk_dsv4_index_score(_ptr(q), _ptr(k), _ptr(w), _ptr(pos), c_int(M), c_int(ih), c_int(ratio), c_int(ld),
                                            c_int(w.stride(0)), c_float(wscale), _ptr(score), _stream())
    _check(st, "pk_dsv4_index_score")
    return score


def topk_select(score: torch.Tensor, k: int, lengths: torch.Tensor | None = None) -> torch.Tensor:
    """Indices (int32 [M, k], ascending index order, -1 padded) of the k largest entries of every row of fp32 `score`
    [M, n]; `lengths` [M] limits each row to its first entries; -inf scores are never selected; among equal scores the
    lowest indices win. A device radix select (five streaming passes) instead of a sort of the row."""
    if score.dtype != torch.float32 or score.dim() != 2 or score.stride(1) != 1:
        raise ValueError("topk_select takes a 2-D fp32 tensor with contiguous rows")
    M, n = score.shape
    out = torch.empty(M, k, device=score.device, dtype=torch.int32)
    st = _lib.kernels().pk_topk_select(_ptr(score), _ptr(lengths), c_int(M), c_int(n), c_int(score.stride(0)), c_int(k), _ptr(out), _stream())
    _check(st, "pk_topk_select")
    return out


def sparse_attn(q: torch.Tensor, kv: torch.Tensor, pos: torch.Tensor, sink: torch.Tensor, cos_t: torch.Tensor, sin_t: torch.Tensor, *,
                win: int, ring: int, ratio: int, rd: int, sel: torch.Tensor | None = None, all_entries: bool = False,
                rope_pos: torch.Tensor | None = None) -> torch.Tensor:
    """Sink-softmax attention of bf16 q [M, H, hd] over window rows and compressed rows of `kv` (K == V);
    the output has the inverse RoPE applied (at `rope_pos` when given, else at `pos`)."""
    M, H, hd = q.shape
    out = torch.empty_like(q)
    mode = 2 if sel is not None else 1 if all_entries else 0
    ksel = 0 if sel is None else sel.shape[1]
    st = _lib.kernels().pk_dsv4_sparse_attn_ex(_ptr(q), _ptr(kv), _ptr(pos), _ptr(rope_pos), _ptr(sel), _ptr(sink), _ptr(cos_t), _ptr(sin_t), c_int(M),
                                            c_int(H), c_int(hd), c_int(win), c_int(ring), c_int(max(ratio, 1)), c_int(mode), c_int(ksel),
                                            c_int(rd), c_float(hd ** -0.5), _ptr(out), _stream())
    _check(st, "pk_dsv4_sparse_attn")
    return out


def hash_route(x: torch.Tensor, gate_w: torch.Tensor, tid2eid: torch.Tensor, tokens: torch.Tensor, score_func: str, route_scale: float):
    T, H = x.shape
    topk = tid2eid.shape[1]
    ids = torch.empty(T, topk, device=x.device, dtype=torch.int32)
    w = torch.empty(T, topk, device=x.device, dtype=torch.float32)
    st = _lib.kernels().pk_dsv4_hash_route(_ptr(x), _ptr(gate_w), _ptr(tid2eid), _ptr(tokens), c_int(T), c_int(H), c_int(topk),
                                           c_int({"sigmoid": 1, "sqrtsoftplus": 2}[score_func]), c_float(route_scale), _ptr(ids), _ptr(w),
                                           _stream())
    _check(st, "pk_dsv4_hash_route")
    return ids, w
