"""Python bindings of the hand-written sm_100a kernels (ctypes over `libpocket_kernels.so`).

Every function takes CUDA tensors, launches on the current torch stream and returns the
output tensor. There is one implementation per op and no fallback: a missing library or
a non-zero status raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_size_t, c_uint64, c_void_p

import torch

from . import lib as _lib

__all__ = [
    "matvec", "gemm_umma", "gemm_bf16", "deltanet_seq", "deltanet_chunked", "qk_norm_rope_append", "gqa_decode", "rmsnorm",
    "embedding", "argmax", "silu_mul", "KernelError",
]

WFMT_FP8_BLOCK128 = 0
WFMT_BF16 = 1
EPI_BF16, EPI_SWIGLU, EPI_RESID, EPI_F32 = 0, 1, 2, 3


class KernelError(RuntimeError):
    pass


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(status: int, what: str) -> None:
    if status != 0:
        err = _lib.kernels().pk_last_cuda_error()
        raise KernelError(f"{what}: status {status} (cuda error {err})")


def _sm_count() -> int:
    return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count


def matvec(x: torch.Tensor, w_fp8: torch.Tensor | None, scale: torch.Tensor | None, w_bf16: torch.Tensor | None = None,
           *, gamma: torch.Tensor | None = None, norm_mode: int = 1, eps: float = 1e-6, parts: torch.Tensor | None = None,
           hidden_out: torch.Tensor | None = None, epi: int = 0) -> torch.Tensor:
    """Small-batch linear (1..8 rows): y = norm(x + sum(parts)) @ [w_fp8 * scale ; w_bf16]^T.

    epi 0 -> bf16, 1 -> SiLU(gate) * up (rows of w_fp8: gate then up), 2 -> fp32.
    """
    M, K = x.shape
    N = 0 if w_fp8 is None else w_fp8.shape[0]
    Nb = 0 if w_bf16 is None else w_bf16.shape[0]
    ncols = N // 2 if epi == 1 else N + Nb
    y = torch.empty(M, ncols, device=x.device, dtype=torch.float32 if epi == 2 else torch.bfloat16)
    nparts = 0 if parts is None else parts.shape[0]
    st = _lib.kernels().pk_matvec(
        _ptr(w_fp8), _ptr(scale), _ptr(w_bf16), c_int(N), c_int(Nb), c_int(K), c_int(M), _ptr(x), _ptr(parts),
        c_int(nparts), _ptr(hidden_out), _ptr(gamma), c_int(norm_mode), c_float(eps), c_void_p(0), c_int(epi),
        _ptr(y), c_int(ncols), c_void_p(0), c_int(_sm_count()), _stream())
    _check(st, "pk_matvec")
    return y


def matvec_ring_status() -> int:
    """First bounded wait of the ring variant of `matvec` that ran out since the last call (0 = none)."""
    torch.cuda.synchronize()
    fn = _lib.kernels().pk_matvec_ring_status
    fn.restype = ctypes.c_uint
    return int(fn())


def gemm_umma(a: torch.Tensor, w: torch.Tensor, scale: torch.Tensor | None = None, *, epi: int = EPI_BF16,
              resid: torch.Tensor | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
    """tcgen05 GEMM: C = A @ dequant(W)^T with a fused epilogue. A bf16 [M, K]; W fp8 [N, K] with
    fp32 scales [N/128, K/128], or bf16 [N, K]."""
    M, K = a.shape
    N = w.shape[0]
    wfmt = WFMT_BF16 if w.dtype == torch.bfloat16 else WFMT_FP8_BLOCK128
    ncols = N // 2 if epi == EPI_SWIGLU else N
    c = torch.empty(M, ncols, device=a.device, dtype=torch.float32 if epi == EPI_F32 else torch.bfloat16)
    if status is None:
        status = torch.zeros(1, device=a.device, dtype=torch.int32)
    st = _lib.kernels().pk_gemm_umma(
        _ptr(a), c_int(a.stride(0)), _ptr(w), _ptr(scale), c_int(wfmt), c_int(M), c_int(N), c_int(K), c_int(epi),
        _ptr(c), _ptr(resid), c_int(ncols), _ptr(status), c_void_p(0), _stream())
    _check(st, "pk_gemm_umma")
    return c


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, *, epi: int = EPI_BF16, resid: torch.Tensor | None = None,
              status: torch.Tensor | None = None) -> torch.Tensor:
    """Persistent tcgen05 GEMM with 128x256 tiles and a double-buffered TMEM accumulator: C = A @ W^T, bf16 A [M, K] and W [N, K].
    Same epilogues as `gemm_umma`."""
    M, K = a.shape
    N = w.shape[0]
    ncols = N // 2 if epi == EPI_SWIGLU else N
    c = torch.empty(M, ncols, device=a.device, dtype=torch.float32 if epi == EPI_F32 else torch.bfloat16)
    if status is None:
        status = torch.zeros(1, device=a.device, dtype=torch.int32)
    st = _lib.kernels().pk_gemm_bf16(_ptr(a), c_int(a.stride(0)), _ptr(w), c_int(M), c_int(N), c_int(K), c_int(epi), _ptr(c), _ptr(resid),
                                     c_int(ncols), _ptr(status), c_void_p(0), c_int(_sm_count()), _stream())
    _check(st, "pk_gemm_bf16")
    return c


def quant_act_fp8(x: torch.Tensor, terms: int = 1) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 rows [M, K] -> (E4M3 codes uint8 [terms, m_pad, K], scales fp32 [K / 128, m_pad]); one scale (amax / 448) per
    row and 128-wide k block. With two terms the second plane holds the codes of the rounding residue of the first, so
    that (plane 0 + plane 1) * scale reproduces x to about 8 significant bits."""
    M, K = x.shape
    m_pad = (M + 127) // 128 * 128
    q = torch.zeros(terms, m_pad, K, device=x.device, dtype=torch.uint8)
    sc = torch.ones(K // 128, m_pad, device=x.device, dtype=torch.float32)
    st = _lib.kernels().pk_quant_act_fp8(_ptr(x), c_int(x.stride(0)), c_int(M), c_int(K), c_int(terms), _ptr(q), c_int(m_pad), _ptr(sc),
                                         c_int(m_pad), _stream())
    _check(st, "pk_quant_act_fp8")
    return q, sc


def gemm_fp8(aq: torch.Tensor, a_scale: torch.Tensor, M: int, w: torch.Tensor, w_scale: torch.Tensor, *, epi: int = EPI_BF16,
             resid: torch.Tensor | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
    """Persistent tcgen05 kind::f8f6f4 GEMM: C = A @ W^T with A from `quant_act_fp8` (one or two E4M3 terms) and W as raw
    E4M3 codes [N, K] with fp32 scales per 128 x 128 block; every k block is scaled and added in fp32. Epilogues as in
    `gemm_bf16`."""
    terms, m_pad, K = aq.shape
    N = w.shape[0]
    ncols = N // 2 if epi == EPI_SWIGLU else N
    c = torch.empty(M, ncols, device=aq.device, dtype=torch.float32 if epi == EPI_F32 else torch.bfloat16)
    if status is None:
        status = torch.zeros(1, device=aq.device, dtype=torch.int32)
    st = _lib.kernels().pk_gemm_fp8(_ptr(aq), c_int(terms), c_int(m_pad), _ptr(a_scale), c_int(a_scale.stride(0)), _ptr(w), _ptr(w_scale),
                                    c_int(M), c_int(N), c_int(K), c_int(epi), _ptr(c), _ptr(resid), c_int(ncols), _ptr(status), c_void_p(0),
                                    c_int(_sm_count()), _stream())
    _check(st, "pk_gemm_fp8")
    return c


def deltanet_seq(proj: torch.Tensor, key_heads: int, value_heads: int, conv_w: torch.Tensor, conv_state: torch.Tensor,
                 A_log: torch.Tensor, dt_bias: torch.Tensor, norm_w: torch.Tensor, eps: float, state: torch.Tensor) -> torch.Tensor:
    """Gated DeltaNet over T tokens in order; updates `state` and `conv_state` in place."""
    T, ld = proj.shape
    out = torch.empty(T, value_heads * 128, device=proj.device, dtype=torch.bfloat16)
    st = _lib.kernels().pk_deltanet_seq(
        _ptr(proj), c_int(ld), c_int(T), c_int(key_heads), c_int(value_heads), c_int(128), c_int(128), _ptr(conv_w),
        _ptr(conv_state), _ptr(A_log), _ptr(dt_bias), _ptr(norm_w), c_float(eps), _ptr(state), _ptr(out), _stream())
    _check(st, "pk_deltanet_seq")
    return out


def deltanet_chunked(proj: torch.Tensor, key_heads: int, value_heads: int, conv_w: torch.Tensor, conv_state: torch.Tensor,
                     A_log: torch.Tensor, dt_bias: torch.Tensor, norm_w: torch.Tensor, eps: float, state: torch.Tensor) -> torch.Tensor:
    """Chunk-parallel (chunk 64) form of `deltanet_seq`: same inputs, outputs and state updates."""
    T, ld = proj.shape
    K = _lib.kernels()
    K.pk_deltanet_chunk_workspace.restype = c_size_t
    nws = K.pk_deltanet_chunk_workspace(c_int(T), c_int(key_heads), c_int(value_heads))
    ws = torch.empty(nws, device=proj.device, dtype=torch.float32)
    out = torch.empty(T, value_heads * 128, device=proj.device, dtype=torch.bfloat16)
    st = K.pk_deltanet_chunked(
        _ptr(proj), c_int(ld), c_int(T), c_int(key_heads), c_int(value_heads), c_int(128), c_int(128), _ptr(conv_w),
        _ptr(conv_state), _ptr(A_log), _ptr(dt_bias), _ptr(norm_w), c_float(eps), _ptr(state), _ptr(out), _ptr(ws), _stream())
    _check(st, "pk_deltanet_chunked")
    return out


def qk_norm_rope_append(proj: torch.Tensor, Hq: int, Hkv: int, pos: torch.Tensor, q_gamma: torch.Tensor,
                        k_gamma: torch.Tensor, eps: float, rotary_dim: int, theta: float, kcache: torch.Tensor,
                        vcache: torch.Tensor, kscale: torch.Tensor | None = None, vscale: torch.Tensor | None = None) -> torch.Tensor:
    """`kscale` / `vscale` (fp32 [Hkv, ctx, 2]) select the FP8 KV cache: `kcache` / `vcache` are then uint8 E4M3 codes
    [Hkv, ctx, 128] with one scale per 64 channels (amax / 448)."""
    M, ld = proj.shape
    q = torch.empty(M, Hq, 128, device=proj.device, dtype=torch.bfloat16)
    st = _lib.kernels().pk_qk_norm_rope_append_kv(
        _ptr(proj), c_int(ld), c_int(M), c_int(Hq), c_int(Hkv), c_int(128), _ptr(pos), _ptr(q_gamma), _ptr(k_gamma),
        c_float(eps), c_int(rotary_dim), c_float(theta), _ptr(q), _ptr(kcache), _ptr(vcache), _ptr(kscale), _ptr(vscale),
        c_int(kcache.shape[1]), _stream())
    _check(st, "pk_qk_norm_rope_append_kv")
    return q


def gqa_decode(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, pos: torch.Tensor, *, nsplit: int = 4,
               gate_proj: torch.Tensor | None = None, window: int = 0, sink: int = 0, kscale: torch.Tensor | None = None,
               vscale: torch.Tensor | None = None) -> torch.Tensor:
    """Split-context GQA attention of M query rows [M, Hq, 128] at positions `pos` over the position-indexed caches.
    Every row is worked by the same code path, split boundaries and summation order as a single-row call at its position,
    so the M rows of a speculative verify equal M successive decode steps bit for bit (the role of the reference's
    exact-order verify kernels, cpp_engine/cuda/qwen_gqa_optimized.cu:567-716)."""
    M, Hq, D = q.shape
    Hkv, cap, _ = kcache.shape
    ws = torch.empty(M * Hq * nsplit * (D + 2), device=q.device, dtype=torch.float32)
    out = torch.empty(M, Hq * D, device=q.device, dtype=torch.bfloat16)
    ld = 0 if gate_proj is None else gate_proj.stride(0)
    st = _lib.kernels().pk_gqa_decode_kv(
        _ptr(q), _ptr(kcache), _ptr(vcache), _ptr(kscale), _ptr(vscale), _ptr(pos), c_int(M), c_int(Hq), c_int(Hkv), c_int(D), c_int(cap),
        c_float(D ** -0.5), c_int(nsplit), c_int(window), c_int(sink), _ptr(ws), _ptr(gate_proj), c_int(ld), _ptr(out),
        _stream())
    _check(st, "pk_gqa_decode_kv")
    return out


def gqa_prefill(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, pos: torch.Tensor, *, gate_proj: torch.Tensor | None = None,
                status: torch.Tensor | None = None) -> torch.Tensor:
    """Causal GQA attention of a prefill chunk on the tensor cores (tcgen05: S = Q K^T and P V per 128 x 128 tile, online
    softmax in between): q bf16 [M, Hq, 128] at consecutive positions `pos`, bf16 caches [Hkv, cap, 128] that already hold
    the chunk's rows. Same output as `gqa_decode` over the same rows."""
    M, Hq, D = q.shape
    Hkv, cap, _ = kcache.shape
    out = torch.empty(M, Hq * D, device=q.device, dtype=torch.bfloat16)
    if status is None:
        status = torch.zeros(1, device=q.device, dtype=torch.int32)
    ld = 0 if gate_proj is None else gate_proj.stride(0)
    st = _lib.kernels().pk_gqa_prefill_umma(_ptr(q), _ptr(kcache), _ptr(vcache), _ptr(pos), c_int(M), c_int(Hq), c_int(Hkv), c_int(D), c_int(cap),
                                            c_float(D ** -0.5), _ptr(gate_proj), c_int(ld), _ptr(out), _ptr(status), _stream())
    _check(st, "pk_gqa_prefill_umma")
    return out


def full_qk_norm_rope_append(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pos: torch.Tensor, q_gamma: torch.Tensor, k_gamma: torch.Tensor,
                             cos_t: torch.Tensor, sin_t: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, *, n_heads: int, n_kv_heads: int,
                             rope_dim: int, eps: float = 1e-6) -> torch.Tensor:
    """bf16 projections q [T, Hq * 128], k / v [T, Hkv * 128] (rows may be strided views of one fused projection) -> RMS over the whole vector with per-element gamma, half-split
    rotation at `pos` (tables [ctx, rope_dim / 2]), k and v written to the caches [Hkv, ctx, 128]; returns bf16 q [T, Hq, 128]."""
    T = q.shape[0]
    out = torch.empty(T, n_heads, 128, device=q.device, dtype=torch.bfloat16)
    st = _lib.kernels().pk_full_qk_norm_rope_append(
        _ptr(q), c_int(q.stride(0)), _ptr(k), c_int(k.stride(0)), _ptr(v), c_int(v.stride(0)), c_int(T), c_int(n_heads), c_int(n_kv_heads),
        c_int(128), _ptr(pos), _ptr(q_gamma), _ptr(k_gamma),
        c_float(eps), c_int(rope_dim), _ptr(cos_t), _ptr(sin_t), _ptr(out), _ptr(kcache), _ptr(vcache), c_int(kcache.shape[1]), _stream())
    _check(st, "pk_full_qk_norm_rope_append")
    return out


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, *, mode: int = 1, eps: float = 1e-6, parts: torch.Tensor | None = None,
            hidden_out: torch.Tensor | None = None) -> torch.Tensor:
    """RMSNorm of bf16 x [M, K] (mode 1: times 1 + gamma, mode 2: times gamma). With `parts` (fp32 [R, M, K]) the input is
    bf16(x + sum of parts), which is also written to `hidden_out` when given: a residual add fused into the norm."""
    M, K = x.shape
    y = torch.empty_like(x)
    st = _lib.kernels().pk_rmsnorm(_ptr(x), _ptr(parts), c_int(0 if parts is None else parts.shape[0]), c_int(M), c_int(K), _ptr(hidden_out),
                                   _ptr(gamma), c_int(mode), c_float(eps), _ptr(y), c_void_p(0), _stream())
    _check(st, "pk_rmsnorm")
    return y


def rmsnorm_quant(x: torch.Tensor, gamma: torch.Tensor, *, mode: int = 1, eps: float = 1e-6, terms: int = 2):
    """RMSNorm of contiguous bf16 x [M, K] that also quantises its output rows for `gemm_fp8` in the same kernel:
    returns (y bf16 [M, K], codes uint8 [terms, m_pad, K], scales fp32 [K / 128, m_pad]), the codes and scales exactly
    those `quant_act_fp8(y, terms)` would give. K must be a multiple of 128."""
    M, K = x.shape
    if not x.is_contiguous() or x.dtype != torch.bfloat16:
        raise ValueError("rmsnorm_quant takes a contiguous bf16 matrix")
    m_pad = (M + 127) // 128 * 128
    y = torch.empty_like(x)
    q = torch.zeros(terms, m_pad, K, device=x.device, dtype=torch.uint8)
    sc = torch.ones(K // 128, m_pad, device=x.device, dtype=torch.float32)
    st = _lib.kernels().pk_rmsnorm_quant(_ptr(x), c_int(M), c_int(K), _ptr(gamma), c_int(mode), c_float(eps), _ptr(y), c_int(terms), _ptr(q),
                                         c_int(m_pad), _ptr(sc), c_int(m_pad), _stream())
    _check(st, "pk_rmsnorm_quant")
    return y, q, sc


def embedding(tokens: torch.Tensor, table: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    M = tokens.numel()
    out = torch.empty(M, table.shape[1], device=table.device, dtype=torch.bfloat16)
    st = _lib.kernels().pk_embedding(_ptr(tokens), c_int(M), _ptr(table), c_int(table.shape[1]), c_int(vocab_start),
                                     c_int(table.shape[0]), _ptr(out), c_void_p(0), _stream())
    _check(st, "pk_embedding")
    return out


def silu_mul(gate_up: torch.Tensor, limit: float = 0.0) -> torch.Tensor:
    M, two_inter = gate_up.shape
    out = torch.empty(M, two_inter // 2, device=gate_up.device, dtype=torch.bfloat16)
    st = _lib.kernels().pk_silu_mul(_ptr(gate_up), c_int(M), c_int(two_inter // 2), _ptr(out), c_float(limit), _stream())
    _check(st, "pk_silu_mul")
    return out


def argmax(logits: torch.Tensor, id_offset: int = 0) -> torch.Tensor:
    """Row argmax of fp32 logits with the lowest index winning ties."""
    M, n = logits.shape
    nb = 64
    cv = torch.empty(M * nb, device=logits.device, dtype=torch.float32)
    ci = torch.empty(M * nb, device=logits.device, dtype=torch.int32)
    ov = torch.empty(M, device=logits.device, dtype=torch.float32)
    oi = torch.empty(M, device=logits.device, dtype=torch.int32)
    st = _lib.kernels().pk_argmax(_ptr(logits), c_int(logits.stride(0)), c_int(M), c_int(n), c_int(id_offset), c_int(nb),
                                  _ptr(cv), _ptr(ci), _ptr(ov), _ptr(oi), _stream())
    _check(st, "pk_argmax")
    return oi
